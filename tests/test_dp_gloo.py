"""Data-parallel shard/gather logic on two gloo ranks on the CPU, with the oracle standing in for the
device kernel: sharded == unsharded, bit for bit, for equal and ragged shards."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_oracle, tab_oracle as O
from util import make_input


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tab_b200 import dp
        from oracle.oracle_ops import torch_cpu_conv
        H, W, C, KN, K = 6, 5, 70, 9, 3
        x, ths = make_input(42, N, H, W, C)
        w, wths = make_input(43, KN, K, K, C)
        for t in range(4):
            qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
            full = dp.conv2d_data_parallel(torch_cpu_conv, torch.from_numpy(x), torch.from_numpy(qw), torch.from_numpy(ths),
                                           torch.from_numpy(btn), t, 1, 1, 1, 2, N, H, W, C, KN, K, K, world, rank)
            np.save(os.path.join(result_dir, "y_t%d_r%d.npy" % (t, rank)), full.numpy())
            if t == 0:
                # the gather alone, without the per-image size: every rank must take part in the agreeing all-reduce
                lo, hi = dp.shard_bounds(N, world, rank)
                per = full.numel() // N
                again = dp.gather_output(full.reshape(N, per)[lo:hi].contiguous(), N, world, rank)
                assert torch.equal(again, full)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run(N, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), N, str(tmp_path)), nprocs=world, join=True)
    H, W, C, KN, K = 6, 5, 70, 9, 3
    x, ths = make_input(42, N, H, W, C)
    w, wths = make_input(43, KN, K, K, C)
    for t in range(4):
        qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
        ref = c_oracle.conv2d(x, qw, ths, btn, t, 1, 1, 1, 2, N, H, W, C, KN, K, K).reshape(-1)
        for r in range(world):
            got = np.load(os.path.join(str(tmp_path), "y_t%d_r%d.npy" % (t, r)))
            assert got.shape == ref.shape and np.array_equal(got, ref), (t, r)


def test_equal_shards(tmp_path):
    _run(4, tmp_path)


def test_ragged_shards(tmp_path):
    _run(5, tmp_path)


def test_fewer_images_than_ranks(tmp_path):
    """N = 1 on two ranks: rank 1 holds nothing and still issues the same collectives as rank 0."""
    _run(1, tmp_path)
