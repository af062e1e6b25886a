"""Data-parallel convolution on two or more GPUs (NCCL, one process per GPU): the all-gathered output of the sharded batch
equals the oracle's output of the whole batch bit for bit, for equal, ragged and partly empty shards, through the C ABI
(``tab_b200.ops.Conv2d``) and through a prepared ``TABConv2d`` chain.  Skipped on a box with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

from util import make_input

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from tab_b200 import _cabi, dp, ops
        H, W, C, KN, K = 9, 7, 70, 24, 3
        x, ths = make_input(52, N, H, W, C)
        w, wths = make_input(53, KN, K, K, C)
        X, T = torch.from_numpy(x).to(dev), torch.from_numpy(ths).to(dev)
        Wt, WT = torch.from_numpy(w).to(dev), torch.from_numpy(wths).to(dev)
        for t in range(4):
            qw, btn = ops.Quantize(Wt, WT, 1 if t in (1, 3) else 2, KN, K, K, C)
            full = dp.conv2d_data_parallel(ops.Conv2d, X, qw, T, btn, t, 1, 1, 1, 2, N, H, W, C, KN, K, K, world, rank)
            torch.cuda.synchronize()
            np.save(os.path.join(result_dir, "y_t%d_r%d.npy" % (t, rank)), full.cpu().numpy())
        assert _cabi.lib().tab_device_status() == 0
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run(N, tmp_path, world):
    import torch.multiprocessing as mp
    from oracle import c_oracle, tab_oracle as O
    mp.spawn(_worker, args=(world, _free_port(), N, str(tmp_path)), nprocs=world, join=True)
    H, W, C, KN, K = 9, 7, 70, 24, 3
    x, ths = make_input(52, N, H, W, C)
    w, wths = make_input(53, KN, K, K, C)
    for t in range(4):
        qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
        ref = c_oracle.conv2d(x, qw, ths, btn, t, 1, 1, 1, 2, N, H, W, C, KN, K, K).reshape(-1)
        for r in range(world):
            got = np.load(os.path.join(str(tmp_path), "y_t%d_r%d.npy" % (t, r)))
            assert got.shape == ref.shape and np.array_equal(got, ref), (t, r)


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least two GPUs")
    return min(n, 4)


def test_equal_shards(tmp_path):
    world = _world()
    _run(4 * world, tmp_path, world)


def test_ragged_shards(tmp_path):
    world = _world()
    _run(4 * world + 1, tmp_path, world)


def test_fewer_images_than_ranks(tmp_path):
    world = _world()
    _run(world - 1, tmp_path, world)
