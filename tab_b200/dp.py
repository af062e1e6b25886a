"""Data-parallel execution over the batch dimension: one process per GPU, every image independent.

The path shards naturally: thresholds are per image, quantisation is per pixel and the convolution is
per output pixel, and N is the outermost dimension of both the input and the output buffer.  Each rank
owns a contiguous slice of images, holds a full replica of the (small) quantised weights, runs its
slice with no communication, and the outputs are gathered once with a single all-gather.  The
reference has no multi-device code; this module adds nothing to the arithmetic.

The functions take the process group and the operators as arguments, so the same code runs on NCCL
with the device operators and, in the CPU tests, on gloo with stand-in operators.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_bounds(N: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of N images: the first N % world ranks hold one image more."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank %d/%d" % (world, rank))
    base, rem = divmod(N, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_batch(x: torch.Tensor, ths: torch.Tensor, N: int, world: int, rank: int):
    """Views of this rank's images of ``x`` (N*... elements, N outermost) and thresholds."""
    lo, hi = shard_bounds(N, world, rank)
    per = x.numel() // N if N else 0
    return x.reshape(-1)[lo * per:hi * per], ths.reshape(-1)[lo:hi], hi - lo


def gather_output(y_local: torch.Tensor, N: int, world: int, rank: int, group=None, per_image: int = None) -> torch.Tensor:
    """All-gather the per-rank output slices (N outermost, so each slice is one contiguous block) into the
    full ``[N, ...]`` buffer on every rank.  Equal shards use one ``all_gather_into_tensor``; ragged
    shards are padded to the largest shard for the collective and trimmed afterwards.

    ``per_image`` is the number of elements of one image's output.  Pass it whenever some rank may hold no image
    (N < world): such a rank cannot derive it from its empty slice.  When it is not passed, every rank takes part in
    one MAX all-reduce that agrees on it - every rank, so that the sequence of collectives is the same everywhere."""
    counts = [shard_bounds(N, world, r)[1] - shard_bounds(N, world, r)[0] for r in range(world)]
    n_local = counts[rank]
    flat = y_local.reshape(-1)
    if world == 1:
        return flat.clone()
    if per_image is None:
        per = flat.numel() // n_local if n_local else 0
        t = torch.tensor([per], dtype=torch.int64, device=y_local.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        per = int(t.item())
    else:
        per = int(per_image)
    if flat.numel() != n_local * per:
        raise ValueError("rank %d holds %d elements, expected %d images x %d" % (rank, flat.numel(), n_local, per))
    if len(set(counts)) == 1:
        out = torch.empty(N * per, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, flat.contiguous(), group=group)
        return out
    mx = max(counts)
    padded = torch.zeros(mx * per, dtype=y_local.dtype, device=y_local.device)
    padded[:flat.numel()] = flat
    buf = torch.empty(world * mx * per, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * mx * per: r * mx * per + counts[r] * per] for r in range(world)])


def conv2d_data_parallel(conv_fn, X, QW, thresholds, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                         world: int, rank: int, group=None, gather: bool = True):
    """``Conv2d`` on the global batch ``X`` ([N,H,W,C], present on every rank or at least this rank's
    slice valid): convolve this rank's images, then all-gather.  Returns the full output (flat,
    ``[N][OH][OW][KN]`` order) when ``gather`` else the local slice."""
    xs, ts, n_local = shard_batch(X, thresholds, N, world, rank)
    y_local = conv_fn(xs, QW, ts, btn, conv_type, p1, p2, s1, s2, n_local, H, W, C, KN, KH, KW)
    if not gather:
        return y_local
    oh = max((H + 2 * p1 - KH + 1) // s1, 0)
    ow = max((W + 2 * p2 - KW + 1) // s2, 0)
    return gather_output(y_local, N, world, rank, group, per_image=oh * ow * KN)
