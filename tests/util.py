"""Shared helpers for the tests: seeded inputs in the shapes the reference's API takes."""
import numpy as np


def make_input(seed, N, H, W, C, scale=1.0):
    """fp32 NHWC N(0,1) data and per-n thresholds 0.7*mean|x|, both computed on the CPU in float32 so that
    the device path and the oracle see identical bits."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((N, H, W, C), dtype=np.float32) * np.float32(scale)).astype(np.float32)
    if x.size:
        ths = (np.float32(0.7) * np.abs(x).reshape(N, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
    else:
        ths = np.zeros(N, dtype=np.float32)
    return x, ths


def weight_bitwidth(conv_type):
    return 1 if conv_type in (1, 3) else 2
