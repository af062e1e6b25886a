"""Regenerates the golden vectors in this directory.  Run from the repository root, in a container
that holds the reference source tree (so that ``oracle/_ref`` can be built):

    python tests/golden/make_golden.py

The reference ships no golden vectors and its GPU backend cannot run here, so the vectors are
produced by the reference's own code compiled for the host by ``oracle/build.py`` into ``oracle/_ref``:
its CUDA kernel bodies (``TAB_GEMM.cu:25-247``, ``TAB_GEMM.cuh:73-115``: quantise, BTN_Weight, pad, im2row,
GEMM, looped over the reference's launch shapes) for every stage, cross-checked here against its CPU GEMM
functions (``TAB_CPU.cpp:242-328``).  The oracle is not used to produce any stored output.  Every file
stores its inputs, so the tests do not depend on any random generator reproducing them.

  gemm_<type>.npz      packed operands a, b (+btn) -> y straight out of the reference GEMM
  conv_cfg1_tnn.npz    the CPU-runnable headline case: N=1, 32x32x64 -> 64, 3x3, pad 1, stride 1, seed 0
  conv_small_<i>.npz   all four types (keys qw_/btn_/y_<type>) on ragged shapes (C not a multiple of 64, stride 2, no padding ...)
  quantize_edges.npz   values equal to +-threshold, +-0, NaN, +-inf, channel tails
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import build, c_oracle, tab_oracle as O  # noqa: E402
from util import make_input  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def main():
    build.build_oracle()
    if not build.build_ref() or not build.build_ref_cuda():
        raise SystemExit("the reference tree is not available: cannot regenerate golden vectors")
    import torch

    def ref_quantize(a, t, bw, n, h, w_, c):
        """Reference kernels; BTN_W of images beyond 16*(n//16), which its launch skips, from a second call on the tail
        padded to 16 images."""
        q, b = c_oracle.ref_cuda_quantize(a, t, bw, n, h, w_, c)
        done = 16 * (n // 16)
        if bw != 1 and done < n:
            tail = np.zeros((16, h, w_, c), np.float32)
            tt = np.zeros(16, np.float32)
            tail[:n - done], tt[:n - done] = a[done:], t[done:]
            b[done:] = c_oracle.ref_cuda_quantize(tail, tt, bw, 16, h, w_, c)[1][:n - done]
        return q, b

    def ref_conv(x_, qw_, ths_, btn_, t, geom):
        """ConvWithCuda_TAB on the reference's kernels, cross-checked against its CPU GEMM on the oracle's stages."""
        y_ = c_oracle.ref_cuda_conv2d(x_, qw_, ths_, btn_, t, *geom)
        assert np.array_equal(y_, c_oracle.conv2d(x_, qw_, ths_, btn_, t, *geom, use_ref_gemm=True))
        return y_

    # 1. raw GEMM vectors from the reference functions
    rng = np.random.default_rng(1234)
    for t, name in enumerate(["tnn", "tbn", "btn", "bnn"]):
        M, KN, K = 37, 19, 11
        ab, wb = O.act_bits(t), O.weight_bits(t)
        a = rng.integers(-2**63, 2**63 - 1, size=(M, K * ab), dtype=np.int64)
        b = rng.integers(-2**63, 2**63 - 1, size=(KN, K * wb), dtype=np.int64)
        if ab == 2:
            a[:, 0::2] &= a[:, 1::2]          # sign bits only where the magnitude bit is set
        if wb == 2:
            b[:, 0::2] &= b[:, 1::2]
        btn = (np.bitwise_count(b[:, 1::2].view(np.uint64)).sum(axis=1).astype(np.int32)
               if wb == 2 else np.zeros(KN, np.int32))
        y = c_oracle.gemm(a, b, btn, t, M, KN, K, K * 64, use_ref=True)
        assert np.array_equal(y.astype(np.float32), c_oracle.ref_cuda_gemm(a, b, btn, t, M, KN, K, K * 64))
        np.savez_compressed(os.path.join(OUT, "gemm_%s.npz" % name), a=a, b=b, btn=btn, y=y, type=t, K=K, NUM=K * 64)

    # 2. headline CPU-runnable configuration (seeded torch.randn as the configuration states)
    torch.manual_seed(0)
    N, H, W, C, KN, KH, KW = 1, 32, 32, 64, 64, 3, 3
    x = torch.randn(N, H, W, C).numpy()
    w = torch.randn(KN, KH, KW, C).numpy()
    ths = (np.float32(0.7) * np.abs(x).reshape(N, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
    wths = (np.float32(0.7) * np.abs(w).reshape(KN, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
    qw, btn = ref_quantize(w, wths, 2, KN, KH, KW, C)
    y = ref_conv(x, qw, ths, btn, 0, (1, 1, 1, 1, N, H, W, C, KN, KH, KW))
    np.savez_compressed(os.path.join(OUT, "conv_cfg1_tnn.npz"), x=x, ths=ths, w=w, wths=wths, qw=qw, btn=btn,
                        y=y.astype(np.int16), type=0, geom=np.array([1, 1, 1, 1, N, H, W, C, KN, KH, KW]))

    # 3. ragged small cases, all four types
    cases = [
        # p1 p2 s1 s2  N  H  W   C  KN KH KW
        (1, 1, 1, 1, 2, 9, 7, 65, 5, 3, 3),
        (0, 0, 2, 2, 3, 8, 10, 130, 7, 3, 3),
        (0, 0, 1, 1, 2, 6, 5, 200, 33, 1, 1),
        (2, 1, 2, 3, 1, 11, 13, 3, 4, 5, 3),
        (1, 1, 2, 2, 2, 14, 14, 128, 66, 3, 3),
    ]
    for ci, g in enumerate(cases):
        p1, p2, s1, s2, N, H, W, C, KN, KH, KW = g
        x, ths = make_input(100 + ci, N, H, W, C)
        w, wths = make_input(200 + ci, KN, KH, KW, C)
        rec = dict(x=x, ths=ths, w=w, wths=wths, geom=np.array(g))
        for t, name in enumerate(["tnn", "tbn", "btn", "bnn"]):
            qw, btn = ref_quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
            y = ref_conv(x, qw, ths, btn, t, g)
            rec["qw_" + name], rec["btn_" + name], rec["y_" + name] = qw, btn, y.astype(np.int16)
        np.savez_compressed(os.path.join(OUT, "conv_small_%d.npz" % ci), **rec)

    # 4. quantiser edge values through TerOnlyKernel / BinOnlyKernel / BTN_Weight (TAB_GEMM.cu:150-247)
    N, H, W, C = 3, 2, 3, 70
    x, _ = make_input(300, N, H, W, C)
    ths = np.array([0.5, 0.0, 1.25], dtype=np.float32)
    x[0, 0, 0, :8] = [0.5, -0.5, np.nextafter(np.float32(0.5), np.float32(1)), np.nextafter(np.float32(-0.5), np.float32(-1)),
                      0.0, -0.0, np.nan, np.inf]
    x[0, 0, 1, :4] = [-np.inf, 0.49999997, -0.49999997, 1e-38]
    x[1, 0, 0, :6] = [0.0, -0.0, 1e-45, -1e-45, np.nan, -np.inf]
    x[2, 1, 2, 64:70] = [1.25, -1.25, 1.2500001, -1.2500001, 3.0, -3.0]
    q2, b2 = ref_quantize(x, ths, 2, N, H, W, C)
    q1, b1 = ref_quantize(x, ths, 1, N, H, W, C)
    np.savez_compressed(os.path.join(OUT, "quantize_edges.npz"), x=x, ths=ths, q2=q2, btn2=b2, q1=q1, btn1=b1)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
