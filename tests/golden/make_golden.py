"""Regenerates the golden vectors in this directory.  Run from the repository root, in a container
that holds the reference source tree (so that ``oracle/_ref`` can be built):

    python tests/golden/make_golden.py

The reference ships no golden vectors and its GPU backend cannot run here, so the vectors are
produced with the reference's own CPU GEMM functions (``TAB_CPU.cpp:242-328``, compiled by
``oracle/build.py`` into ``oracle/_ref``) running the GEMM stage, and with the oracle's restatement of
the stages the reference CPU file gets wrong for NHWC input (quantise, pad, im2row).  Every file
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
    if not build.build_ref():
        raise SystemExit("the reference tree is not available: cannot regenerate golden vectors")
    import torch

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
        np.savez_compressed(os.path.join(OUT, "gemm_%s.npz" % name), a=a, b=b, btn=btn, y=y, type=t, K=K, NUM=K * 64)

    # 2. headline CPU-runnable configuration (seeded torch.randn as the configuration states)
    torch.manual_seed(0)
    N, H, W, C, KN, KH, KW = 1, 32, 32, 64, 64, 3, 3
    x = torch.randn(N, H, W, C).numpy()
    w = torch.randn(KN, KH, KW, C).numpy()
    ths = (np.float32(0.7) * np.abs(x).reshape(N, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
    wths = (np.float32(0.7) * np.abs(w).reshape(KN, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
    qw, btn = O.quantize(w, wths, 2, KN, KH, KW, C)
    y = c_oracle.conv2d(x, qw, ths, btn, 0, 1, 1, 1, 1, N, H, W, C, KN, KH, KW, use_ref_gemm=True)
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
            qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
            y = c_oracle.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, use_ref_gemm=True)
            rec["qw_" + name], rec["btn_" + name], rec["y_" + name] = qw, btn, y.astype(np.int16)
        np.savez_compressed(os.path.join(OUT, "conv_small_%d.npz" % ci), **rec)

    # 4. quantiser edge values (encoding rules read from TAB_GEMM.cu:184-192,231)
    N, H, W, C = 3, 2, 3, 70
    x, _ = make_input(300, N, H, W, C)
    ths = np.array([0.5, 0.0, 1.25], dtype=np.float32)
    x[0, 0, 0, :8] = [0.5, -0.5, np.nextafter(np.float32(0.5), np.float32(1)), np.nextafter(np.float32(-0.5), np.float32(-1)),
                      0.0, -0.0, np.nan, np.inf]
    x[0, 0, 1, :4] = [-np.inf, 0.49999997, -0.49999997, 1e-38]
    x[1, 0, 0, :6] = [0.0, -0.0, 1e-45, -1e-45, np.nan, -np.inf]
    x[2, 1, 2, 64:70] = [1.25, -1.25, 1.2500001, -1.2500001, 3.0, -3.0]
    q2, b2 = O.quantize(x, ths, 2, N, H, W, C)
    q1, b1 = O.quantize(x, ths, 1, N, H, W, C)
    np.savez_compressed(os.path.join(OUT, "quantize_edges.npz"), x=x, ths=ths, q2=q2, btn2=b2, q1=q1, btn1=b1)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
