"""CPU oracle for TAB's ternary/binary quantise + popcount-convolution path (TEST INFRASTRUCTURE).

This module is a checker, not a product path: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import it.  It restates, in numpy, the algorithm of the reference's
CUDA backend (the behavioural authority for the API) with the integer arithmetic of the reference's
CPU GEMMs.  Every function cites the reference lines it follows.

Parity status: pinned.  The reference ships no tests, golden vectors or seeded outputs for this path,
so the oracle is pinned against outputs of the reference's own code run in the container that built
it: (a) every stage - quantise, BTN_Weight, pad, im2row, the four GEMMs and the whole
``ConvWithCuda_TAB`` sequence - against the reference's CUDA kernel bodies (``TAB_GEMM.cu:25-247``,
``TAB_GEMM.cuh:73-115``) compiled for the host and looped over their own launch shapes
(``oracle/_ref/libtab_ref_cuda.so``, built by ``build.py`` through ``ref_cuda_shim.cpp``), (b) the GEMMs
also against the reference's ``*GEMM_baseline`` functions compiled from ``TAB_CPU.cpp:242-328``, (c) the
committed golden vectors under ``tests/golden``, which that same reference code produced, (d) the
facts recorded in the reference's demo notebook (shapes, dtypes, "binary word == complement of ternary
magnitude word"), and (e) an independent float64 dense convolution of the de-quantised values.

Decisions where the reference's two backends disagree or are defective (each is followed here):
  * input layout is NHWC                                  (TAB_GEMM.cu:184,231; TAB_GPU.cpp:48)
  * one threshold per image / filter, ``ths[n]``           (TAB_GPU.cpp:23,49; TAB_CPU.cpp:67)
  * ternary: ``x > t`` -> +1, else ``x < -t`` -> -1, else 0   (TAB_GEMM.cu:184-192)
  * binary : bit = 1 (value -1) iff ``x < t``               (TAB_GEMM.cu:231)
  * channel c -> word c//64, bit c%64, LSB first; tail 0   (TAB_GEMM.cu:193-206,252-258)
  * QX is ``[N][H][W][PC][bits]``; plane 0 sign, 1 magnitude (TAB_GEMM.cu:196-197,321)
  * BTN_W[n] = popcount of the magnitude plane of n        (TAB_GEMM.cu:150-160)
  * padding words are zero: ternary pads with 0, binary activations pad with +1
                                                           (TAB_GEMM.cuh:73-89, TAB_CPU.cpp:39,155)
  * OH = (H + 2*p1 - KH + 1) // s1 (and likewise OW)       (TAB_GEMM.cu:354-357)
  * output is float32 with physical order [N][OH][OW][KN], relabelled to shape (N,KN,OH,OW)
                                                           (TAB_GEMM.cu:53,349,509,526)
"""
from __future__ import annotations

import numpy as np

CNTBITS = 64  # TAB_GEMM.cuh:10
TNN, TBN, BTN, BNN = 0, 1, 2, 3


def packed_channels(C: int) -> int:
    """PC = ceil(C / 64)  (TAB_GEMM.cu:262-265)."""
    return (C + CNTBITS - 1) // CNTBITS


def act_bits(conv_type: int) -> int:
    """Activation planes: types 2,3 use 1, types 0,1 use 2 (TAB_GEMM.cu:367-372)."""
    return 1 if conv_type in (BTN, BNN) else 2


def weight_bits(conv_type: int) -> int:
    """Weight planes: types 1,3 use 1, types 0,2 use 2 (TAB_GEMM.cu:374-379)."""
    return 1 if conv_type in (TBN, BNN) else 2


def out_size(H: int, W: int, KH: int, KW: int, p1: int, p2: int, s1: int, s2: int):
    """Reference output extent, C integer division (TAB_GEMM.cu:354-357)."""
    oh = (H + 2 * p1 - KH + 1) // s1
    ow = (W + 2 * p2 - KW + 1) // s2
    return max(oh, 0), max(ow, 0)


def _pack_bits(bits: np.ndarray) -> np.ndarray:
    """bool [..., C] -> int64 [..., PC]; channel c is bit c%64 of word c//64 (TAB_GEMM.cu:252-258)."""
    C = bits.shape[-1]
    pc = packed_channels(C)
    padded = np.zeros(bits.shape[:-1] + (pc * CNTBITS,), dtype=np.uint8)
    padded[..., :C] = bits
    by = np.packbits(padded, axis=-1, bitorder="little")           # [..., PC*8] bytes, LSB first
    words = by.reshape(bits.shape[:-1] + (pc, 8)).copy().view("<u8")[..., 0]
    return words.view(np.int64)


def quantize(x: np.ndarray, ths: np.ndarray, bitwidth: int, N: int, H: int, W: int, C: int):
    """TAB_Quantize: fp32 NHWC -> (QX int64 [N,H,W,PC,bits], BTN_W int32 [N]).

    Follows TerOnlyKernel (TAB_GEMM.cu:163-208), BinOnlyKernel (:211-247), BTN_Weight (:150-160)
    and QuanWithCuda_TAB (:250-322).  ``bitwidth == 1`` is binary, anything else ternary (:267,309).
    """
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(N, H, W, C)
    t = np.ascontiguousarray(ths, dtype=np.float32).reshape(N, 1, 1, 1)
    if bitwidth == 1:
        with np.errstate(invalid="ignore"):
            neg = x < t                                            # TAB_GEMM.cu:231
        qx = _pack_bits(neg)[..., None]                            # [N,H,W,PC,1]
        btn = np.zeros(N, dtype=np.int32)                          # TAB_GEMM.cu:283,314-317
        return np.ascontiguousarray(qx), btn
    with np.errstate(invalid="ignore"):
        pos = x > t                                                # TAB_GEMM.cu:184
        neg = (~pos) & (x < -t)                                    # TAB_GEMM.cu:188
    sign = _pack_bits(neg)                                         # plane 0 (bit1 in the reference)
    mag = _pack_bits(pos | neg)                                    # plane 1 (bit2 in the reference)
    qx = np.stack([sign, mag], axis=-1)                            # TAB_GEMM.cu:196-197
    btn = np.bitwise_count(mag.view(np.uint64)).reshape(N, -1).sum(axis=1).astype(np.int32)
    return np.ascontiguousarray(qx), btn


def pad_packed(q: np.ndarray, p1: int, p2: int) -> np.ndarray:
    """PadKernel (TAB_GEMM.cuh:73-89) with zero borders (TAB_CPU.cpp:39,155)."""
    if p1 == 0 and p2 == 0:
        return q
    N, H, W, Cp = q.shape
    out = np.zeros((N, H + 2 * p1, W + 2 * p2, Cp), dtype=q.dtype)
    out[:, p1:p1 + H, p2:p2 + W, :] = q
    return out


def im2row(q: np.ndarray, KH: int, KW: int, s1: int, s2: int) -> np.ndarray:
    """Img2RowKernel (TAB_GEMM.cuh:92-115; same as TAB_CPU.h:27-63 for 3x3).

    q is the padded packed tensor [N][PH][PW][C'] -> rows [N*OH*OW][KH*KW*C'], where output pixel
    (oh, ow) reads taps (oh*s1 + kh, ow*s2 + kw).
    """
    N, PH, PW, Cp = q.shape
    OH = max((PH - KH + 1) // s1, 0)
    OW = max((PW - KW + 1) // s2, 0)
    rows = np.empty((N, OH, OW, KH, KW, Cp), dtype=q.dtype)
    for kh in range(KH):
        for kw in range(KW):
            rows[:, :, :, kh, kw, :] = q[:, kh:kh + OH * s1:s1, kw:kw + OW * s2:s2, :][:, :OH, :OW]
    return rows.reshape(N * OH * OW, KH * KW * Cp)


def _popc(a: np.ndarray) -> np.ndarray:
    return np.bitwise_count(a.view(np.uint64)).astype(np.int64)


def gemm(a: np.ndarray, b: np.ndarray, btn: np.ndarray, conv_type: int, K: int, NUM: int,
         block: int = 256) -> np.ndarray:
    """The four popcount GEMMs (TAB_CPU.cpp:242-328, identical to TAB_GEMM.cu:25-147).

    a: int64 [M][K*ab] rows, b: int64 [KN][K*wb] rows, planes interleaved per word.  int32 [M][KN].
    """
    M = a.shape[0]
    KN = b.shape[0]
    y = np.empty((M, KN), dtype=np.int32)
    for m0 in range(0, M, block):
        am = a[m0:m0 + block]
        if conv_type == TNN:        # TAB_CPU.cpp:252-259
            sa, ma = am[:, None, 0::2], am[:, None, 1::2]
            sw, mw = b[None, :, 0::2], b[None, :, 1::2]
            p2 = ma & mw
            c1 = _popc(p2).sum(-1)
            c2 = _popc((sa ^ sw) & p2).sum(-1)
            y[m0:m0 + block] = c1 - 2 * c2
        elif conv_type == TBN:      # TAB_CPU.cpp:276-283
            sa, ma = am[:, None, 0::2], am[:, None, 1::2]
            bw = b[None, :, :]
            c1 = _popc(ma).sum(-1)
            c2 = _popc((sa ^ bw) & ma).sum(-1)
            y[m0:m0 + block] = c1 - 2 * c2
        elif conv_type == BTN:      # TAB_CPU.cpp:299-304
            ba = am[:, None, :]
            sw, mw = b[None, :, 0::2], b[None, :, 1::2]
            c2 = _popc((ba ^ sw) & mw).sum(-1)
            y[m0:m0 + block] = btn.astype(np.int64)[None, :] - 2 * c2
        elif conv_type == BNN:      # TAB_CPU.cpp:320-324
            c1 = _popc(am[:, None, :] ^ b[None, :, :]).sum(-1)
            y[m0:m0 + block] = NUM - 2 * c1
        else:
            raise ValueError("type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)")
    return y


def conv2d(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW) -> np.ndarray:
    """TAB_Conv2d: ConvWithCuda_TAB (TAB_GEMM.cu:325-527) as a CPU pipeline.

    quantise activations (:419-426) -> pad (:447-451) -> im2row (:482-488) -> GEMM (:509) -> float32
    buffer in [N][OH][OW][KN] order relabelled as shape (N, KN, OH, OW) (:526).
    """
    ab, wb = act_bits(conv_type), weight_bits(conv_type)
    PC = packed_channels(C)
    qx, _ = quantize(x, ths, 1 if ab == 1 else 2, N, H, W, C)
    q = pad_packed(qx.reshape(N, H, W, PC * ab), p1, p2)
    rows = im2row(q, KH, KW, s1, s2)
    qw = np.ascontiguousarray(qw, dtype=np.int64)
    if qw.size != KN * KH * KW * PC * wb:
        raise ValueError("QW has %d words, type %d needs %d" % (qw.size, conv_type, KN * KH * KW * PC * wb))
    b = qw.reshape(KN, KH * KW * PC * wb)
    OH, OW = out_size(H, W, KH, KW, p1, p2, s1, s2)
    y = gemm(rows, b, np.asarray(btn, dtype=np.int32).reshape(-1), conv_type, KH * KW * PC, KH * KW * C)
    return y.astype(np.float32).reshape(N, KN, OH, OW)


# ---------------------------------------------------------------------------------------------
# Independent second formulation (used by the tests to cross-check the oracle itself).
# ---------------------------------------------------------------------------------------------

def dequantize(qx: np.ndarray, C: int) -> np.ndarray:
    """Packed planes [..., PC, bits] -> float64 values [..., C] in {-1, 0, +1} / {-1, +1}."""
    bits = qx.shape[-1]
    u = np.ascontiguousarray(qx).view(np.uint64)
    shifts = np.arange(CNTBITS, dtype=np.uint64)

    def unpack(plane):
        b = (plane[..., None] >> shifts) & np.uint64(1)
        return b.reshape(plane.shape[:-1] + (-1,))[..., :C].astype(np.float64)

    if bits == 1:
        return 1.0 - 2.0 * unpack(u[..., 0])
    s, m = unpack(u[..., 0]), unpack(u[..., 1])
    return m * (1.0 - 2.0 * s)


def conv2d_dense(x, w_q, ths, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW) -> np.ndarray:
    """Dense float64 convolution of the de-quantised operands: sum a*w with the padding rule that
    zero words mean value 0 for ternary activations and +1 for binary activations.
    ``w_q`` is the already quantised weight tensor [KN,KH,KW,PC,wb]."""
    ab = act_bits(conv_type)
    qx, _ = quantize(x, ths, 1 if ab == 1 else 2, N, H, W, C)
    a = dequantize(qx, C)                                          # [N,H,W,C]
    w = dequantize(np.asarray(w_q).reshape(KN, KH, KW, packed_channels(C), -1), C)  # [KN,KH,KW,C]
    pad_val = 1.0 if ab == 1 else 0.0
    ap = np.full((N, H + 2 * p1, W + 2 * p2, C), pad_val)
    ap[:, p1:p1 + H, p2:p2 + W, :] = a
    OH, OW = out_size(H, W, KH, KW, p1, p2, s1, s2)
    y = np.zeros((N, OH, OW, KN))
    for kh in range(KH):
        for kw in range(KW):
            patch = ap[:, kh:kh + OH * s1:s1, kw:kw + OW * s2:s2, :][:, :OH, :OW]
            y += np.einsum("nhwc,kc->nhwk", patch, w[:, kh, kw, :])
    return y.astype(np.float32).reshape(N, KN, OH, OW)
