"""``Quantize`` / ``Conv2d`` on torch CUDA tensors, calling the C ABI through ctypes.

Argument order and meaning follow the reference binding (``TAB_GPU.cpp:34,53``); tensor checks follow
its ``CHECK_INPUT`` macro (``TAB_GPU.cpp:7-9``): every tensor argument must be a contiguous CUDA tensor
or a ``RuntimeError`` is raised.  Unlike the reference, dtypes are checked instead of converted (the
reference takes ``data_ptr()`` of a converted temporary, ``TAB_GEMM.cu:279,341``) and CUDA failures
raise instead of returning a partially written tensor (``TAB_GEMM.cu:292-321``).
"""
from __future__ import annotations

import torch

from . import _cabi


def _check_input(t: torch.Tensor, name: str, dtype: torch.dtype) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s" % (name, dtype))


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def conv_out_size(H, W, KH, KW, p1, p2, s1, s2):
    """OH, OW as the reference computes them (``TAB_GEMM.cu:354-357``), clamped at 0."""
    return max((H + 2 * p1 - KH + 1) // s1, 0), max((W + 2 * p2 - KW + 1) // s2, 0)


def Quantize(X, thresholds, bitwidth, N, H, W, C):
    """``TAB_Quantize`` (``TAB_GPU.cpp:53-58``): returns ``[QX, BTN_W]``.

    ``QX`` int64 ``{N,H,W,ceil(C/64),bits}``; ``BTN_W`` int32 ``{N}`` (zeros when ``bitwidth == 1``).
    """
    _check_input(X, "X", torch.float32)
    _check_input(thresholds, "thresholds", torch.float32)
    N, H, W, C, bitwidth = int(N), int(H), int(W), int(C), int(bitwidth)
    if min(N, H, W) < 0 or C < 1 or bitwidth < 1:
        raise RuntimeError("Quantize: sizes must be non-negative, C >= 1 and bitwidth >= 1")
    if X.numel() != N * H * W * C:
        raise RuntimeError("X has %d elements, expected N*H*W*C = %d" % (X.numel(), N * H * W * C))
    if thresholds.numel() != N:
        raise RuntimeError("thresholds has %d elements, expected N = %d" % (thresholds.numel(), N))
    bits = 1 if bitwidth == 1 else 2
    PC = (C + 63) // 64
    with torch.cuda.device(X.device):
        QX = torch.empty((N, H, W, PC, bits), dtype=torch.int64, device=X.device)
        BTN = torch.empty((N,), dtype=torch.int32, device=X.device)
        rc = _cabi.lib().tab_quantize_launch(X.data_ptr(), thresholds.data_ptr(), QX.data_ptr(), BTN.data_ptr(),
                                             bitwidth, N, H, W, C, _stream_ptr(X.device))
    _cabi.check(rc, "tab_quantize_launch")
    return [QX, BTN]


def _conv_checks(conv_type, QW, btn, N, H, W, C, KN, KH, KW, p1, p2, s1, s2):
    if conv_type not in (0, 1, 2, 3):
        raise RuntimeError("type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)")
    if min(N, H, W, KN) < 0 or C < 1 or KH < 1 or KW < 1 or p1 < 0 or p2 < 0 or s1 < 1 or s2 < 1:
        raise RuntimeError("Conv2d: invalid size, padding or stride")
    wb = 1 if conv_type in (1, 3) else 2
    need = KN * KH * KW * ((C + 63) // 64) * wb
    if QW.numel() != need:
        raise RuntimeError("QW has %d words, type %d needs KN*KH*KW*ceil(C/64)*%d = %d "
                           "(quantise the weights at bitwidth %d)" % (QW.numel(), conv_type, wb, need, wb))
    if conv_type == 2 and btn.numel() != KN:
        raise RuntimeError("btn has %d elements, expected KN = %d" % (btn.numel(), KN))


def Conv2d(X, QW, thresholds, btn, type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW):
    """``TAB_Conv2d`` (``TAB_GPU.cpp:34-42``): float32 tensor of shape ``{N,KN,OH,OW}`` whose buffer is in
    ``[N][OH][OW][KN]`` order (``TAB_GEMM.cu:509,526``)."""
    _check_input(X, "X", torch.float32)
    _check_input(QW, "QW", torch.int64)
    _check_input(thresholds, "thresholds", torch.float32)
    _check_input(btn, "btn", torch.int32)
    conv_type = int(type)
    p1, p2, s1, s2 = int(padding1), int(padding2), int(stride1), int(stride2)
    N, H, W, C, KN, KH, KW = (int(v) for v in (N, H, W, C, KN, KH, KW))
    _conv_checks(conv_type, QW, btn, N, H, W, C, KN, KH, KW, p1, p2, s1, s2)
    if X.numel() != N * H * W * C:
        raise RuntimeError("X has %d elements, expected N*H*W*C = %d" % (X.numel(), N * H * W * C))
    if thresholds.numel() != N:
        raise RuntimeError("thresholds has %d elements, expected N = %d" % (thresholds.numel(), N))
    OH, OW = conv_out_size(H, W, KH, KW, p1, p2, s1, s2)
    l = _cabi.lib()
    with torch.cuda.device(X.device):
        Y = torch.empty((N, KN, OH, OW), dtype=torch.float32, device=X.device)
        ws_bytes = l.tab_conv2d_workspace_bytes(conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
        ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=X.device)
        rc = l.tab_conv2d_launch(X.data_ptr(), QW.data_ptr(), thresholds.data_ptr(), btn.data_ptr(), Y.data_ptr(),
                                 ws.data_ptr(), ws.numel(), conv_type, p1, p2, s1, s2,
                                 N, H, W, C, KN, KH, KW, _stream_ptr(X.device))
    _cabi.check(rc, "tab_conv2d_launch")
    return Y


def conv2d_packed(QX, QW, btn, type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW):
    """The GEMM stage alone on already packed activations (``GEMMWithCuda``, ``TAB_GEMM.cuh:22-66``, with
    the padding and im2row stages folded in)."""
    _check_input(QX, "QX", torch.int64)
    _check_input(QW, "QW", torch.int64)
    _check_input(btn, "btn", torch.int32)
    conv_type = int(type)
    p1, p2, s1, s2 = int(padding1), int(padding2), int(stride1), int(stride2)
    N, H, W, C, KN, KH, KW = (int(v) for v in (N, H, W, C, KN, KH, KW))
    _conv_checks(conv_type, QW, btn, N, H, W, C, KN, KH, KW, p1, p2, s1, s2)
    ab = 1 if conv_type in (2, 3) else 2
    if QX.numel() != N * H * W * ((C + 63) // 64) * ab:
        raise RuntimeError("QX has %d words, type %d needs %d" % (QX.numel(), conv_type, N * H * W * ((C + 63) // 64) * ab))
    OH, OW = conv_out_size(H, W, KH, KW, p1, p2, s1, s2)
    with torch.cuda.device(QX.device):
        Y = torch.empty((N, KN, OH, OW), dtype=torch.float32, device=QX.device)
        rc = _cabi.lib().tab_conv2d_packed_launch(QX.data_ptr(), QW.data_ptr(), btn.data_ptr(), Y.data_ptr(),
                                                  conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                                  _stream_ptr(QX.device))
    _cabi.check(rc, "tab_conv2d_packed_launch")
    return Y


# The reference's CPU module and README use these names for the same operators (TAB_CPU.cpp:637-638).
TAB_Quantize = Quantize
TAB_Conv2d = Conv2d


def residual_threshold(Y, residual=None, scale=0.7):
    """In place ``Y += residual`` (when given), then the per-image thresholds ``scale * mean|Y[n]|`` as a
    float32 CUDA tensor ``{N}`` - the ``thresholds`` argument of the next ``Conv2d``.  N is ``Y.shape[0]``.
    Not part of the reference's interface (its callers compute thresholds with framework ops)."""
    _check_input(Y, "Y", torch.float32)
    if residual is not None:
        _check_input(residual, "residual", torch.float32)
        if residual.numel() != Y.numel():
            raise RuntimeError("residual has %d elements, expected %d" % (residual.numel(), Y.numel()))
    N = int(Y.shape[0]) if Y.dim() > 0 else 1
    per_image = Y.numel() // N if N else 0
    with torch.cuda.device(Y.device):
        ths = torch.empty((N,), dtype=torch.float32, device=Y.device)
        sums = torch.empty((max(N, 1),), dtype=torch.float64, device=Y.device)
        rc = _cabi.lib().tab_residual_threshold_launch(Y.data_ptr(), residual.data_ptr() if residual is not None else None,
                                                       ths.data_ptr(), sums.data_ptr(), float(scale), N, per_image,
                                                       _stream_ptr(Y.device))
    _cabi.check(rc, "tab_residual_threshold_launch")
    return ths


# ---- stages of the tensor-core path, for callers that keep prepared weights -----------------------------------

def expand_weights(QW, bitwidth, KN, KH, KW, C):
    """Packed weights (``Quantize`` output) -> int8 ``{KN,KH,KW,Cp}`` holding {-1,0,+1}, ``Cp = 64*ceil(C/64)``."""
    _check_input(QW, "QW", torch.int64)
    Cp = (int(C) + 63) // 64 * 64
    bits = 1 if int(bitwidth) == 1 else 2
    if QW.numel() != KN * KH * KW * (Cp // 64) * bits:
        raise RuntimeError("QW has %d words, expected %d" % (QW.numel(), KN * KH * KW * (Cp // 64) * bits))
    with torch.cuda.device(QW.device):
        w8 = torch.empty((KN, KH, KW, Cp), dtype=torch.int8, device=QW.device)
        rc = _cabi.lib().tab_expand_weights_launch(QW.data_ptr(), w8.data_ptr(), bits, KN, KH, KW, C, _stream_ptr(QW.device))
    _cabi.check(rc, "tab_expand_weights_launch")
    return w8


def new_state(N, device):
    """Zeroed state block for ``conv2d_bits(..., threshold_scale=...)``; one block serves any number of calls that are
    ordered on a stream (every call leaves it zeroed)."""
    return torch.zeros((max(_cabi.lib().tab_conv2d_state_bytes(int(N)), 8),), dtype=torch.uint8, device=device)


def quantize_auto(X, scale, bitwidth, N, H, W, C, state=None):
    """``Quantize`` with the thresholds computed on the way: ``thresholds[n] = scale * mean|X[n]|``.  One launch (sums, a
    grid-wide meeting point, quantisation) where C is a multiple of 64, else the three launches it replaces.  Returns
    ``(QX, thresholds)``.  ``state``: a block from ``new_state(N, device)`` to reuse (zero before and after)."""
    _check_input(X, "X", torch.float32)
    N, H, W, C = int(N), int(H), int(W), int(C)
    if X.numel() != N * H * W * C:
        raise RuntimeError("X has %d elements, expected N*H*W*C = %d" % (X.numel(), N * H * W * C))
    bits = 1 if int(bitwidth) == 1 else 2
    with torch.cuda.device(X.device):
        if state is None:
            state = new_state(N, X.device)
        QX = torch.empty((N, H, W, (C + 63) // 64, bits), dtype=torch.int64, device=X.device)
        ths = torch.empty((N,), dtype=torch.float32, device=X.device)
        rc = _cabi.lib().tab_quantize_auto_launch(X.data_ptr(), float(scale), state.data_ptr(), ths.data_ptr(), QX.data_ptr(), int(bitwidth),
                                                  N, H, W, C, _stream_ptr(X.device))
    _cabi.check(rc, "tab_quantize_auto_launch")
    return QX, ths


def quantize_i16(X16, thresholds, bitwidth, N, H, W, C):
    """``Quantize`` on the compact int16 output of ``conv2d_bits(..., out_int16=True)``: returns ``QX`` only."""
    _check_input(X16, "X16", torch.int16)
    _check_input(thresholds, "thresholds", torch.float32)
    N, H, W, C = int(N), int(H), int(W), int(C)
    if X16.numel() != N * H * W * C or thresholds.numel() != N:
        raise RuntimeError("X16 / thresholds do not match N*H*W*C / N")
    bits = 1 if int(bitwidth) == 1 else 2
    with torch.cuda.device(X16.device):
        QX = torch.empty((N, H, W, (C + 63) // 64, bits), dtype=torch.int64, device=X16.device)
        rc = _cabi.lib().tab_quantize_i16_launch(X16.data_ptr(), thresholds.data_ptr(), QX.data_ptr(), int(bitwidth), N, H, W, C,
                                                 _stream_ptr(X16.device))
    _cabi.check(rc, "tab_quantize_i16_launch")
    return QX


def conv2d_bits(QX, W8, type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW,
                residual=None, threshold_scale=None, state=None, out_int16=False, next_bitwidth=None):
    """The GEMM stage on the tensor cores: activations as ``Quantize`` wrote them (bitwidth 2 for types 0,1; 1 for
    types 2,3), weights from ``expand_weights``.  Returns ``(Y, next_thresholds_or_None)``; ``Y = conv + residual``.
    ``threshold_scale`` needs ``state`` (``new_state``).  ``out_int16``: ``Y`` as int16 (no residual; the values are
    integers of magnitude at most KH*KW*C) for ``quantize_i16``.  ``next_bitwidth`` (needs ``threshold_scale``): the same
    launch also quantises ``Y`` against the next thresholds at that bitwidth and a third value is returned, ``QX`` of the
    next convolution (``[N,OH,OW,ceil(KN/64),bits]`` int64, what ``Quantize(Y, next_thresholds, ...)`` gives).
    Raises ``TabError`` (TAB_E_TOO_LARGE) for shapes the tensor-core kernel does not cover."""
    _check_input(QX, "QX", torch.int64)
    _check_input(W8, "W8", torch.int8)
    conv_type = int(type)
    p1, p2, s1, s2 = int(padding1), int(padding2), int(stride1), int(stride2)
    N, H, W, C, KN, KH, KW = (int(v) for v in (N, H, W, C, KN, KH, KW))
    PC = (C + 63) // 64
    ab = 1 if conv_type in (2, 3) else 2
    if QX.numel() != N * H * W * PC * ab:
        raise RuntimeError("QX has %d words, type %d needs %d" % (QX.numel(), conv_type, N * H * W * PC * ab))
    if W8.numel() != KN * KH * KW * PC * 64:
        raise RuntimeError("W8 has %d bytes, expected KN*KH*KW*Cp = %d" % (W8.numel(), KN * KH * KW * PC * 64))
    OH, OW = conv_out_size(H, W, KH, KW, p1, p2, s1, s2)
    if residual is not None:
        _check_input(residual, "residual", torch.float32)
        if residual.numel() != N * KN * OH * OW:
            raise RuntimeError("residual has %d elements, expected %d" % (residual.numel(), N * KN * OH * OW))
    if threshold_scale is not None and state is None:
        raise RuntimeError("threshold_scale needs a state block (new_state)")
    if out_int16 and residual is not None:
        raise RuntimeError("out_int16 cannot be combined with a residual")
    if next_bitwidth is not None and threshold_scale is None:
        raise RuntimeError("next_bitwidth needs threshold_scale (the thresholds the result is quantised against)")
    with torch.cuda.device(QX.device):
        Y = torch.empty((N, KN, OH, OW), dtype=torch.int16 if out_int16 else torch.float32, device=QX.device)
        nxt = torch.empty((N,), dtype=torch.float32, device=QX.device) if threshold_scale is not None else None
        if next_bitwidth is not None:
            nb = 1 if int(next_bitwidth) == 1 else 2
            QN = torch.empty((N, OH, OW, (KN + 63) // 64, nb), dtype=torch.int64, device=QX.device)
            rc = _cabi.lib().tab_conv2d_bits_next_launch(QX.data_ptr(), W8.data_ptr(), Y.data_ptr(), 1 if out_int16 else 0, conv_type,
                                                         p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                                         residual.data_ptr() if residual is not None else None,
                                                         state.data_ptr(), nxt.data_ptr(), float(threshold_scale),
                                                         QN.data_ptr(), nb, _stream_ptr(QX.device))
            _cabi.check(rc, "tab_conv2d_bits_next_launch")
            return Y, nxt, QN
        if out_int16:
            rc = _cabi.lib().tab_conv2d_bits_i16_launch(QX.data_ptr(), W8.data_ptr(), Y.data_ptr(), conv_type, p1, p2, s1, s2,
                                                        N, H, W, C, KN, KH, KW,
                                                        state.data_ptr() if nxt is not None else None,
                                                        nxt.data_ptr() if nxt is not None else None,
                                                        float(threshold_scale) if threshold_scale is not None else 0.0,
                                                        _stream_ptr(QX.device))
            _cabi.check(rc, "tab_conv2d_bits_i16_launch")
            return Y, nxt
        rc = _cabi.lib().tab_conv2d_bits_launch(QX.data_ptr(), W8.data_ptr(), Y.data_ptr(), conv_type, p1, p2, s1, s2,
                                                N, H, W, C, KN, KH, KW,
                                                residual.data_ptr() if residual is not None else None,
                                                state.data_ptr() if nxt is not None else None,
                                                nxt.data_ptr() if nxt is not None else None,
                                                float(threshold_scale) if threshold_scale is not None else 0.0,
                                                _stream_ptr(QX.device))
    _cabi.check(rc, "tab_conv2d_bits_launch")
    return Y, nxt


def Conv2dFused(X, QW, thresholds, btn, type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW,
                residual=None, threshold_scale=None):
    """``Conv2d`` with the chaining fusions of ``tab_conv2d_chain_launch``: ``Y = conv(X) + residual`` and,
    when ``threshold_scale`` is given, the next layer's thresholds ``threshold_scale * mean|Y[n]|``.
    Returns ``(Y, next_thresholds_or_None)``.  Not part of the reference's interface."""
    _check_input(X, "X", torch.float32)
    _check_input(QW, "QW", torch.int64)
    _check_input(thresholds, "thresholds", torch.float32)
    _check_input(btn, "btn", torch.int32)
    conv_type = int(type)
    p1, p2, s1, s2 = int(padding1), int(padding2), int(stride1), int(stride2)
    N, H, W, C, KN, KH, KW = (int(v) for v in (N, H, W, C, KN, KH, KW))
    _conv_checks(conv_type, QW, btn, N, H, W, C, KN, KH, KW, p1, p2, s1, s2)
    if X.numel() != N * H * W * C or thresholds.numel() != N:
        raise RuntimeError("X / thresholds do not match N*H*W*C / N")
    OH, OW = conv_out_size(H, W, KH, KW, p1, p2, s1, s2)
    if residual is not None:
        _check_input(residual, "residual", torch.float32)
        if residual.numel() != N * KN * OH * OW:
            raise RuntimeError("residual has %d elements, expected %d" % (residual.numel(), N * KN * OH * OW))
    l = _cabi.lib()
    with torch.cuda.device(X.device):
        Y = torch.empty((N, KN, OH, OW), dtype=torch.float32, device=X.device)
        ws = torch.empty((max(l.tab_conv2d_workspace_bytes(conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW), 256),), dtype=torch.uint8, device=X.device)
        sums = torch.empty((max(N, 1),), dtype=torch.float64, device=X.device) if threshold_scale is not None else None
        nxt = torch.empty((N,), dtype=torch.float32, device=X.device) if threshold_scale is not None else None
        st = _stream_ptr(X.device)
        rc = l.tab_conv2d_chain_launch(X.data_ptr(), QW.data_ptr(), thresholds.data_ptr(), btn.data_ptr(), Y.data_ptr(),
                                       ws.data_ptr(), ws.numel(), conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                       residual.data_ptr() if residual is not None else None,
                                       sums.data_ptr() if sums is not None else None,
                                       nxt.data_ptr() if nxt is not None else None,
                                       float(threshold_scale) if threshold_scale is not None else 0.0, st)
        _cabi.check(rc, "tab_conv2d_chain_launch")
    return Y, nxt
