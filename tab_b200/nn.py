"""``TABConv2d``: the caller the reference's demo notebook imports the pieces for (``nn``, ``F``, ``Function``) but never
writes - a module that owns one convolution's prepared weights and calls the two operators in the right order.

The reference's only interface is positional ``Conv2d(X, QW, thresholds, btn, type, ...16 ints)``
(``TAB_GPU.cpp:34-42``); its notebook quantises the weights once (cells 5-10) and then passes 1-bit weights to 2-bit
types (cells 12, 17), which reads past the end of ``QW`` (``TAB_GEMM.cu:47-52``).  This module

  * quantises the fp32 weights once, at the bitwidth the type needs (``TAB_GEMM.cu:374-379``), keeps ``QW`` and
    ``BTN_W`` (what ``Conv2d`` takes) and the byte-expanded form the tensor-core kernel multiplies, so that no call
    re-expands weights;
  * refuses weights quantised at the wrong bitwidth instead of reading out of bounds;
  * computes the per-image activation thresholds ``scale * mean|x|`` when the caller does not pass them;
  * exposes the two stages separately (``quantize`` / ``conv_bits``) so that several convolutions of one input -
    a block's first convolution and its strided shortcut - share one quantised tensor, and chained layers get
    ``y = conv + residual`` and the next thresholds from the convolution's own epilogue.

Results are those of ``Conv2d`` bit for bit.  Inference only: there is no backward (the reference has none).
"""
from __future__ import annotations

import torch

from . import _cabi, ops

TYPE_NAMES = {0: "TNN", 1: "TBN", 2: "BTN", 3: "BNN"}


def weight_bitwidth(conv_type: int) -> int:
    return 1 if conv_type in (1, 3) else 2


def act_bitwidth(conv_type: int) -> int:
    return 1 if conv_type in (2, 3) else 2


class TABConv2d(torch.nn.Module):
    """One TAB convolution with prepared weights.  ``forward(x)`` takes fp32 NHWC activations ``[N,H,W,C]`` and returns
    what ``Conv2d`` returns: float32 ``{N,KN,OH,OW}`` over a ``[N][OH][OW][KN]`` buffer (``TAB_GEMM.cu:509,526``)."""

    def __init__(self, QW, BTN_W, conv_type, KN, KH, KW, C, padding=(0, 0), stride=(1, 1), threshold_scale=0.7):
        super().__init__()
        conv_type = int(conv_type)
        if conv_type not in TYPE_NAMES:
            raise ValueError("type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)")
        self.conv_type, self.KN, self.KH, self.KW, self.C = conv_type, int(KN), int(KH), int(KW), int(C)
        self.padding = (int(padding), int(padding)) if isinstance(padding, int) else tuple(int(v) for v in padding)
        self.stride = (int(stride), int(stride)) if isinstance(stride, int) else tuple(int(v) for v in stride)
        self.threshold_scale = float(threshold_scale)
        wb = weight_bitwidth(conv_type)
        need = self.KN * self.KH * self.KW * ((self.C + 63) // 64) * wb
        if QW.numel() != need:
            raise ValueError("QW has %d words but type %d (%s) needs weights quantised at bitwidth %d: %d words"
                             % (QW.numel(), conv_type, TYPE_NAMES[conv_type], wb, need))
        if BTN_W.numel() != self.KN:
            raise ValueError("BTN_W has %d elements, expected KN = %d" % (BTN_W.numel(), self.KN))
        self.register_buffer("QW", QW.contiguous())
        self.register_buffer("BTN_W", BTN_W.contiguous())
        self.register_buffer("W8", ops.expand_weights(self.QW, wb, self.KN, self.KH, self.KW, self.C))
        self._state = None

    @classmethod
    def from_float(cls, weight, conv_type, padding=(0, 0), stride=(1, 1), weight_thresholds=None, threshold_scale=0.7):
        """``weight``: fp32 CUDA tensor ``[KN,KH,KW,C]``; per-filter thresholds default to ``threshold_scale * mean|w|``."""
        if weight.dim() != 4:
            raise ValueError("weight must be [KN,KH,KW,C]")
        KN, KH, KW, C = (int(v) for v in weight.shape)
        w = weight.contiguous().float()
        if weight_thresholds is None:
            weight_thresholds = (threshold_scale * w.abs().reshape(KN, -1).mean(dim=1)).float()
        QW, BTN_W = ops.Quantize(w, weight_thresholds.contiguous(), weight_bitwidth(int(conv_type)), KN, KH, KW, C)
        return cls(QW, BTN_W, conv_type, KN, KH, KW, C, padding, stride, threshold_scale)

    # ---- geometry -----------------------------------------------------------------------------------------------
    def geometry(self, N, H, W):
        return (self.padding[0], self.padding[1], self.stride[0], self.stride[1], int(N), int(H), int(W), self.C, self.KN, self.KH, self.KW)

    def out_size(self, H, W):
        return ops.conv_out_size(H, W, self.KH, self.KW, self.padding[0], self.padding[1], self.stride[0], self.stride[1])

    def state(self, N, device):
        """The zeroed state block ``conv_bits`` needs for thresholds; kept, every call leaves it zeroed."""
        if self._state is None or self._state.numel() < _cabi.lib().tab_conv2d_state_bytes(int(N)) or self._state.device != device:
            self._state = ops.new_state(N, device)
        return self._state

    # ---- the two stages -----------------------------------------------------------------------------------------
    def quantize(self, x, thresholds=None):
        """NHWC ``[N,H,W,C]`` activations -> bit-planes at the activation bitwidth of this convolution's type.  ``x`` is fp32,
        or the int16 a previous ``conv_bits(..., out_int16=True)`` returned (then ``thresholds`` must be given)."""
        N, H, W = (int(v) for v in x.shape[:3])
        if x.dtype == torch.int16:
            if thresholds is None:
                raise ValueError("int16 activations come with the thresholds their convolution produced")
            return ops.quantize_i16(x, thresholds, act_bitwidth(self.conv_type), N, H, W, self.C)
        if thresholds is None:
            return self.quantize_auto(x)[0]
        return ops.Quantize(x, thresholds, act_bitwidth(self.conv_type), N, H, W, self.C)[0]

    def quantize_auto(self, x):
        """``quantize`` of fp32 activations against ``threshold_scale * mean|x[n]|``, both from one launch.  Returns
        ``(QX, thresholds)``."""
        N, H, W = (int(v) for v in x.shape[:3])
        return ops.quantize_auto(x, self.threshold_scale, act_bitwidth(self.conv_type), N, H, W, self.C, self.state(N, x.device))

    def conv_bits(self, QX, N, H, W, residual=None, next_threshold_scale=None, state=None, out_int16=False, next_bitwidth=None):
        """GEMM stage on quantised activations.  Returns ``(Y, next_thresholds_or_None)``.  ``out_int16``: ``Y`` as int16
        where that is possible (no residual, KH*KW*C <= 32767, a shape the tensor-core kernel covers), else fp32 as usual:
        look at ``Y.dtype``.  ``next_bitwidth`` (with ``next_threshold_scale``): a third value is returned, ``Y`` quantised
        against the next thresholds at that bitwidth - the next convolution's ``QX`` - from the same launch."""
        if next_threshold_scale is not None and state is None:
            state = self.state(N, QX.device)
        if next_bitwidth is not None and next_threshold_scale is None:
            raise ValueError("next_bitwidth needs next_threshold_scale")
        compact = out_int16 and residual is None and self.KH * self.KW * self.C <= 32767
        try:
            return ops.conv2d_bits(QX, self.W8, self.conv_type, *self.geometry(N, H, W), residual=residual,
                                   threshold_scale=next_threshold_scale, state=state, out_int16=compact, next_bitwidth=next_bitwidth)
        except _cabi.TabError as exc:
            if exc.code != -5:
                raise
        # shapes the tensor-core kernel does not cover: the bit-packed popcount kernel, then the chaining in one pass
        Y = ops.conv2d_packed(QX, self.QW, self.BTN_W, self.conv_type, *self.geometry(N, H, W))
        nxt = None
        if residual is not None or next_threshold_scale is not None:
            nxt = ops.residual_threshold(Y, residual, next_threshold_scale if next_threshold_scale is not None else 0.0)
            if next_threshold_scale is None:
                nxt = None
        if next_bitwidth is not None:
            OH, OW = self.out_size(H, W)
            return Y, nxt, ops.Quantize(Y, nxt, next_bitwidth, N, OH, OW, self.KN)[0]
        return Y, nxt

    def forward(self, x, thresholds=None):
        if x.dim() != 4 or int(x.shape[3]) != self.C:
            raise ValueError("x must be fp32 NHWC [N,H,W,%d]" % self.C)
        N, H, W = (int(v) for v in x.shape[:3])
        return self.conv_bits(self.quantize(x.contiguous(), thresholds), N, H, W)[0]

    def extra_repr(self):
        return "%s, C=%d, KN=%d, kernel=%dx%d, padding=%s, stride=%s" % (
            TYPE_NAMES[self.conv_type], self.C, self.KN, self.KH, self.KW, self.padding, self.stride)
