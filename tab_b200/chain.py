"""ResNet-18-shaped chain of TAB convolutions (the network-level workload of the benchmark).

The reference defines no network: it exposes ``Quantize`` and ``Conv2d`` only, and leaves thresholds,
residual additions and layer chaining to the caller.  This module writes that caller down once, so that
the benchmark, the tests and the CPU oracle all run the very same sequence:

  * input: fp32 NHWC activations ``[N,56,56,64]`` (the output of a ResNet-18 stem; the first
    convolution and the final classifier are not part of the chain);
  * four stages of two basic blocks; a block is ``conv3x3 -> conv3x3`` plus a shortcut, added
    elementwise: the identity, or a ``conv1x1`` stride 2 pad 0 where the stage halves the resolution
    and doubles the width (64 -> 128 -> 256 -> 512 channels, 56 -> 28 -> 14 -> 7 pixels);
    16 3x3 convolutions and 3 1x1 convolutions in all;
  * every convolution input is re-quantised with a per-image threshold ``0.7 * mean|x|``
    (``Conv2d`` takes fp32 activations, TAB_GEMM.cu:419-426); there is no batch-norm and no other
    non-linearity; ``Conv2d``'s output buffer ``[N][OH][OW][KN]`` is the next layer's NHWC input as is;
  * weights: seeded N(0,1), quantised per filter at ``0.7 * mean|w|`` with the bitwidth the type needs.

``forward`` is written against a small ``ops`` interface (``Conv2d``, ``residual_threshold``) so that
the identical topology runs on the device operators of this package and, in the tests, on a CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np

THRESHOLD_SCALE = 0.7


@dataclass
class ConvSpec:
    name: str
    C: int
    KN: int
    K: int
    stride: int
    pad: int


@dataclass
class BlockSpec:
    conv_a: ConvSpec
    conv_b: ConvSpec
    shortcut: Optional[ConvSpec]     # None = identity


def resnet18_blocks() -> List[BlockSpec]:
    blocks = []
    c_in = 64
    for stage, c_out in enumerate([64, 128, 256, 512]):
        for b in range(2):
            down = (b == 0 and stage > 0)
            s = 2 if down else 1
            blocks.append(BlockSpec(
                ConvSpec("s%db%d.a" % (stage + 1, b), c_in, c_out, 3, s, 1),
                ConvSpec("s%db%d.b" % (stage + 1, b), c_out, c_out, 3, 1, 1),
                ConvSpec("s%db%d.sc" % (stage + 1, b), c_in, c_out, 1, 2, 0) if down else None))
            c_in = c_out
    return blocks


def conv_specs() -> List[ConvSpec]:
    out = []
    for b in resnet18_blocks():
        out += [b.conv_a, b.conv_b] + ([b.shortcut] if b.shortcut else [])
    return out


def chain_binary_ops(N: int, H: int = 56, W: int = 56) -> int:
    """2*M*KN*KH*KW*C summed over the 19 convolutions (one multiply and one add per tap)."""
    total = 0
    h, w = H, W
    for b in resnet18_blocks():
        oh, ow = (h + 2 - 3 + 1) // b.conv_a.stride, (w + 2 - 3 + 1) // b.conv_a.stride
        total += 2 * N * oh * ow * b.conv_a.KN * 9 * b.conv_a.C
        total += 2 * N * oh * ow * b.conv_b.KN * 9 * b.conv_b.C
        if b.shortcut:
            total += 2 * N * oh * ow * b.shortcut.KN * b.shortcut.C
        h, w = oh, ow
    return total


def make_weights(seed: int, conv_type: int = 0):
    """Seeded fp32 weights ``[KN,K,K,C]`` and per-filter thresholds for every convolution, as numpy arrays
    keyed by layer name (seed + layer index per tensor)."""
    out = {}
    for i, cs in enumerate(conv_specs()):
        rng = np.random.default_rng(seed + i)
        w = rng.standard_normal((cs.KN, cs.K, cs.K, cs.C), dtype=np.float32)
        t = (np.float32(THRESHOLD_SCALE) * np.abs(w).reshape(cs.KN, -1).mean(axis=1, dtype=np.float32)).astype(np.float32)
        out[cs.name] = (w, t)
    return out


def weight_bitwidth(conv_type: int) -> int:
    return 1 if conv_type in (1, 3) else 2


def quantize_weights(weights, conv_type, quantize_fn, to_backend=lambda a: a):
    """name -> (QW, BTN_W) using the backend's ``Quantize``."""
    q = {}
    specs = {cs.name: cs for cs in conv_specs()}
    for name, (w, t) in weights.items():
        cs = specs[name]
        qw, btn = quantize_fn(to_backend(w), to_backend(t), weight_bitwidth(conv_type), cs.KN, cs.K, cs.K, cs.C)
        q[name] = (qw, btn)
    return q


def forward(ops, x, ths, qweights, conv_type: int, N: int, H: int = 56, W: int = 56):
    """Run the chain.  ``x``: fp32 activations with N*H*W*64 elements (NHWC); ``ths``: thresholds ``[N]``
    for ``x``.  Returns ``(y, OH, OW, KN)`` where ``y`` holds N*OH*OW*KN floats in NHWC order.  ``x`` is
    not modified.

    ``ops`` provides ``Conv2d(...)`` and ``residual_threshold(Y, residual, scale)``; if it also provides
    ``Conv2dFused(..., residual, threshold_scale) -> (Y, next_thresholds)`` the residual addition and the
    threshold statistics ride in the convolution's epilogue instead of separate passes (same results)."""
    fused = getattr(ops, "Conv2dFused", None)
    h, w = H, W
    for b in resnet18_blocks():
        a, bb, sc = b.conv_a, b.conv_b, b.shortcut
        qa, ba = qweights[a.name]
        qb, bbt = qweights[bb.name]
        oh, ow = (h + 2 * a.pad - a.K + 1) // a.stride, (w + 2 * a.pad - a.K + 1) // a.stride
        ga = (a.pad, a.pad, a.stride, a.stride, N, h, w, a.C, a.KN, a.K, a.K)
        gb = (bb.pad, bb.pad, bb.stride, bb.stride, N, oh, ow, bb.C, bb.KN, bb.K, bb.K)
        if sc is None:
            short = x
        else:
            qs, bs = qweights[sc.name]
            short = ops.Conv2d(x, qs, ths, bs, conv_type, sc.pad, sc.pad, sc.stride, sc.stride, N, h, w, sc.C, sc.KN, sc.K, sc.K)
        if fused is not None:
            y1, t1 = fused(x, qa, ths, ba, conv_type, *ga, None, THRESHOLD_SCALE)
            y2, ths = fused(y1, qb, t1, bbt, conv_type, *gb, short, THRESHOLD_SCALE)   # y2 = conv + shortcut
        else:
            y1 = ops.Conv2d(x, qa, ths, ba, conv_type, *ga)
            t1 = ops.residual_threshold(y1, None, THRESHOLD_SCALE)
            y2 = ops.Conv2d(y1, qb, t1, bbt, conv_type, *gb)
            ths = ops.residual_threshold(y2, short, THRESHOLD_SCALE)      # y2 += short; thresholds of the sum
        x, h, w = y2, oh, ow
    return x, h, w, resnet18_blocks()[-1].conv_b.KN


def forward_prepared(convs, x, ths, N: int, H: int = 56, W: int = 56, compact_mid: bool = False, fused_quant: bool = False, qx0=None):
    """The same chain on prepared convolutions: ``convs`` maps a layer name to an object with
    ``quantize(x, thresholds) -> QX`` and ``conv_bits(QX, N, H, W, residual, next_threshold_scale) -> (Y, next_ths)``
    (``tab_b200.nn.TABConv2d``: weights quantised and expanded once).  Every convolution input is quantised once:
    a block's first convolution and its strided shortcut read the same bit-planes (same input, same thresholds).
    ``compact_mid``: a block's first convolution hands its result to the second one's quantiser as int16 (it is
    integer-valued and nothing else reads it), half the bytes of fp32; the convolution objects must accept
    ``conv_bits(..., out_int16=True)`` and int16 input to ``quantize``.
    ``fused_quant``: every convolution that feeds another one also hands it its quantised input
    (``conv_bits(..., next_bitwidth=bits) -> (Y, next_ths, next_QX)``; the objects need a ``conv_type``), so that only the
    chain's input is quantised by a launch of its own; ``qx0``: that quantised input, when the caller already has it
    (``quantize_auto`` gives it together with ``ths``).
    Returns ``(y, OH, OW, KN)`` like ``forward``; the results are identical."""
    h, w = H, W
    if fused_quant:
        blocks = resnet18_blocks()
        act_bits = lambda conv: 1 if conv.conv_type in (2, 3) else 2
        qx = qx0 if qx0 is not None else convs[blocks[0].conv_a.name].quantize(x, ths)
        for i, b in enumerate(blocks):
            a, bb, sc = convs[b.conv_a.name], convs[b.conv_b.name], (convs[b.shortcut.name] if b.shortcut else None)
            oh, ow = (h + 2 * b.conv_a.pad - b.conv_a.K + 1) // b.conv_a.stride, (w + 2 * b.conv_a.pad - b.conv_a.K + 1) // b.conv_a.stride
            short = x if sc is None else sc.conv_bits(qx, N, h, w, None, None)[0]
            _, _, q1 = a.conv_bits(qx, N, h, w, None, THRESHOLD_SCALE, out_int16=compact_mid, next_bitwidth=act_bits(bb))
            if i + 1 < len(blocks):
                x, ths, qx = bb.conv_bits(q1, N, oh, ow, short, THRESHOLD_SCALE, next_bitwidth=act_bits(convs[blocks[i + 1].conv_a.name]))
            else:
                x, ths = bb.conv_bits(q1, N, oh, ow, short, THRESHOLD_SCALE)
            h, w = oh, ow
        return x, h, w, blocks[-1].conv_b.KN
    for b in resnet18_blocks():
        a, bb, sc = convs[b.conv_a.name], convs[b.conv_b.name], (convs[b.shortcut.name] if b.shortcut else None)
        oh, ow = (h + 2 * b.conv_a.pad - b.conv_a.K + 1) // b.conv_a.stride, (w + 2 * b.conv_a.pad - b.conv_a.K + 1) // b.conv_a.stride
        qx = a.quantize(x, ths)
        short = x if sc is None else sc.conv_bits(qx, N, h, w, None, None)[0]
        y1, t1 = a.conv_bits(qx, N, h, w, None, THRESHOLD_SCALE, out_int16=True) if compact_mid else a.conv_bits(qx, N, h, w, None, THRESHOLD_SCALE)
        y2, ths = bb.conv_bits(bb.quantize(y1, t1), N, oh, ow, short, THRESHOLD_SCALE)     # y2 = conv + shortcut
        x, h, w = y2, oh, ow
    return x, h, w, resnet18_blocks()[-1].conv_b.KN
