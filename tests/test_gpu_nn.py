"""``tab_b200.nn.TABConv2d`` (prepared weights, the caller above the raw operators) and the chain written on it,
against the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

import tab_b200 as TAB
from tab_b200 import _cabi, chain, nn as tab_nn
from oracle import c_oracle, tab_oracle as O
from oracle.oracle_ops import OracleOps
from util import make_input

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("geom", [
    # pad stride N  H   W   C   KN K
    (1, 1, 3, 14, 14, 256, 96, 3),
    (0, 2, 2, 28, 28, 128, 256, 1),
    (1, 2, 2, 15, 11, 70, 33, 3),
    (3, 2, 1, 40, 40, 3, 16, 7),
])
def test_module_matches_oracle(cuda, t, geom):
    pad, stride, N, H, W, C, KN, K = geom
    x, ths = make_input(31, N, H, W, C)
    w, wths = make_input(32, KN, K, K, C)
    m = tab_nn.TABConv2d.from_float(torch.from_numpy(w).to(cuda), t, pad, stride, torch.from_numpy(wths).to(cuda))
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
    assert np.array_equal(m.QW.cpu().numpy().reshape(-1), qw.reshape(-1)) and np.array_equal(m.BTN_W.cpu().numpy(), btn)
    y = m(torch.from_numpy(x).to(cuda), torch.from_numpy(ths).to(cuda))
    yo = c_oracle.conv2d(x, qw, ths, btn, t, pad, pad, stride, stride, N, H, W, C, KN, K, K)
    assert tuple(y.shape) == yo.shape and np.array_equal(y.cpu().numpy(), yo)
    # thresholds computed by the module when none are passed: 0.7 * mean|x| per image, in double
    y2 = m(torch.from_numpy(x).to(cuda))
    tho = OracleOps.residual_threshold(x.copy(), None, 0.7)
    assert np.array_equal(y2.cpu().numpy(), c_oracle.conv2d(x, qw, tho, btn, t, pad, pad, stride, stride, N, H, W, C, KN, K, K))
    assert _cabi.lib().tab_device_status() == 0


def test_module_rejects_weights_of_the_wrong_bitwidth(cuda):
    """The reference's notebook passes 1-bit weights to 2-bit types (an out-of-bounds read there); here it is an error."""
    w, wths = make_input(1, 8, 3, 3, 64)
    q1, b1 = TAB.Quantize(torch.from_numpy(w).to(cuda), torch.from_numpy(wths).to(cuda), 1, 8, 3, 3, 64)
    with pytest.raises(ValueError, match="bitwidth 2"):
        tab_nn.TABConv2d(q1, b1, 0, 8, 3, 3, 64, 1, 1)
    tab_nn.TABConv2d(q1, b1, 1, 8, 3, 3, 64, 1, 1)          # the same weights are right for TBN


@pytest.mark.parametrize("t", [0, 3])
def test_prepared_chain_matches_oracle(cuda, t):
    """The 19-convolution chain on prepared modules (one quantised tensor per input, shared with the shortcut; residual and
    thresholds in the epilogue; one state block reused by every layer), N = 3, N(0,1) input like the benchmark's: the
    oracle gets the input thresholds the device computed, every later threshold follows from the data."""
    N = 3
    rng = np.random.default_rng(8)
    x = rng.standard_normal((N, 56, 56, 64), dtype=np.float32)
    weights = chain.make_weights(2000, t)
    specs = {cs.name: cs for cs in chain.conv_specs()}
    convs = {}
    for name, (w, wt) in weights.items():
        cs = specs[name]
        convs[name] = tab_nn.TABConv2d.from_float(torch.from_numpy(w).to(cuda), t, cs.pad, cs.stride, torch.from_numpy(wt).to(cuda))

    class Nhwc:
        def __init__(self, c):
            self.c = c
            self.conv_type = c.conv_type

        def quantize(self, xx, th):
            return self.c.quantize(xx, th)

        def conv_bits(self, *a, **k):
            out = self.c.conv_bits(*a, **k)
            y = out[0]
            return (y.view(y.shape[0], y.shape[2], y.shape[3], y.shape[1]),) + tuple(out[1:])

    xd = torch.from_numpy(x).to(cuda)
    thd = TAB.ops.residual_threshold(xd.reshape(N, -1), None, chain.THRESHOLD_SCALE)
    qo = chain.quantize_weights(weights, t, OracleOps.Quantize)
    yo, _, _, _ = chain.forward(OracleOps, x, thd.cpu().numpy(), qo, t, N)
    for compact in (False, True):                                      # fp32 everywhere / int16 between a block's two convolutions
        for fused_quant in (False, True):                              # quantiser launches / every convolution hands on its quantised result
            yd, oh, ow, kn = chain.forward_prepared({k: Nhwc(v) for k, v in convs.items()}, xd, thd, N, compact_mid=compact, fused_quant=fused_quant)
            assert (oh, ow, kn) == (7, 7, 512)
            assert np.array_equal(yd.cpu().numpy().reshape(-1), np.asarray(yo).reshape(-1)), (compact, fused_quant)
    assert _cabi.lib().tab_device_status() == 0
