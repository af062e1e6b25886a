"""Host-side logic that needs no GPU: input checks of the operator mirror, the chain definition (run on
the CPU oracle), shard arithmetic."""
import numpy as np
import pytest
import torch

import tab_b200
from tab_b200 import chain, dp
from oracle.oracle_ops import OracleOps
from oracle import tab_oracle as O


def test_check_input_messages_match_the_reference_binding():
    x = torch.zeros(1, 2, 2, 64)
    t = torch.zeros(1)
    with pytest.raises(RuntimeError, match="X must be a CUDA tensor"):
        tab_b200.Quantize(x, t, 2, 1, 2, 2, 64)
    qw = torch.zeros(4 * 9 * 2, dtype=torch.int64)
    btn = torch.zeros(4, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="X must be a CUDA tensor"):
        tab_b200.Conv2d(x, qw, t, btn, 0, 1, 1, 1, 1, 1, 2, 2, 64, 4, 3, 3)
    assert tab_b200.TAB_Quantize is tab_b200.Quantize and tab_b200.TAB_Conv2d is tab_b200.Conv2d


def test_out_size_uses_the_reference_formula():
    # (H + 2p - KH + 1) // s, not floor((H + 2p - KH) / s) + 1
    assert tab_b200.conv_out_size(10, 7, 3, 3, 1, 1, 3, 2) == (10 // 3, 7 // 2)
    assert tab_b200.conv_out_size(56, 56, 3, 3, 1, 1, 2, 2) == (28, 28)
    assert tab_b200.conv_out_size(56, 56, 1, 1, 0, 0, 2, 2) == (28, 28)
    assert tab_b200.conv_out_size(2, 2, 3, 3, 0, 0, 1, 1) == (0, 0)


def test_chain_shape_and_op_count():
    specs = chain.conv_specs()
    assert len(specs) == 19 and sum(1 for s in specs if s.K == 3) == 16 and sum(1 for s in specs if s.K == 1) == 3
    assert abs(chain.chain_binary_ops(256) / 1e12 - 0.868) < 0.001


def test_chain_on_the_cpu_oracle_matches_layer_by_layer_dense_math():
    N = 1
    rng = np.random.default_rng(5)
    x = np.round(rng.standard_normal((N, 56, 56, 64)) * 4).astype(np.float32)
    ths = OracleOps.residual_threshold(x.copy(), None, chain.THRESHOLD_SCALE)
    weights = chain.make_weights(1000, 0)
    qw = chain.quantize_weights(weights, 0, OracleOps.Quantize)
    y, oh, ow, kn = chain.forward(OracleOps, x, ths, qw, 0, N)
    assert (oh, ow, kn) == (7, 7, 512) and y.size == N * 7 * 7 * 512
    assert np.array_equal(y, np.round(y))                     # integer-valued all the way through
    # first convolution of the chain against the independent dense formulation
    a = chain.resnet18_blocks()[0].conv_a
    y1 = OracleOps.Conv2d(x, qw[a.name][0], ths, qw[a.name][1], 0, 1, 1, 1, 1, N, 56, 56, 64, 64, 3, 3)
    assert np.array_equal(y1, O.conv2d_dense(x, qw[a.name][0], ths, 0, 1, 1, 1, 1, N, 56, 56, 64, 64, 3, 3))
    # the same chain written on prepared convolutions (one quantised tensor per input, shared with the shortcut)
    from oracle.oracle_ops import OraclePreparedConv
    specs = {cs.name: cs for cs in chain.conv_specs()}
    convs = {k: OraclePreparedConv(v[0], v[1], 0, specs[k]) for k, v in qw.items()}
    for compact in (False, True):
        for fused_quant in (False, True):                     # every convolution hands on its quantised result itself
            yp, oh2, ow2, kn2 = chain.forward_prepared(convs, x, ths, N, compact_mid=compact, fused_quant=fused_quant)
            assert (oh2, ow2, kn2) == (7, 7, 512) and np.array_equal(np.asarray(yp).reshape(-1), np.asarray(y).reshape(-1))


@pytest.mark.parametrize("N,world", [(8, 1), (8, 2), (5, 2), (3, 4), (256, 8), (0, 2)])
def test_shard_bounds_partition_the_batch(N, world):
    spans = [dp.shard_bounds(N, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == N
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a1 - a0 >= b1 - b0 >= 0
    assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
