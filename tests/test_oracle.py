"""The oracle is pinned before anything is compared with it: against golden vectors produced by the
reference's own code (its CUDA kernel bodies run on the host for every stage, its CPU GEMMs), against
that code directly when ``oracle/_ref`` is present, against the facts the reference's demo notebook
records, and against an independent dense formulation."""
import glob
import os

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import c_oracle, tab_oracle as O
from util import make_input

GOLD = os.path.join(os.path.dirname(__file__), "golden")
NAMES = ["tnn", "tbn", "btn", "bnn"]


@pytest.mark.parametrize("name", NAMES)
def test_gemm_golden(name):
    g = np.load(os.path.join(GOLD, "gemm_%s.npz" % name))
    t, K, NUM = int(g["type"]), int(g["K"]), int(g["NUM"])
    a, b, btn, y = g["a"], g["b"], g["btn"], g["y"]
    assert np.array_equal(O.gemm(a, b, btn, t, K, NUM), y)
    assert np.array_equal(c_oracle.gemm(a, b, btn, t, a.shape[0], b.shape[0], K, NUM), y)


def test_conv_cfg1_golden():
    g = np.load(os.path.join(GOLD, "conv_cfg1_tnn.npz"))
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = (int(v) for v in g["geom"])
    qw, btn = O.quantize(g["w"], g["wths"], 2, KN, KH, KW, C)
    assert np.array_equal(qw, g["qw"]) and np.array_equal(btn, g["btn"])
    y = O.conv2d(g["x"], qw, g["ths"], btn, 0, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    assert y.shape == (N, KN, 32, 32) and y.dtype == np.float32
    assert np.array_equal(y, g["y"].astype(np.float32))
    yc = c_oracle.conv2d(g["x"], qw, g["ths"], btn, 0, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    assert np.array_equal(yc, y)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "conv_small_*.npz"))))
def test_conv_small_golden(path):
    g = np.load(path)
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = (int(v) for v in g["geom"])
    for t, name in enumerate(NAMES):
        qw, btn = O.quantize(g["w"], g["wths"], O.weight_bits(t), KN, KH, KW, C)
        assert np.array_equal(qw, g["qw_" + name]) and np.array_equal(btn, g["btn_" + name])
        y = O.conv2d(g["x"], qw, g["ths"], btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
        assert np.array_equal(y, g["y_" + name].astype(np.float32)), name
        yc = c_oracle.conv2d(g["x"], qw, g["ths"], btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, variant="shipped")
        assert np.array_equal(yc, y), name


def test_quantize_edges_golden():
    g = np.load(os.path.join(GOLD, "quantize_edges.npz"))
    x, ths = g["x"], g["ths"]
    N, H, W, C = x.shape
    for bw, qk, bk in ((2, "q2", "btn2"), (1, "q1", "btn1")):
        for q, b in (O.quantize(x, ths, bw, N, H, W, C), c_oracle.quantize(x, ths, bw, N, H, W, C)):
            assert np.array_equal(q, g[qk]) and np.array_equal(b, g[bk])
    # spelled-out rules (TAB_GEMM.cu:184-192, :231): strict compares, NaN -> 0 / +1, equality -> 0 / +1
    q2, q1 = g["q2"], g["q1"]
    s0, m0 = int(q2[0, 0, 0, 0, 0]), int(q2[0, 0, 0, 0, 1])
    # channels 0..7 of pixel (0,0,0): 0.5, -0.5, 0.5+, -0.5-, 0, -0, NaN, inf with t = 0.5
    assert (m0 & 0xFF) == 0b10001100 and (s0 & 0xFF) == 0b00001000
    b0 = int(q1[0, 0, 0, 0, 0])
    assert (b0 & 0xFF) == 0b00111010     # x < 0.5: -0.5, -0.5-, 0, -0 ; not 0.5, 0.5+, NaN, inf


@pytest.mark.skipif(not c_oracle.ref_available(), reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("t", range(4))
def test_gemm_against_reference_build(t):
    rng = np.random.default_rng(t)
    for M, KN, K in [(1, 1, 1), (5, 3, 2), (33, 17, 9), (64, 64, 36)]:
        ab, wb = O.act_bits(t), O.weight_bits(t)
        a = rng.integers(-2**63, 2**63 - 1, size=(M, K * ab), dtype=np.int64)
        b = rng.integers(-2**63, 2**63 - 1, size=(KN, K * wb), dtype=np.int64)
        btn = rng.integers(0, 64 * K, size=KN).astype(np.int32)
        ref = c_oracle.gemm(a, b, btn, t, M, KN, K, 64 * K, use_ref=True)
        assert np.array_equal(O.gemm(a, b, btn, t, K, 64 * K), ref)
        assert np.array_equal(c_oracle.gemm(a, b, btn, t, M, KN, K, 64 * K), ref)


@pytest.mark.skipif(not c_oracle.ref_available(), reason="oracle/_ref not built (reference tree absent)")
def test_im2row_against_reference_build():
    rng = np.random.default_rng(7)
    # The reference's loop walks h < H-KH+1 in steps of s and overruns its own OH*OW buffer when s does
    # not divide H-KH+1 (TAB_CPU.h:39,41), so it is only callable on sizes where it divides.
    N, H, W, Cp, KH, KW = 2, 8, 10, 3, 3, 3
    q = rng.integers(-2**63, 2**63 - 1, size=(N, H, W, Cp), dtype=np.int64)
    for s in (1, 2):
        rows = O.im2row(q, KH, KW, s, s)
        out = np.zeros_like(rows)
        n = c_oracle.ref_lib().ref_im2row_3x3(q.ctypes.data, out.ctypes.data, N, Cp, H, W, KH, KW, s, s)
        assert n == rows.size
        assert np.array_equal(out, rows)


need_ref_cuda = pytest.mark.skipif(not c_oracle.ref_cuda_available(),
                                   reason="oracle/_ref/libtab_ref_cuda.so not built (reference tree absent)")
CHANNELS = [3, 64, 65, 200]


def _edge_input(N, H, W, C, seed):
    """N(0,1) data with the compare edge cases planted in every image: +-threshold, the floats next to it,
    +-0, NaN, +-inf, denormals."""
    x, ths = make_input(seed, N, H, W, C)
    for n in range(N):
        t = ths[n]
        edge = np.array([t, -t, np.nextafter(t, np.float32(9)), np.nextafter(-t, np.float32(-9)), np.nextafter(t, np.float32(0)),
                         np.nextafter(-t, np.float32(0)), 0.0, -0.0, np.nan, np.inf, -np.inf, 1e-45, -1e-45], dtype=np.float32)
        flat = x[n].reshape(-1)
        k = min(edge.size, flat.size)
        flat[(np.arange(k) * 7 + n) % flat.size] = edge[:k]
    return x, ths


@need_ref_cuda
@pytest.mark.parametrize("C", CHANNELS)
@pytest.mark.parametrize("bw", [2, 1])
def test_quantize_against_reference_cuda_kernels(C, bw):
    """TerOnlyKernel / BinOnlyKernel / BTN_Weight themselves (TAB_GEMM.cu:150-247), on random data with edge values."""
    for N, H, W in [(16, 3, 5), (32, 1, 1), (5, 4, 3)]:
        x, ths = _edge_input(N, H, W, C, 40 + C + bw)
        ths[0] = 0.0                                               # +-0 against a zero threshold
        qr, br = c_oracle.ref_cuda_quantize(x, ths, bw, N, H, W, C)
        for q, b in (O.quantize(x, ths, bw, N, H, W, C), c_oracle.quantize(x, ths, bw, N, H, W, C)):
            assert np.array_equal(q, qr)
            done = 16 * (N // 16)                                  # the reference's <<<16, N/16>>> launch covers these
            assert np.array_equal(b[:done], br[:done])
            if bw == 1:
                assert not b.any() and not br.any()


@need_ref_cuda
@pytest.mark.parametrize("Cw", [1, 2, 3, 8])
def test_pad_and_im2row_against_reference_cuda_kernels(Cw):
    rng = np.random.default_rng(Cw)
    for N, H, W, p1, p2, KH, KW, s1, s2 in [(2, 5, 6, 1, 1, 3, 3, 1, 1), (1, 7, 4, 2, 0, 3, 1, 2, 1), (3, 6, 6, 0, 3, 1, 5, 1, 2),
                                            (2, 9, 8, 1, 1, 3, 3, 3, 2), (1, 4, 4, 0, 0, 1, 1, 2, 2)]:
        q = rng.integers(-2**63, 2**63 - 1, size=(N, H, W, Cw), dtype=np.int64)
        padded = O.pad_packed(q, p1, p2)
        assert np.array_equal(padded, c_oracle.ref_cuda_pad(q, p1, p2))
        assert np.array_equal(O.im2row(padded, KH, KW, s1, s2), c_oracle.ref_cuda_im2row(padded, KH, KW, s1, s2))


@need_ref_cuda
@pytest.mark.parametrize("t", range(4))
def test_gemm_against_reference_cuda_kernels(t):
    """TNN/TBN/BTN/BNNGEMM (TAB_GEMM.cu:25-147) under GEMMWithCuda's launch shape, incl. KN >= 1008 where that
    shape is not launchable on a device (a block of 16 x 64 threads) but is still well defined."""
    rng = np.random.default_rng(50 + t)
    for M, KN, K in [(1, 1, 1), (17, 5, 3), (40, 33, 9), (3, 1030, 2)]:
        ab, wb = O.act_bits(t), O.weight_bits(t)
        a = rng.integers(-2**63, 2**63 - 1, size=(M, K * ab), dtype=np.int64)
        b = rng.integers(-2**63, 2**63 - 1, size=(KN, K * wb), dtype=np.int64)
        btn = rng.integers(0, 64 * K, size=KN).astype(np.int32)
        ref = c_oracle.ref_cuda_gemm(a, b, btn, t, M, KN, K, 64 * K)
        assert ref.dtype == np.float32
        assert np.array_equal(O.gemm(a, b, btn, t, K, 64 * K).astype(np.float32), ref)
        assert np.array_equal(c_oracle.gemm(a, b, btn, t, M, KN, K, 64 * K).astype(np.float32), ref)


@need_ref_cuda
@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("C", CHANNELS)
def test_conv2d_against_reference_cuda_pipeline(t, C):
    """The whole ConvWithCuda_TAB sequence on the reference's kernels == both oracles."""
    geoms = [(1, 1, 1, 1, 2, 6, 7, 5, 3, 3), (0, 0, 1, 1, 2, 3, 4, 6, 1, 1), (1, 0, 2, 1, 1, 7, 5, 4, 3, 3),
             (0, 0, 2, 2, 3, 6, 6, 17, 1, 1), (2, 2, 1, 1, 1, 5, 5, 3, 5, 5), (1, 1, 3, 2, 2, 10, 7, 6, 3, 3)]
    for gi, (p1, p2, s1, s2, N, H, W, KN, KH, KW) in enumerate(geoms):
        x, ths = _edge_input(N, H, W, C, 60 + gi)
        w, wths = make_input(70 + gi, KN, KH, KW, C)
        qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
        ref = c_oracle.ref_cuda_conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
        assert np.array_equal(O.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW), ref)
        assert np.array_equal(c_oracle.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW), ref)


def test_notebook_facts():
    """Shapes/dtypes printed by the reference's demo notebook (cells 7, 10) for KN=64, KH=KW=3, C=256 with
    all-positive data: QW [64,3,3,4,2] int64, BTN_W [64]; all sign words zero; with the same data and
    threshold each binary word is the complement of the ternary magnitude word."""
    rng = np.random.default_rng(0)
    w = rng.random((64, 3, 3, 256), dtype=np.float32)
    t = (0.7 * w.reshape(64, -1).mean(axis=1)).astype(np.float32)
    q2, b2 = O.quantize(w, t, 2, 64, 3, 3, 256)
    q1, b1 = O.quantize(w, t, 1, 64, 3, 3, 256)
    assert q2.shape == (64, 3, 3, 4, 2) and q2.dtype == np.int64 and b2.shape == (64,) and b2.dtype == np.int32
    assert q1.shape == (64, 3, 3, 4, 1) and not b1.any()
    assert not q2[..., 0].any()
    assert np.array_equal(q1[..., 0], ~q2[..., 1])
    assert np.array_equal(b2, np.bitwise_count(q2[..., 1].view(np.uint64)).reshape(64, -1).sum(1))


GEOMS = [
    # p1 p2 s1 s2  N  H  W   C  KN KH KW
    (1, 1, 1, 1, 1, 5, 5, 64, 3, 3, 3),
    (0, 0, 1, 1, 2, 4, 6, 3, 2, 1, 1),
    (1, 0, 2, 1, 2, 7, 5, 65, 4, 3, 3),
    (0, 0, 2, 2, 1, 8, 8, 128, 5, 1, 1),
    (2, 2, 1, 1, 1, 6, 6, 70, 3, 5, 5),
    (3, 3, 2, 2, 1, 9, 9, 10, 2, 7, 7),
    (1, 1, 3, 2, 2, 10, 7, 200, 6, 3, 3),    # stride does not divide PH-KH+1
    (0, 0, 1, 1, 1, 2, 2, 64, 2, 3, 3),      # empty output (kernel larger than image)
]


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("g", GEOMS)
def test_oracle_equals_dense_convolution(t, g):
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = g
    x, ths = make_input(11, N, H, W, C)
    w, wths = make_input(12, KN, KH, KW, C)
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
    y = O.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    yd = O.conv2d_dense(x, qw, ths, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    yc = c_oracle.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    assert y.shape == yd.shape == yc.shape
    assert np.array_equal(y, yd) and np.array_equal(y, yc)


def test_binary_padding_is_plus_one():
    """Zero words in the border mean +1 for binary activations (types 2, 3) and 0 for ternary ones."""
    N, H, W, C, KN = 1, 1, 1, 64, 1
    x = np.full((N, H, W, C), 5.0, np.float32)          # all +1
    ths = np.array([1.0], np.float32)
    w = np.full((KN, 3, 3, C), 5.0, np.float32)         # all +1
    wths = np.array([1.0], np.float32)
    for t, expect in ((0, 64), (1, 64), (2, 9 * 64), (3, 9 * 64)):
        qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, 3, 3, C)
        y = O.conv2d(x, qw, ths, btn, t, 1, 1, 1, 1, N, H, W, C, KN, 3, 3)
        assert y.shape == (1, 1, 1, 1) and y[0, 0, 0, 0] == expect


def test_wrong_weight_bitwidth_is_rejected():
    w, wths = make_input(1, 4, 3, 3, 64)
    x, ths = make_input(2, 1, 5, 5, 64)
    qw1, btn = O.quantize(w, wths, 1, 4, 3, 3, 64)
    with pytest.raises(ValueError):
        O.conv2d(x, qw1, ths, btn, 0, 1, 1, 1, 1, 1, 5, 5, 64, 4, 3, 3)


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 3), st.integers(1, 3), st.integers(1, 9), st.integers(1, 9), st.integers(1, 140),
       st.integers(1, 9), st.sampled_from([1, 2, 3, 5]), st.sampled_from([1, 3]), st.integers(0, 2), st.integers(0, 2),
       st.integers(1, 3), st.integers(1, 3), st.integers(0, 2**31 - 1))
def test_random_shapes(t, N, H, W, C, KN, KH, KW, p1, p2, s1, s2, seed):
    x, ths = make_input(seed, N, H, W, C)
    w, wths = make_input(seed + 1, KN, KH, KW, C)
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
    qwc, btnc = c_oracle.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
    assert np.array_equal(qw, qwc) and np.array_equal(btn, btnc)
    y = O.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    assert np.array_equal(y, O.conv2d_dense(x, qw, ths, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW))
    assert np.array_equal(y, c_oracle.conv2d(x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW))
