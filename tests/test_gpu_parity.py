"""Parity of the CUDA path, called through the C ABI, with the CPU oracle: bit-exact (integer-valued
results; the comparison is array equality, tolerance 0)."""
import glob
import os

import numpy as np
import pytest
import torch

import tab_b200 as TAB
from tab_b200 import _cabi, chain
from oracle import c_oracle, tab_oracle as O
from oracle.oracle_ops import OracleOps
from util import make_input

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
NAMES = ["tnn", "tbn", "btn", "bnn"]


@pytest.fixture(autouse=True, params=["tensor", "popcount", "popcount-plain"])
def conv_path(request):
    """Every test of this module runs once per compute path of the convolution entry points: the persistent tcgen05
    kernel (shapes it does not cover fall back to the popcount kernel inside the call), the bit-packed popcount
    kernel with its carry-save tree, and the same with one POPC per word.  After each test the tensor-core kernel's
    record of expired waits must be clean."""
    l = _cabi.lib()
    prev = l.tab_conv2d_set_path({"tensor": 0, "popcount": 1, "popcount-plain": 2}[request.param])
    yield request.param
    l.tab_conv2d_set_path(prev)
    torch.cuda.synchronize()
    assert l.tab_device_status() == 0


def dev_t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def gpu_conv(cuda, x, qw, ths, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW):
    y = TAB.Conv2d(dev_t(x, cuda), dev_t(qw, cuda), dev_t(ths, cuda), dev_t(btn, cuda), t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    return y.cpu().numpy()


# ------------------------------------------------------------------------------------------ quantise

@pytest.mark.parametrize("bw", [2, 1])
@pytest.mark.parametrize("C", [3, 64, 65, 128, 200, 256])
@pytest.mark.parametrize("N,H,W", [(1, 1, 1), (3, 5, 7), (16, 9, 4)])
def test_quantize_matches_oracle(cuda, bw, C, N, H, W):
    x, ths = make_input(C * 7 + N, N, H, W, C)
    q, b = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), bw, N, H, W, C)
    qo, bo = O.quantize(x, ths, bw, N, H, W, C)
    assert q.dtype == torch.int64 and tuple(q.shape) == qo.shape and b.dtype == torch.int32
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(b.cpu().numpy(), bo)


def test_quantize_edge_values_golden(cuda):
    g = np.load(os.path.join(GOLD, "quantize_edges.npz"))
    x, ths = g["x"], g["ths"]
    N, H, W, C = x.shape
    for bw, qk, bk in ((2, "q2", "btn2"), (1, "q1", "btn1")):
        q, b = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), bw, N, H, W, C)
        assert np.array_equal(q.cpu().numpy(), g[qk]) and np.array_equal(b.cpu().numpy(), g[bk])
    # the same edge values through the vectorised path (C = 128)
    x2 = np.zeros((1, 2, 2, 128), np.float32)
    x2[0, 0, 0, :8] = x[0, 0, 0, :8]
    x2[0, 1, 1, 120:128] = x[0, 0, 0, :8]
    t2 = np.array([0.5], np.float32)
    for bw in (2, 1):
        q, b = TAB.Quantize(dev_t(x2, cuda), dev_t(t2, cuda), bw, 1, 2, 2, 128)
        qo, bo = O.quantize(x2, t2, bw, 1, 2, 2, 128)
        assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(b.cpu().numpy(), bo)


def test_quantize_empty_and_unaligned(cuda):
    q, b = TAB.Quantize(torch.empty(0, device=cuda), torch.empty(0, device=cuda), 2, 0, 4, 4, 64)
    assert tuple(q.shape) == (0, 4, 4, 1, 2) and tuple(b.shape) == (0,)
    q, b = TAB.Quantize(torch.empty(0, device=cuda), torch.zeros(3, device=cuda), 2, 3, 0, 4, 64)
    assert tuple(q.shape) == (3, 0, 4, 1, 2) and not b.cpu().numpy().any()
    # input that starts 4 bytes past a 16-byte boundary: the scalar path must take over
    N, H, W, C = 2, 3, 5, 64
    x, ths = make_input(9, N, H, W, C)
    buf = torch.zeros(x.size + 1, device=cuda)
    buf[1:] = dev_t(x.reshape(-1), cuda)
    q, b = TAB.Quantize(buf[1:], dev_t(ths, cuda), 2, N, H, W, C)
    qo, bo = O.quantize(x, ths, 2, N, H, W, C)
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(b.cpu().numpy(), bo)


def test_notebook_facts_on_device(cuda):
    g = torch.Generator(device=cuda)
    g.manual_seed(11)
    w = torch.rand(64, 3, 3, 256, device=cuda, generator=g)
    t = 0.7 * w.reshape(64, -1).mean(dim=1)
    # a value equal to its threshold is neither "< t" nor "> t": the complement relation below holds for all other values
    w = torch.where(w == t.reshape(64, 1, 1, 1), w + 0.25, w)
    q2, b2 = TAB.Quantize(w, t, 2, 64, 3, 3, 256)
    q1, b1 = TAB.Quantize(w, t, 1, 64, 3, 3, 256)
    assert tuple(q2.shape) == (64, 3, 3, 4, 2) and q2.dtype == torch.int64 and tuple(b2.shape) == (64,)
    assert not q2[..., 0].any().item()
    assert torch.equal(q1[..., 0], ~q2[..., 1])
    assert not b1.any().item()


@pytest.mark.parametrize("bw", [2, 1])
def test_quantize_full_size_configuration(cuda, bw):
    """N=256, 56x56x256 (822 MB): two images against the oracle, and the BTN_W counts against a popcount
    of the device's own magnitude plane (a checksum over everything that was written)."""
    N, H, W, C = 256, 56, 56, 256
    g = torch.Generator(device=cuda)
    g.manual_seed(1)
    x = torch.randn(N, H, W, C, device=cuda, generator=g)
    ths = (0.7 * x.abs().mean(dim=(1, 2, 3))).contiguous()
    q, b = TAB.Quantize(x, ths, bw, N, H, W, C)
    th = ths.cpu().numpy()
    for n in (0, 131, N - 1):
        qo, bo = c_oracle.quantize(x[n].cpu().numpy(), th[n:n + 1], bw, 1, H, W, C)
        assert np.array_equal(q[n].cpu().numpy(), qo[0])
        assert int(b[n].item()) == int(bo[0])
    if bw == 2:
        lut = torch.tensor([bin(i).count("1") for i in range(256)], dtype=torch.int32, device=cuda)
        mag_bytes = q[..., 1].contiguous().view(torch.uint8).reshape(N, -1)
        counts = lut[mag_bytes.long()].sum(dim=1, dtype=torch.int64)
        assert torch.equal(counts, b.long())
        assert not (q[..., 0] & ~q[..., 1]).any().item()      # a sign bit never without its magnitude bit
    else:
        assert not b.any().item()


# ------------------------------------------------------------------------------------------ convolution

def test_conv_cfg1_golden(cuda):
    g = np.load(os.path.join(GOLD, "conv_cfg1_tnn.npz"))
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = (int(v) for v in g["geom"])
    qw, btn = TAB.Quantize(dev_t(g["w"], cuda), dev_t(g["wths"], cuda), 2, KN, KH, KW, C)
    assert np.array_equal(qw.cpu().numpy(), g["qw"]) and np.array_equal(btn.cpu().numpy(), g["btn"])
    y = TAB.Conv2d(dev_t(g["x"], cuda), qw, dev_t(g["ths"], cuda), btn, 0, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    assert tuple(y.shape) == (1, 64, 32, 32) and y.dtype == torch.float32
    assert np.array_equal(y.cpu().numpy(), g["y"].astype(np.float32))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "conv_small_*.npz"))))
def test_conv_small_golden(cuda, path):
    g = np.load(path)
    geom = [int(v) for v in g["geom"]]
    for t, name in enumerate(NAMES):
        y = gpu_conv(cuda, g["x"], g["qw_" + name], g["ths"], g["btn_" + name], t, *geom)
        assert np.array_equal(y, g["y_" + name].astype(np.float32)), name


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("K,p", [(1, 0), (1, 1), (3, 0), (3, 1)])
@pytest.mark.parametrize("s", [1, 2])
def test_conv_grid(cuda, t, K, p, s):
    """types x {1x1,3x3} x stride x pad, over channel counts with and without a tail word and batch sizes."""
    for C in (3, 64, 65, 128, 200, 256):
        for N, H, W, KN in ((1, 6, 6, 4), (3, 9, 5, 70)):
            x, ths = make_input(C + N, N, H, W, C)
            w, wths = make_input(C + N + 1, KN, K, K, C)
            qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
            y = gpu_conv(cuda, x, qw, ths, btn, t, p, p, s, s, N, H, W, C, KN, K, K)
            yo = c_oracle.conv2d(x, qw, ths, btn, t, p, p, s, s, N, H, W, C, KN, K, K)
            assert y.shape == yo.shape and np.array_equal(y, yo), (C, N, H, W, KN)


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("geom", [
    # p1 p2 s1 s2  N   H   W    C   KN KH KW
    (2, 2, 1, 1, 2, 12, 12, 128, 130, 5, 5),
    (3, 3, 2, 2, 1, 15, 13, 64, 20, 7, 7),
    (1, 2, 3, 2, 2, 10, 7, 200, 6, 3, 5),       # non-square everything; stride does not divide
    (0, 0, 1, 1, 1, 2, 2, 64, 8, 3, 3),         # kernel larger than image: empty output
    (1, 1, 1, 1, 5, 13, 11, 64, 257, 3, 3),     # M and KN not multiples of the CTA tile
    (0, 0, 1, 1, 2, 3, 3, 1024, 1024, 1, 1),    # KN = 1024 (impossible on the reference launch shape)
    (1, 1, 1, 1, 1, 4, 4, 4608, 3, 3, 3),       # 72 words per tap
    (0, 0, 2, 3, 2, 11, 10, 128, 70, 1, 1),     # strided 1x1 without padding: only the pixels it reads are quantised
    (0, 0, 2, 2, 3, 14, 14, 256, 512, 1, 1),
    (0, 0, 1, 1, 2, 9, 9, 64, 64, 2, 2),        # 2x2 taps, no padding
])
def test_conv_shapes(cuda, t, geom):
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
    x, ths = make_input(31, N, H, W, C)
    w, wths = make_input(32, KN, KH, KW, C)
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
    y = gpu_conv(cuda, x, qw, ths, btn, t, *geom)
    yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
    assert y.shape == yo.shape and np.array_equal(y, yo)
    yd = O.conv2d_dense(x, qw, ths, t, *geom) if N * H * W * C * KN < 4e7 else yo
    assert np.array_equal(y, yd)


@pytest.mark.parametrize("t", range(4))
def test_selected_path_is_the_one_that_runs(cuda, t, conv_path):
    """The path setting is honoured: the tensor-core kernel reports its tile, the popcount paths report none."""
    N, H, W, C, KN = 4, 14, 14, 256, 96
    x, ths = make_input(5, N, H, W, C)
    w, wths = make_input(6, KN, 3, 3, C)
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, 3, 3, C)
    y = gpu_conv(cuda, x, qw, ths, btn, t, 1, 1, 1, 1, N, H, W, C, KN, 3, 3)
    name = _cabi.lib().tab_last_conv_kernel().decode()
    assert name.startswith("conv_umma_persist_kernel<") if conv_path == "tensor" else name == "none"
    assert np.array_equal(y, c_oracle.conv2d(x, qw, ths, btn, t, 1, 1, 1, 1, N, H, W, C, KN, 3, 3))


RESNET_LAYERS = [
    # H   C   KN  K s p
    (56, 64, 64, 3, 1, 1), (28, 128, 128, 3, 1, 1), (14, 256, 256, 3, 1, 1), (7, 512, 512, 3, 1, 1),
    (56, 64, 128, 3, 2, 1), (28, 128, 256, 3, 2, 1), (14, 256, 512, 3, 2, 1),
]


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("layer", RESNET_LAYERS)
def test_resnet_layers_full_batch_sampled_images(cuda, t, layer):
    """The N=64 ResNet-18-shaped layers at full size on the device; the oracle checks images 0, 37 and 63
    (every image is independent, so a sample of images is an exact check of those outputs)."""
    H, C, KN, K, s, p = layer
    N = 64
    g = torch.Generator(device=cuda)
    g.manual_seed(H * 1000 + C + t)
    x = torch.randn(N, H, H, C, device=cuda, generator=g)
    ths = (0.7 * x.abs().mean(dim=(1, 2, 3))).contiguous()
    w, wths = make_input(H + C, KN, K, K, C)
    qw, btn = TAB.Quantize(dev_t(w, cuda), dev_t(wths, cuda), O.weight_bits(t), KN, K, K, C)
    y = TAB.Conv2d(x, qw, ths, btn, t, p, p, s, s, N, H, H, C, KN, K, K)
    OH = (H + 2 * p - K + 1) // s
    assert tuple(y.shape) == (N, KN, OH, OH)
    yb = y.reshape(N, OH, OH, KN)
    qwh, btnh, thh = qw.cpu().numpy(), btn.cpu().numpy(), ths.cpu().numpy()
    for n in (0, 37, 63):
        yo = c_oracle.conv2d(x[n].cpu().numpy(), qwh, thh[n:n + 1], btnh, t, p, p, s, s, 1, H, H, C, KN, K, K)
        assert np.array_equal(yb[n].cpu().numpy().reshape(-1), yo.reshape(-1)), n
    # sharding property: the first 8 images alone give the same answer as inside the full batch
    y8 = TAB.Conv2d(x[:8].contiguous(), qw, ths[:8].contiguous(), btn, t, p, p, s, s, 8, H, H, C, KN, K, K)
    assert torch.equal(y8.reshape(-1), y.reshape(-1)[:y8.numel()])


@pytest.mark.parametrize("t", [3, 0])
def test_large_1x1_configuration(cuda, t):
    """N=128, 14x14x1024 -> 1024, 1x1 (M=25088, KN=1024, K=1024 bits), types BNN and TNN."""
    N, H, C, KN = 128, 14, 1024, 1024
    g = torch.Generator(device=cuda)
    g.manual_seed(4 + t)
    x = torch.randn(N, H, H, C, device=cuda, generator=g)
    ths = (0.7 * x.abs().mean(dim=(1, 2, 3))).contiguous()
    w, wths = make_input(77, KN, 1, 1, C)
    qw, btn = TAB.Quantize(dev_t(w, cuda), dev_t(wths, cuda), O.weight_bits(t), KN, 1, 1, C)
    y = TAB.Conv2d(x, qw, ths, btn, t, 0, 0, 1, 1, N, H, H, C, KN, 1, 1).reshape(N, -1)
    qwh, btnh, thh = qw.cpu().numpy(), btn.cpu().numpy(), ths.cpu().numpy()
    for n in (0, 64, 127):
        yo = c_oracle.conv2d(x[n].cpu().numpy(), qwh, thh[n:n + 1], btnh, t, 0, 0, 1, 1, 1, H, H, C, KN, 1, 1)
        assert np.array_equal(y[n].cpu().numpy(), yo.reshape(-1))


def test_packed_entry_point_equals_fused_call(cuda):
    N, H, W, C, KN = 3, 9, 8, 130, 33
    x, ths = make_input(1, N, H, W, C)
    w, wths = make_input(2, KN, 3, 3, C)
    for t in range(4):
        qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, 3, 3, C)
        qx, _ = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), O.act_bits(t), N, H, W, C)
        y = TAB.conv2d_packed(qx, dev_t(qw, cuda), dev_t(btn, cuda), t, 1, 1, 2, 1, N, H, W, C, KN, 3, 3)
        yo = c_oracle.conv2d(x, qw, ths, btn, t, 1, 1, 2, 1, N, H, W, C, KN, 3, 3)
        assert np.array_equal(y.cpu().numpy(), yo)


def test_expand_weights(cuda):
    """expand_weights against the de-quantised oracle planes (channel padding 0)."""
    KN, K, C, Cp = 70, 3, 130, 192
    w, wths = make_input(2, KN, K, K, C)
    for wb in (2, 1):
        qw, _ = O.quantize(w, wths, wb, KN, K, K, C)
        w8 = TAB.ops.expand_weights(dev_t(qw, cuda), wb, KN, K, K, C)
        assert tuple(w8.shape) == (KN, K, K, Cp)
        exp_w = np.zeros((KN, K, K, Cp), np.int8)
        exp_w[..., :C] = O.dequantize(qw, C).astype(np.int8)
        assert np.array_equal(w8.cpu().numpy(), exp_w)


@pytest.mark.parametrize("geom", [
    # p1 p2 s1 s2  N  H  W   C   KN KH KW
    (1, 1, 2, 1, 3, 9, 8, 130, 70, 3, 3),
    (1, 2, 1, 1, 3, 9, 8, 130, 70, 3, 3),
    (1, 2, 2, 2, 3, 9, 8, 130, 70, 3, 3),
    (1, 2, 3, 2, 3, 9, 8, 130, 70, 3, 3),
    (0, 0, 2, 2, 5, 14, 14, 64, 128, 1, 1),
    (3, 3, 1, 1, 2, 6, 5, 64, 16, 3, 3),         # padding wider than the kernel reaches: the grid does not share padding
    (0, 0, 1, 1, 2, 9, 9, 200, 300, 3, 3),
    (1, 1, 1, 1, 5, 10, 12, 64, 192, 3, 3),       # filter count a multiple of 64: the grid quantises its own result
    (1, 1, 2, 2, 4, 12, 12, 128, 64, 3, 3),
])
def test_bits_stage_entry_point(cuda, geom):
    """Quantize -> expand_weights -> conv2d_bits (the tensor-core GEMM stage on its own, prepared weights) equals the
    oracle's Conv2d, plain and chained through one state block that every call leaves zeroed."""
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
    x, ths = make_input(7, N, H, W, C)
    w, wths = make_input(8, KN, KH, KW, C)
    state = TAB.ops.new_state(N, cuda)
    for t in range(4):
        ab, wb = O.act_bits(t), O.weight_bits(t)
        qw, btn = O.quantize(w, wths, wb, KN, KH, KW, C)
        qx, _ = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), ab, N, H, W, C)
        w8 = TAB.ops.expand_weights(dev_t(qw, cuda), wb, KN, KH, KW, C)
        yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
        y, nxt = TAB.ops.conv2d_bits(qx, w8, t, *geom)
        assert nxt is None and np.array_equal(y.cpu().numpy(), yo)
        r = torch.round(torch.randn(*yo.shape, device=cuda) * 5)
        y2, nxt = TAB.ops.conv2d_bits(qx, w8, t, *geom, residual=r, threshold_scale=0.7, state=state)
        y2o = yo + r.cpu().numpy()
        assert np.array_equal(y2.cpu().numpy(), y2o)
        assert np.array_equal(nxt.cpu().numpy(), OracleOps.residual_threshold(y2o.copy(), None, 0.7))
        assert not state.any().item()
        # the compact form for chained layers: the same integers as int16, and the quantiser that reads them
        y16, nxt16 = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, out_int16=True)
        assert y16.dtype == torch.int16 and np.array_equal(y16.cpu().numpy().astype(np.float32), yo)
        assert np.array_equal(nxt16.cpu().numpy(), OracleOps.residual_threshold(yo.copy(), None, 0.7))
        OH, OW = yo.shape[2], yo.shape[3]
        if OH * OW:
            for bw in (2, 1):
                # the same launch handing on the quantised result (in the kernel where KN is a multiple of 64, else behind it)
                for kw in (dict(residual=r), dict(out_int16=True)):
                    ya, na, qa = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, next_bitwidth=bw, **kw)
                    yb, nb_ = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, **kw)
                    assert torch.equal(ya, yb) and torch.equal(na, nb_) and not state.any().item()
                    want = (TAB.ops.quantize_i16(yb, nb_, bw, N, OH, OW, KN) if yb.dtype == torch.int16
                            else TAB.Quantize(yb, nb_, bw, N, OH, OW, KN)[0])
                    assert torch.equal(qa.reshape(-1), want.reshape(-1))
                q16 = TAB.ops.quantize_i16(y16, nxt16, bw, N, OH, OW, KN)
                qf, _ = TAB.Quantize(dev_t(yo, cuda), nxt16, bw, N, OH, OW, KN)
                assert torch.equal(q16, qf)
                assert np.array_equal(q16.cpu().numpy(), O.quantize(yo.reshape(N, OH, OW, KN), nxt16.cpu().numpy(), bw, N, OH, OW, KN)[0])
        assert _cabi.lib().tab_device_status() == 0


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("geom", [
    # p1 p2 s1 s2  N   H   W   C   KN KH KW
    (1, 1, 1, 1, 48, 14, 14, 256, 320, 3, 3),    # two filter blocks, the second ragged
    (0, 0, 1, 1, 80, 16, 16, 100, 256, 3, 3),    # no padding, one ragged channel word
    (1, 1, 1, 1, 153, 7, 7, 192, 512, 3, 3),     # odd number of 128-row blocks: the last pair's second CTA has no rows
])
def test_cta_pair_kernel(cuda, t, geom, conv_path):
    """Wide filter blocks with many tiles run on clusters of two CTAs (tcgen05 cta_group::2): plain and with next thresholds
    and 16-bit output, against the oracle; the same shapes with a residual."""
    if conv_path != "tensor":
        pytest.skip("tensor-core path only")
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
    x, ths = make_input(61, N, H, W, C)
    w, wths = make_input(62, KN, KH, KW, C)
    ab, wb = O.act_bits(t), O.weight_bits(t)
    qw, btn = O.quantize(w, wths, wb, KN, KH, KW, C)
    qx, _ = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), ab, N, H, W, C)
    w8 = TAB.ops.expand_weights(dev_t(qw, cuda), wb, KN, KH, KW, C)
    yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
    state = TAB.ops.new_state(N, cuda)
    y, _ = TAB.ops.conv2d_bits(qx, w8, t, *geom)
    assert ",pair>" in _cabi.lib().tab_last_conv_kernel().decode()
    assert np.array_equal(y.cpu().numpy(), yo)
    r = torch.round(torch.randn(*yo.shape, device=cuda) * 5)
    y2, nxt = TAB.ops.conv2d_bits(qx, w8, t, *geom, residual=r, threshold_scale=0.7, state=state)   # (a residual layer runs on single CTAs)
    y2o = yo + r.cpu().numpy()
    assert np.array_equal(y2.cpu().numpy(), y2o)
    assert np.array_equal(nxt.cpu().numpy(), OracleOps.residual_threshold(y2o.copy(), None, 0.7))
    y16, nxt16 = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, out_int16=True)
    assert ",pair>" in _cabi.lib().tab_last_conv_kernel().decode()
    assert y16.dtype == torch.int16 and np.array_equal(y16.cpu().numpy().astype(np.float32), yo)
    assert np.array_equal(nxt16.cpu().numpy(), OracleOps.residual_threshold(yo.copy(), None, 0.7))
    assert not state.any().item()
    # the pairs' grid quantising its own result
    OH, OW = yo.shape[2], yo.shape[3]
    ya, na, qa = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, out_int16=True, next_bitwidth=ab)
    assert ",pair>" in _cabi.lib().tab_last_conv_kernel().decode()
    assert torch.equal(ya, y16) and torch.equal(na, nxt16) and not state.any().item()
    assert np.array_equal(qa.cpu().numpy().reshape(-1), O.quantize(yo.reshape(N, OH, OW, KN), nxt16.cpu().numpy(), ab, N, OH, OW, KN)[0].reshape(-1))
    assert _cabi.lib().tab_device_status() == 0


@pytest.mark.parametrize("t", [0, 3])
@pytest.mark.parametrize("geom", [
    # p1 p2 s1 s2  N   H   W   C   KN KH KW
    (1, 1, 2, 2, 200, 14, 14, 256, 512, 3, 3),   # strided: 200 tiles, a last round of 52
    (0, 0, 2, 2, 200, 14, 14, 256, 512, 1, 1),   # 1x1 stride 2: 154 tiles, a last round of 6
    (1, 1, 1, 1, 200, 7, 7, 128, 512, 3, 3),     # residual layer shape: 200 tiles
    (1, 1, 1, 1, 48, 14, 14, 192, 320, 3, 3),    # ragged filter count: the second half of the last filter block is empty
])
def test_last_round_in_halves(cuda, t, geom, conv_path):
    """A last round of 256-filter tiles that fills at most half of the persistent grid is worked as halves of 128 filters:
    plain, with a residual and next thresholds, and with 16-bit output plus the next layer's quantised input, against the
    oracle."""
    if conv_path != "tensor":
        pytest.skip("tensor-core path only")
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
    x, ths = make_input(71, N, H, W, C)
    w, wths = make_input(72, KN, KH, KW, C)
    ab, wb = O.act_bits(t), O.weight_bits(t)
    qw, btn = O.quantize(w, wths, wb, KN, KH, KW, C)
    qx, _ = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), ab, N, H, W, C)
    w8 = TAB.ops.expand_weights(dev_t(qw, cuda), wb, KN, KH, KW, C)
    yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
    OH, OW = yo.shape[2], yo.shape[3]
    state = TAB.ops.new_state(N, cuda)
    r = torch.round(torch.randn(*yo.shape, device=cuda) * 5)
    y2, nxt = TAB.ops.conv2d_bits(qx, w8, t, *geom, residual=r, threshold_scale=0.7, state=state)
    name = _cabi.lib().tab_last_conv_kernel().decode()
    if torch.cuda.get_device_properties(cuda).multi_processor_count == 148:
        assert " halves" in name and ",pair" not in name, name
    y2o = yo + r.cpu().numpy()
    assert np.array_equal(y2.cpu().numpy(), y2o)
    assert np.array_equal(nxt.cpu().numpy(), OracleOps.residual_threshold(y2o.copy(), None, 0.7))
    if KH * KW == 1 or s1 > 1:                                      # (unit-stride 3x3 layers without a residual run on CTA pairs)
        y, _ = TAB.ops.conv2d_bits(qx, w8, t, *geom)
        assert np.array_equal(y.cpu().numpy(), yo)
        ya, na, qa = TAB.ops.conv2d_bits(qx, w8, t, *geom, threshold_scale=0.7, state=state, out_int16=True, next_bitwidth=ab)
        tn = OracleOps.residual_threshold(yo.copy(), None, 0.7)
        assert ya.dtype == torch.int16 and np.array_equal(ya.cpu().numpy().astype(np.float32), yo) and np.array_equal(na.cpu().numpy(), tn)
        assert np.array_equal(qa.cpu().numpy().reshape(-1), O.quantize(yo.reshape(N, OH, OW, KN), tn, ab, N, OH, OW, KN)[0].reshape(-1))
    assert not state.any().item()
    assert _cabi.lib().tab_device_status() == 0


@pytest.mark.parametrize("t", [0, 3])
@pytest.mark.parametrize("geom", [
    # p1 p2 s1 s2  N   H    W    C   KN KH KW
    (3, 3, 2, 2, 2, 224, 224, 3, 64, 7, 7),      # ResNet stem: 49 taps over four parity planes
    (1, 1, 1, 1, 1, 224, 224, 64, 64, 3, 3),     # wide image: the patch only fits with one row block per tile
    (1, 1, 1, 1, 1, 300, 500, 64, 40, 3, 3),     # wide image: a 1 130-row patch
    (2, 1, 3, 2, 2, 33, 17, 192, 200, 5, 3),     # stride 3 x 2, six parity planes, ragged filter count
    (1, 1, 1, 1, 70, 3, 3, 64, 64, 3, 3),        # 25 grid positions per image: a 32-row slab spans three images
    (0, 0, 1, 1, 2, 28, 28, 128, 1000, 1, 1),    # 1x1, filter count not a multiple of 32
])
def test_large_and_odd_shapes_plain_and_chained(cuda, t, geom):
    """Shapes that steer the dispatch to every branch, as plain Conv2d and as the chained call (residual, |y| sums, next
    thresholds from the GEMM's last CTA)."""
    p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
    x, ths = make_input(41, N, H, W, C)
    w, wths = make_input(42, KN, KH, KW, C)
    qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
    yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
    xd, qd, td, bd = dev_t(x, cuda), dev_t(qw, cuda), dev_t(ths, cuda), dev_t(btn, cuda)
    y = TAB.Conv2d(xd, qd, td, bd, t, *geom)
    assert np.array_equal(y.cpu().numpy(), yo)
    r = torch.round(torch.randn(*yo.shape, device=cuda) * 5)
    y2, nxt = TAB.ops.Conv2dFused(xd, qd, td, bd, t, *geom, r, 0.7)
    y2o = yo + r.cpu().numpy()
    assert np.array_equal(y2.cpu().numpy(), y2o)
    exp = (np.float64(np.float32(0.7)) * (np.abs(y2o).astype(np.float64).reshape(N, -1).sum(1) / y2o[0].size)).astype(np.float32)
    assert np.array_equal(nxt.cpu().numpy(), exp)


def test_shapes_beyond_the_tensor_kernel_fall_back(cuda):
    """A 9x9 kernel on a 300-pixel-wide image needs a patch that does not fit shared memory: the call falls back to the
    popcount kernel and must still be exact; the same kernel on a narrow image stays on the tensor cores."""
    for N, H, W, C, KN, K in ((1, 12, 12, 64, 8, 9), (1, 20, 300, 64, 8, 9)):
        x, ths = make_input(3, N, H, W, C)
        w, wths = make_input(4, KN, K, K, C)
        for t in (0, 3):
            qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, K, K, C)
            y = gpu_conv(cuda, x, qw, ths, btn, t, 4, 4, 1, 1, N, H, W, C, KN, K, K)
            assert np.array_equal(y, c_oracle.conv2d(x, qw, ths, btn, t, 4, 4, 1, 1, N, H, W, C, KN, K, K))


# ------------------------------------------------------------------------------------------ chain

def test_residual_threshold(cuda):
    rng = np.random.default_rng(3)
    for shape in ((3, 5, 4, 4), (2, 7, 3, 3), (4, 64, 7, 7)):
        y = np.round(rng.standard_normal(shape) * 50).astype(np.float32)
        r = np.round(rng.standard_normal(shape) * 50).astype(np.float32)
        yd = dev_t(y, cuda)
        t0 = TAB.ops.residual_threshold(yd, None, 0.7)
        assert np.array_equal(t0.cpu().numpy(), OracleOps.residual_threshold(y.copy(), None, 0.7))
        t1 = TAB.ops.residual_threshold(yd, dev_t(r, cuda), 0.7)
        yo = y.copy()
        to = OracleOps.residual_threshold(yo, r, 0.7)
        assert np.array_equal(yd.cpu().numpy(), yo) and np.array_equal(t1.cpu().numpy(), to)


@pytest.mark.parametrize("bw", [2, 1])
@pytest.mark.parametrize("shape", [(3, 5, 7, 64), (16, 9, 4, 128), (2, 56, 56, 64), (5, 3, 3, 70), (300, 2, 2, 64)])
def test_quantize_auto(cuda, bw, shape):
    """Thresholds scale * mean|x[n]| and the bit-planes against them from one call: the thresholds equal the double-precision
    reference (integer-valued data: every summation order gives the same sum), the bit-planes are the oracle's for those
    thresholds, and the state block comes back zeroed; also with real-valued data against the device's own thresholds."""
    N, H, W, C = shape
    rng = np.random.default_rng(N + C)
    state = TAB.ops.new_state(N, cuda)
    for integer in (True, False):
        x = rng.standard_normal((N, H, W, C)).astype(np.float32)
        if integer:
            x = np.round(x * 40).astype(np.float32)
        for rep in range(2):                                           # twice through the same state block
            qx, ths = TAB.ops.quantize_auto(dev_t(x, cuda), 0.7, bw, N, H, W, C, state)
            t = ths.cpu().numpy()
            if integer:
                assert np.array_equal(t, OracleOps.residual_threshold(x.reshape(N, -1).copy(), None, 0.7))
            else:
                assert np.allclose(t, 0.7 * np.abs(x).reshape(N, -1).mean(1), rtol=1e-6)
            assert np.array_equal(qx.cpu().numpy(), O.quantize(x, t, bw, N, H, W, C)[0])
            assert not state.any().item()
    assert _cabi.lib().tab_device_status() == 0


def test_next_layer_quantisation_with_many_images(cuda):
    """More images than the kernel's second phase keeps thresholds for (8192): the quantiser runs behind the GEMM stage and the
    call returns the same three results."""
    N, H, W, C, KN = 8200, 2, 2, 64, 64
    x, ths = make_input(71, N, H, W, C)
    w, wths = make_input(72, KN, 1, 1, C)
    qw, btn = O.quantize(w, wths, 2, KN, 1, 1, C)
    qx, _ = TAB.Quantize(dev_t(x, cuda), dev_t(ths, cuda), 2, N, H, W, C)
    w8 = TAB.ops.expand_weights(dev_t(qw, cuda), 2, KN, 1, 1, C)
    state = TAB.ops.new_state(N, cuda)
    y, nxt, qn = TAB.ops.conv2d_bits(qx, w8, 0, 0, 0, 1, 1, N, H, W, C, KN, 1, 1, threshold_scale=0.7, state=state, next_bitwidth=2)
    assert "+next" not in _cabi.lib().tab_last_conv_kernel().decode()
    yo = c_oracle.conv2d(x, qw, ths, btn, 0, 0, 0, 1, 1, N, H, W, C, KN, 1, 1)
    assert np.array_equal(y.cpu().numpy(), yo)
    to = OracleOps.residual_threshold(yo.copy(), None, 0.7)
    assert np.array_equal(nxt.cpu().numpy(), to)
    assert np.array_equal(qn.cpu().numpy(), O.quantize(yo.reshape(N, H, W, KN), to, 2, N, H, W, KN)[0])
    assert not state.any().item() and _cabi.lib().tab_device_status() == 0


@pytest.mark.parametrize("C", [64, 70])
def test_quantize_i16_threshold_edge_values(cuda, C):
    """The 16-bit quantiser must agree with the fp32 quantiser (and the oracle) for every kind of threshold: fractions, exact
    integers, negative, zero, beyond the 16-bit range, infinities and NaN - on values that include the extremes and every
    integer around the thresholds."""
    ths = np.array([0.0, -0.0, 0.5, 5.0, 5.5, -3.0, -3.2, 32766.5, 32767.0, 40000.0, -40000.0, 1e30, -1e30, np.inf, -np.inf, np.nan, 1e-30, 7.999999],
                   dtype=np.float32)
    N, H, W = len(ths), 4, 8
    rng = np.random.default_rng(C)
    v = rng.integers(-12, 13, size=(N, H, W, C)).astype(np.int16)
    v[:, 0, 0, :8] = np.array([-32767, 32767, -32766, 32766, 0, 1, -1, 8], dtype=np.int16)
    v[:, 0, 1, :6] = np.array([5, 6, -5, -6, -3, -4], dtype=np.int16)
    vd = torch.from_numpy(v).to(cuda)
    td = torch.from_numpy(ths).to(cuda)
    xf = v.astype(np.float32)
    for bw in (2, 1):
        q16 = TAB.ops.quantize_i16(vd, td, bw, N, H, W, C)
        qf, _ = TAB.Quantize(torch.from_numpy(xf).to(cuda), td, bw, N, H, W, C)
        assert torch.equal(q16, qf)
        assert np.array_equal(q16.cpu().numpy(), O.quantize(xf, ths, bw, N, H, W, C)[0])


def test_fused_conv_matches_unfused(cuda):
    """tab_conv2d_fused_launch: residual and per-image |y| statistics in the epilogue == separate passes."""
    rng = np.random.default_rng(11)
    for geom in ((1, 1, 1, 1, 5, 7, 7, 128, 130, 3, 3), (0, 0, 2, 2, 3, 14, 14, 64, 33, 1, 1), (1, 1, 1, 1, 2, 56, 56, 64, 64, 3, 3)):
        p1, p2, s1, s2, N, H, W, C, KN, KH, KW = geom
        x, ths = make_input(5, N, H, W, C)
        w, wths = make_input(6, KN, KH, KW, C)
        OH, OW = (H + 2 * p1 - KH + 1) // s1, (W + 2 * p2 - KW + 1) // s2
        r = np.round(rng.standard_normal((N, KN, OH, OW)) * 20).astype(np.float32)
        for t in range(4):
            qw, btn = O.quantize(w, wths, O.weight_bits(t), KN, KH, KW, C)
            args = (dev_t(x, cuda), dev_t(qw, cuda), dev_t(ths, cuda), dev_t(btn, cuda), t, *geom)
            yo = c_oracle.conv2d(x, qw, ths, btn, t, *geom)
            y0, n0 = TAB.Conv2dFused(*args, None, None)
            assert n0 is None and np.array_equal(y0.cpu().numpy(), yo)
            y1, t1 = TAB.Conv2dFused(*args, None, 0.7)
            assert np.array_equal(y1.cpu().numpy(), yo)
            assert np.array_equal(t1.cpu().numpy(), OracleOps.residual_threshold(yo.copy(), None, 0.7))
            y2, t2 = TAB.Conv2dFused(*args, dev_t(r, cuda), 0.7)
            yr = yo.copy()
            tr = OracleOps.residual_threshold(yr, r, 0.7)
            assert np.array_equal(y2.cpu().numpy(), yr) and np.array_equal(t2.cpu().numpy(), tr)


@pytest.mark.parametrize("t", [0, 3])
def test_chain_matches_oracle(cuda, t):
    """The 19-convolution ResNet-18-shaped chain, N=3, integer-valued input so that every threshold is an
    exact function of the data on both sides."""
    N = 3
    rng = np.random.default_rng(8)
    x = np.round(rng.standard_normal((N, 56, 56, 64)) * 4).astype(np.float32)
    weights = chain.make_weights(2000, t)
    qo = chain.quantize_weights(weights, t, OracleOps.Quantize)
    ths = OracleOps.residual_threshold(x.copy(), None, chain.THRESHOLD_SCALE)
    yo, oh, ow, kn = chain.forward(OracleOps, x, ths, qo, t, N)
    qd = chain.quantize_weights(weights, t, TAB.Quantize, lambda a: dev_t(a, cuda))
    for k in qo:
        assert np.array_equal(qd[k][0].cpu().numpy(), qo[k][0]) and np.array_equal(qd[k][1].cpu().numpy(), qo[k][1])
    xd = dev_t(x, cuda)
    thd = TAB.ops.residual_threshold(xd, None, chain.THRESHOLD_SCALE)
    assert np.array_equal(thd.cpu().numpy(), ths)
    yd, oh2, ow2, kn2 = chain.forward(TAB.ops, xd, thd, qd, t, N)        # fused epilogues
    assert (oh, ow, kn) == (oh2, ow2, kn2) == (7, 7, 512)
    assert np.array_equal(yd.cpu().numpy().reshape(-1), yo.reshape(-1))

    class Unfused:
        Conv2d = staticmethod(TAB.ops.Conv2d)
        residual_threshold = staticmethod(TAB.ops.residual_threshold)
    yu, _, _, _ = chain.forward(Unfused, xd, thd, qd, t, N)              # separate passes
    assert np.array_equal(yu.cpu().numpy().reshape(-1), yo.reshape(-1))


# ------------------------------------------------------------------------------------------ errors

def test_error_behaviour(cuda):
    x = torch.zeros(1, 4, 4, 64, device=cuda)
    t = torch.zeros(1, device=cuda)
    qw2 = torch.zeros(4, 3, 3, 1, 2, dtype=torch.int64, device=cuda)
    qw1 = torch.zeros(4, 3, 3, 1, 1, dtype=torch.int64, device=cuda)
    btn = torch.zeros(4, dtype=torch.int32, device=cuda)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        TAB.Conv2d(x.cpu(), qw2, t, btn, 0, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        TAB.Conv2d(x.permute(0, 2, 1, 3), qw2, t, btn, 0, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3)
    with pytest.raises(RuntimeError, match="bitwidth 2"):
        TAB.Conv2d(x, qw1, t, btn, 0, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3)       # 1-bit weights given to TNN
    with pytest.raises(RuntimeError, match="type must be"):
        TAB.Conv2d(x, qw2, t, btn, 4, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3)
    l = _cabi.lib()
    y = torch.zeros(64, device=cuda)
    ws = torch.zeros(64, dtype=torch.uint8, device=cuda)          # too small
    rc = l.tab_conv2d_launch(x.data_ptr(), qw2.data_ptr(), t.data_ptr(), btn.data_ptr(), y.data_ptr(), ws.data_ptr(), 64,
                             0, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3, None)
    assert rc == -3
    # after the rejected calls the device path still works
    yy = TAB.Conv2d(x, qw2, t, btn, 0, 1, 1, 1, 1, 1, 4, 4, 64, 4, 3, 3)
    assert not yy.any().item()
