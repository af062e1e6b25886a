"""The TAB_CUDA extension module (the reference-named plugin): surface, dtypes, and equality with the
C-ABI path and the oracle."""
import numpy as np
import pytest
import torch

from oracle import c_oracle, tab_oracle as O
from util import make_input

pytestmark = pytest.mark.gpu


def test_module_surface_and_results(cuda):
    import TAB_CUDA as TAB
    names = [n for n in dir(TAB) if not n.startswith("_")]
    assert {"Conv2d", "Quantize", "TAB_Conv2d", "TAB_Quantize"} <= set(names)
    N, H, W, C, KN, K = 2, 10, 9, 130, 37, 3
    x, ths = make_input(3, N, H, W, C)
    w, wths = make_input(4, KN, K, K, C)
    xd, td = torch.from_numpy(x).to(cuda), torch.from_numpy(ths).to(cuda)
    for t in range(4):
        bw = O.weight_bits(t)
        qw, btn = TAB.Quantize(torch.from_numpy(w).to(cuda), torch.from_numpy(wths).to(cuda), bw, KN, K, K, C)
        qo, bo = O.quantize(w, wths, bw, KN, K, K, C)
        assert qw.dtype == torch.int64 and tuple(qw.shape) == (KN, K, K, 3, bw) and btn.dtype == torch.int32
        assert np.array_equal(qw.cpu().numpy(), qo) and np.array_equal(btn.cpu().numpy(), bo)
        y = TAB.Conv2d(xd, qw, td, btn, t, 1, 1, 1, 1, N, H, W, C, KN, K, K)
        assert y.dtype == torch.float32 and tuple(y.shape) == (N, KN, H, W) and y.is_cuda
        yo = c_oracle.conv2d(x, qo, ths, bo, t, 1, 1, 1, 1, N, H, W, C, KN, K, K)
        assert np.array_equal(y.cpu().numpy(), yo)
    # extension: fused residual + thresholds
    qw, btn = TAB.Quantize(torch.from_numpy(w).to(cuda), torch.from_numpy(wths).to(cuda), 2, KN, K, K, C)
    r = torch.round(torch.randn(N, KN, H, W, device=cuda) * 9)
    y, nxt = TAB.Conv2dFused(xd, qw, td, btn, 0, 1, 1, 1, 1, N, H, W, C, KN, K, K, r, 0.7)
    y_ref = TAB.Conv2d(xd, qw, td, btn, 0, 1, 1, 1, 1, N, H, W, C, KN, K, K) + r
    assert torch.equal(y, y_ref) and tuple(nxt.shape) == (N,)
    exp = (np.float64(np.float32(0.7)) * (y_ref.abs().double().reshape(N, -1).sum(1).cpu().numpy() / (KN * H * W))).astype(np.float32)
    assert np.array_equal(nxt.cpu().numpy(), exp)
    with pytest.raises(RuntimeError, match="X must be a CUDA tensor"):
        TAB.Quantize(torch.from_numpy(x), td, 2, N, H, W, C)
    with pytest.raises(RuntimeError, match="X must be contiguous"):
        TAB.Quantize(xd.permute(0, 2, 1, 3), td, 2, N, H, W, C)


def test_notebook_demo_shapes(cuda):
    """The largest problem the reference's notebook shows: N=16, 112x112x256 -> 64, 3x3, pad 1, stride 1, all
    four types give a float tensor of shape [16, 64, 112, 112]."""
    import TAB_CUDA as TAB
    N, H, W, C, KN, K = 16, 112, 112, 256, 64, 3
    x = torch.rand(N, H, W, C, device=cuda)
    w = torch.rand(KN, K, K, C, device=cuda)
    xt = 0.7 * x.reshape(N, -1).mean(dim=1)
    wt = 0.7 * w.reshape(KN, -1).mean(dim=1)
    for t in range(4):
        qw, btn = TAB.Quantize(w, wt, 1 if t in (1, 3) else 2, KN, K, K, C)
        y = TAB.Conv2d(x, qw, xt, btn, t, 1, 1, 1, 1, N, H, W, C, KN, K, K)
        assert list(y.size()) == [16, 64, 112, 112] and y.dtype == torch.float32
        yo = c_oracle.conv2d(x[5].cpu().numpy(), qw.cpu().numpy(), xt[5:6].cpu().numpy(), btn.cpu().numpy(), t,
                             1, 1, 1, 1, 1, H, W, C, KN, K, K)
        assert np.array_equal(y.reshape(N, -1)[5].cpu().numpy(), yo.reshape(-1))


def test_module_prepared_stages(cuda):
    """ExpandWeights / NewState / Conv2dBits / QuantizeI16 of the module: the GEMM stage on prepared weights, with the next
    thresholds, 16-bit output and the next layer's quantised input from the same call, against the oracle."""
    import TAB_CUDA as TAB
    N, H, W, C, KN, K = 3, 12, 10, 64, 128, 3
    x, ths = make_input(13, N, H, W, C)
    w, wths = make_input(14, KN, K, K, C)
    xd, td = torch.from_numpy(x).to(cuda), torch.from_numpy(ths).to(cuda)
    for t in (0, 3):
        ab, wb = O.act_bits(t), O.weight_bits(t)
        qo, bo = O.quantize(w, wths, wb, KN, K, K, C)
        qw, _ = TAB.Quantize(torch.from_numpy(w).to(cuda), torch.from_numpy(wths).to(cuda), wb, KN, K, K, C)
        w8 = TAB.ExpandWeights(qw, wb, KN, K, K, C)
        qx = TAB.Quantize(xd, td, ab, N, H, W, C)[0]
        yo = c_oracle.conv2d(x, qo, ths, bo, t, 1, 1, 1, 1, N, H, W, C, KN, K, K)
        state = TAB.NewState(qx, N)
        y, nxt = TAB.Conv2dBits(qx, w8, t, 1, 1, 1, 1, N, H, W, C, KN, K, K, None, state, 0.7)
        assert np.array_equal(y.cpu().numpy(), yo)
        to = (np.float64(np.float32(0.7)) * (np.abs(yo).astype(np.float64).reshape(N, -1).sum(1) / yo[0].size)).astype(np.float32)
        assert np.array_equal(nxt.cpu().numpy(), to)
        for nb in (2, 1):
            y16, n16, qn = TAB.Conv2dBits(qx, w8, t, 1, 1, 1, 1, N, H, W, C, KN, K, K, None, state, 0.7, True, nb)
            assert y16.dtype == torch.int16 and np.array_equal(y16.cpu().numpy().astype(np.float32), yo) and torch.equal(n16, nxt)
            want = O.quantize(yo.reshape(N, H, W, KN), to, nb, N, H, W, KN)[0]
            assert np.array_equal(qn.cpu().numpy(), want)
            assert torch.equal(TAB.QuantizeI16(y16.view(N, H, W, KN), n16, nb, N, H, W, KN), qn)
        assert not state.any().item()
