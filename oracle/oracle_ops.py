"""The ``ops`` interface of ``tab_b200.chain`` / ``tab_b200.dp`` implemented with the CPU oracle, on numpy
arrays (and a torch-CPU adapter for the gloo tests).  TEST INFRASTRUCTURE ONLY."""
import numpy as np

from . import c_oracle, tab_oracle as O


class OracleOps:
    @staticmethod
    def Quantize(x, ths, bitwidth, N, H, W, C):
        return list(c_oracle.quantize(x, ths, bitwidth, N, H, W, C))

    @staticmethod
    def Conv2d(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW):
        return c_oracle.conv2d(np.asarray(x).reshape(-1), qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)

    @staticmethod
    def residual_threshold(y, residual=None, scale=0.7):
        N = y.shape[0]
        if residual is not None:
            y += np.asarray(residual, dtype=np.float32).reshape(y.shape)
        per = y.size // N
        s = np.abs(y.astype(np.float64)).reshape(N, -1).sum(axis=1)
        return (np.float64(np.float32(scale)) * (s / np.float64(per))).astype(np.float32)


class OracleOpsFused(OracleOps):
    """Same results through the fused interface (composition of the two oracle steps)."""

    @staticmethod
    def Conv2dFused(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, residual=None, threshold_scale=None):
        y = OracleOps.Conv2d(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
        if threshold_scale is None:
            if residual is not None:
                y += np.asarray(residual, dtype=np.float32).reshape(y.shape)
            return y, None
        return y, OracleOps.residual_threshold(y, residual, threshold_scale)


def torch_cpu_conv(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW):
    """Oracle convolution on torch CPU tensors (stand-in "kernel" for the gloo data-parallel tests)."""
    import torch
    y = c_oracle.conv2d(x.numpy().reshape(-1), qw.numpy(), ths.numpy(), btn.numpy(), conv_type,
                        p1, p2, s1, s2, N, H, W, C, KN, KH, KW)
    return torch.from_numpy(y)


class OraclePreparedConv:
    """Stand-in for ``tab_b200.nn.TABConv2d`` on the CPU oracle: ``quantize`` / ``conv_bits`` with the same meaning."""

    def __init__(self, qw, btn, conv_type, cs):
        self.qw, self.btn, self.t, self.cs = qw, btn, conv_type, cs
        self.conv_type = conv_type

    def quantize(self, x, ths):
        N, H, W = x.shape[:3]
        return (np.ascontiguousarray(x, dtype=np.float32), np.asarray(ths, dtype=np.float32), N, H, W)     # the oracle quantises inside conv2d

    def conv_bits(self, qx, N, H, W, residual=None, next_threshold_scale=None, out_int16=False, next_bitwidth=None):
        x, ths, _, _, _ = qx
        cs = self.cs
        y = c_oracle.conv2d(x.reshape(-1), self.qw, ths, self.btn, self.t, cs.pad, cs.pad, cs.stride, cs.stride, N, H, W, cs.C, cs.KN, cs.K, cs.K)
        y = y.reshape(N, y.shape[2], y.shape[3], y.shape[1])                    # the buffer is [N][OH][OW][KN]
        if next_threshold_scale is None:
            if residual is not None:
                y += np.asarray(residual, dtype=np.float32).reshape(y.shape)
            return y, None
        nxt = OracleOps.residual_threshold(y, residual, next_threshold_scale)
        out = (y.astype(np.int16) if out_int16 and residual is None else y), nxt
        if next_bitwidth is not None:                          # the next layer's "quantised input": (values, thresholds) for the oracle's conv2d
            out = out + ((np.ascontiguousarray(y, dtype=np.float32), nxt, N, y.shape[1], y.shape[2]),)
        return out
