"""ctypes access to the compiled CPU oracle (``tab_oracle.c``) and, when built, to the reference's own
CPU GEMMs (``oracle/_ref``).  TEST INFRASTRUCTURE ONLY: used by the tests, the smoke check and the
benchmark's CPU-baseline leg, never by the product path."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_GEMM_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_long, C.c_int, C.c_int, C.c_int)
_libs = {}


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def oracle_lib(variant="v3"):
    key = ("oracle", variant)
    if key not in _libs:
        path = os.path.join(HERE, "liboracle_%s.so" % variant)
        if not os.path.exists(path):
            from . import build
            build.build_oracle()
        l = C.CDLL(path)
        l.oracle_quantize.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        l.oracle_quantize.restype = None
        l.oracle_gemm.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_long, C.c_int, C.c_int, C.c_int]
        l.oracle_gemm.restype = None
        l.oracle_pad.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 6
        l.oracle_pad.restype = None
        l.oracle_im2row.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 8
        l.oracle_im2row.restype = None
        l.oracle_conv2d_with.argtypes = [C.c_void_p] * 6 + [C.c_int] * 12
        l.oracle_conv2d_with.restype = C.c_int
        l.oracle_omp_threads.argtypes = [C.c_int]
        l.oracle_omp_threads.restype = C.c_int
        _libs[key] = l
    return _libs[key]


def omp_threads(n=0, variant="v3"):
    """OpenMP threads the CPU pipeline uses (``omp_get_max_threads``); ``n > 0`` sets the count first."""
    return int(oracle_lib(variant).oracle_omp_threads(int(n)))


def ref_available(variant="v3"):
    return os.path.exists(os.path.join(HERE, "_ref", "libtab_ref_%s.so" % variant))


def ref_lib(variant="v3"):
    """The reference's own ``*GEMM_baseline`` / im2row, compiled from its source by ``build.py``."""
    key = ("ref", variant)
    if key not in _libs:
        l = C.CDLL(os.path.join(HERE, "_ref", "libtab_ref_%s.so" % variant))
        l.ref_gemm.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_long, C.c_int, C.c_int, C.c_int]
        l.ref_gemm.restype = None
        l.ref_im2row_3x3.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 8
        l.ref_im2row_3x3.restype = C.c_long
        _libs[key] = l
    return _libs[key]


def quantize(x, ths, bitwidth, N, H, W, Cc, variant="v3"):
    x = np.ascontiguousarray(x, dtype=np.float32)
    ths = np.ascontiguousarray(ths, dtype=np.float32)
    bits = 1 if bitwidth == 1 else 2
    PC = (Cc + 63) // 64
    qx = np.zeros((N, H, W, PC, bits), dtype=np.int64)
    btn = np.zeros(N, dtype=np.int32)
    oracle_lib(variant).oracle_quantize(_ptr(x), _ptr(ths), _ptr(qx), _ptr(btn), bitwidth, N, H, W, Cc)
    return qx, btn


def gemm(a, b, btn, conv_type, M, KN, K, NUM, use_ref=False, variant="v3"):
    a = np.ascontiguousarray(a, dtype=np.int64)
    b = np.ascontiguousarray(b, dtype=np.int64)
    btn = np.ascontiguousarray(btn if btn is not None else np.zeros(KN), dtype=np.int32)
    y = np.zeros((M, KN), dtype=np.int32)
    fn = ref_lib(variant).ref_gemm if use_ref else oracle_lib(variant).oracle_gemm
    fn(_ptr(a), _ptr(b), _ptr(btn), _ptr(y), conv_type, M, KN, K, NUM)
    return y


def conv2d(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, Cc, KN, KH, KW, use_ref_gemm=False, variant="v3"):
    """Whole TAB_Conv2d on the CPU; ``use_ref_gemm`` runs the reference's compiled GEMM in the GEMM stage."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    qw = np.ascontiguousarray(qw, dtype=np.int64)
    ths = np.ascontiguousarray(ths, dtype=np.float32)
    btn = np.ascontiguousarray(btn if btn is not None else np.zeros(max(KN, 1)), dtype=np.int32)
    OH = max((H + 2 * p1 - KH + 1) // s1, 0)
    OW = max((W + 2 * p2 - KW + 1) // s2, 0)
    wb = 1 if conv_type in (1, 3) else 2
    if qw.size != KN * KH * KW * ((Cc + 63) // 64) * wb:
        raise ValueError("QW has %d words, type %d needs %d" % (qw.size, conv_type, KN * KH * KW * ((Cc + 63) // 64) * wb))
    y = np.zeros((N, KN, OH, OW), dtype=np.float32)
    fnp = C.cast(ref_lib(variant).ref_gemm, C.c_void_p) if use_ref_gemm else None
    rc = oracle_lib(variant).oracle_conv2d_with(fnp, _ptr(x), _ptr(qw), _ptr(ths), _ptr(btn), _ptr(y), conv_type,
                                                p1, p2, s1, s2, N, H, W, Cc, KN, KH, KW)
    if rc != 0:
        raise RuntimeError("oracle_conv2d failed with code %d" % rc)
    return y


# ---- the reference's CUDA kernel bodies, executed on the host (oracle/_ref/libtab_ref_cuda.so) -------------

def ref_cuda_available():
    return os.path.exists(os.path.join(HERE, "_ref", "libtab_ref_cuda.so"))


def ref_cuda_lib():
    """``TerOnlyKernel``, ``BinOnlyKernel``, ``BTN_Weight``, ``PadKernel``, ``Img2RowKernel`` and the four ``*GEMM``
    kernels of the reference's ``TAB_GEMM.cu`` / ``.cuh``, compiled for the host by ``build.build_ref_cuda``."""
    key = ("ref_cuda",)
    if key not in _libs:
        l = C.CDLL(os.path.join(HERE, "_ref", "libtab_ref_cuda.so"))
        l.ref_cuda_quantize.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        l.ref_cuda_quantize.restype = None
        l.ref_cuda_pad.argtypes = [C.c_void_p] * 2 + [C.c_int] * 6
        l.ref_cuda_pad.restype = None
        l.ref_cuda_im2row.argtypes = [C.c_void_p] * 2 + [C.c_int] * 8
        l.ref_cuda_im2row.restype = None
        l.ref_cuda_gemm.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        l.ref_cuda_gemm.restype = None
        l.ref_cuda_conv2d.argtypes = [C.c_void_p] * 5 + [C.c_int] * 12
        l.ref_cuda_conv2d.restype = C.c_int
        _libs[key] = l
    return _libs[key]


def ref_cuda_quantize(x, ths, bitwidth, N, H, W, Cc):
    """``QuanWithCuda_TAB``'s kernels.  Like the reference, ``BTN_W`` is computed for the first ``16*(N//16)``
    entries only (the rest stay 0)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ths = np.ascontiguousarray(ths, dtype=np.float32)
    bits = 1 if bitwidth == 1 else 2
    qx = np.zeros((N, H, W, (Cc + 63) // 64, bits), dtype=np.int64)
    btn = np.zeros(N, dtype=np.int32)
    ref_cuda_lib().ref_cuda_quantize(_ptr(x), _ptr(ths), _ptr(qx), _ptr(btn), bitwidth, N, H, W, Cc)
    return qx, btn


def ref_cuda_pad(q, p1, p2):
    """``PadKernel`` on packed activations ``[N,H,W,Cw]`` (any trailing word layout folded into ``Cw``)."""
    q = np.ascontiguousarray(q, dtype=np.int64)
    N, H, W = q.shape[:3]
    Cw = int(np.prod(q.shape[3:]))
    y = np.empty((N, H + 2 * p1, W + 2 * p2) + q.shape[3:], dtype=np.int64)
    ref_cuda_lib().ref_cuda_pad(_ptr(q), _ptr(y), N, H, W, Cw, p1, p2)
    return y


def ref_cuda_im2row(q, KH, KW, s1, s2):
    """``Img2RowKernel`` on (already padded) packed activations ``[N,H,W,Cw]`` -> ``[N*OH*OW, KH*KW*Cw]``."""
    q = np.ascontiguousarray(q, dtype=np.int64)
    N, H, W = q.shape[:3]
    Cw = int(np.prod(q.shape[3:]))
    OH, OW = max((H - KH + 1) // s1, 0), max((W - KW + 1) // s2, 0)
    y = np.zeros((N * OH * OW, KH * KW * Cw), dtype=np.int64)
    ref_cuda_lib().ref_cuda_im2row(_ptr(q), _ptr(y), N, H, W, Cw, KH, KW, s1, s2)
    return y


def ref_cuda_gemm(a, b, btn, conv_type, M, KN, K, NUM):
    a = np.ascontiguousarray(a, dtype=np.int64)
    b = np.ascontiguousarray(b, dtype=np.int64)
    btn = np.ascontiguousarray(btn if btn is not None else np.zeros(max(KN, 1)), dtype=np.int32)
    y = np.zeros((M, KN), dtype=np.float32)
    ref_cuda_lib().ref_cuda_gemm(_ptr(a), _ptr(b), _ptr(btn), _ptr(y), conv_type, M, KN, K, NUM)
    return y


def ref_cuda_conv2d(x, qw, ths, btn, conv_type, p1, p2, s1, s2, N, H, W, Cc, KN, KH, KW):
    """The whole ``ConvWithCuda_TAB`` sequence on the reference's kernels; float32 ``{N,KN,OH,OW}`` label over the
    ``[N][OH][OW][KN]`` buffer, as the reference returns it."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    qw = np.ascontiguousarray(qw, dtype=np.int64)
    ths = np.ascontiguousarray(ths, dtype=np.float32)
    btn = np.ascontiguousarray(btn if btn is not None else np.zeros(max(KN, 1)), dtype=np.int32)
    OH = max((H + 2 * p1 - KH + 1) // s1, 0)
    OW = max((W + 2 * p2 - KW + 1) // s2, 0)
    y = np.zeros((N, KN, OH, OW), dtype=np.float32)
    if y.size:
        rc = ref_cuda_lib().ref_cuda_conv2d(_ptr(x), _ptr(qw), _ptr(ths), _ptr(btn), _ptr(y), conv_type,
                                            p1, p2, s1, s2, N, H, W, Cc, KN, KH, KW)
        if rc != 0:
            raise RuntimeError("ref_cuda_conv2d failed with code %d" % rc)
    return y
