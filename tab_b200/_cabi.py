"""ctypes binding of the C ABI declared in ``include/tab_b200.h`` (``libtab_b200.so``).

The library is built in-tree by ``tab_b200.build``.  There is no CPU fallback: if the shared library
is missing the import of any operator fails with an explicit error.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtab_b200.so")

# name -> (restype, argtypes); must list every symbol include/tab_b200.h declares.
_c = ctypes
SYMBOLS = {
    "tab_error_string": (_c.c_char_p, [_c.c_int]),
    "tab_last_cuda_error": (_c.c_int, []),
    "tab_version": (_c.c_int, []),
    "tab_quantize_launch": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                       _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "tab_conv2d_workspace_bytes": (_c.c_size_t, [_c.c_int] * 12),
    "tab_conv2d_set_path": (_c.c_int, [_c.c_int]),
    "tab_conv2d_launch": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_size_t] + [_c.c_int] * 12 + [_c.c_void_p]),
    "tab_conv2d_fused_launch": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_size_t] + [_c.c_int] * 12 + [_c.c_void_p] * 3),
    "tab_conv2d_chain_launch": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_size_t] + [_c.c_int] * 12 + [_c.c_void_p] * 3 + [_c.c_float, _c.c_void_p]),
    "tab_threshold_from_sums_launch": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_float, _c.c_int, _c.c_longlong, _c.c_void_p]),
    "tab_conv2d_packed_launch": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 12 + [_c.c_void_p]),
    "tab_expand_weights_launch": (_c.c_int, [_c.c_void_p] * 2 + [_c.c_int] * 5 + [_c.c_void_p]),
    "tab_conv2d_state_bytes": (_c.c_size_t, [_c.c_int]),
    "tab_conv2d_bits_launch": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 12 + [_c.c_void_p] * 3 + [_c.c_float, _c.c_void_p]),
    "tab_conv2d_bits_i16_launch": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 12 + [_c.c_void_p] * 2 + [_c.c_float, _c.c_void_p]),
    "tab_conv2d_bits_next_launch": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 13 + [_c.c_void_p] * 3 + [_c.c_float, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "tab_quantize_auto_launch": (_c.c_int, [_c.c_void_p, _c.c_float, _c.c_void_p, _c.c_void_p, _c.c_void_p] + [_c.c_int] * 5 + [_c.c_void_p]),
    "tab_quantize_i16_launch": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 5 + [_c.c_void_p]),
    "tab_last_conv_kernel": (_c.c_char_p, []),
    "tab_device_status": (_c.c_int, []),
    "tab_conv2d_static_launch": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 12 + [_c.c_void_p]),
    "tab_residual_threshold_launch": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_float, _c.c_int, _c.c_longlong, _c.c_void_p]),
    "tab_pipe_probe_sink_bytes": (_c.c_size_t, []),
    "tab_pipe_probe_launch": (_c.c_int, [_c.c_int, _c.c_int, _c.c_void_p, _c.POINTER(_c.c_double), _c.c_void_p]),
}

_lib = None


class TabError(RuntimeError):
    """A C-ABI entry point returned a negative code."""

    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().tab_error_string(code).decode()
        if code == -4:
            msg += " [cudaError %d]" % lib().tab_last_cuda_error()
        super().__init__("%s: %s (code %d)" % (where, msg, code))


def lib() -> ctypes.CDLL:
    """Load ``libtab_b200.so`` once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "tab_b200: %s is missing - build it with `python -m tab_b200.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(l, name)          # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(code: int, where: str) -> None:
    if code != 0:
        raise TabError(code, where)
