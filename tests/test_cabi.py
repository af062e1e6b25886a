"""The C-ABI library loads and exports every symbol the public header declares; argument validation that
returns before any CUDA call behaves as documented.  No kernel runs here."""
import ctypes
import os
import re

import pytest

from tab_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tab_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tab_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built():
    assert os.path.exists(_cabi.LIB_PATH), "run `python -m tab_b200.build` (or __graft_entry__.build())"


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 9
    raw = ctypes.CDLL(_cabi.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "%s declared in include/tab_b200.h but not exported" % n
        assert n in _cabi.SYMBOLS, "%s has no ctypes prototype in tab_b200/_cabi.py" % n
    for n in _cabi.SYMBOLS:
        assert n in names, "%s bound but not declared in the header" % n
    _cabi.lib()


def test_error_strings_and_version():
    l = _cabi.lib()
    assert l.tab_version() >= 100
    assert l.tab_error_string(0) == b"success"
    for code in (-1, -2, -3, -4, -5, -6):
        assert l.tab_error_string(code) and l.tab_error_string(code) != b"unknown error code"
    assert l.tab_error_string(-99) == b"unknown error code"


def test_argument_validation_without_a_device():
    l = _cabi.lib()
    assert l.tab_quantize_launch(None, None, None, None, 0, 1, 1, 1, 64, None) == -1          # bitwidth < 1
    assert l.tab_quantize_launch(None, None, None, None, 2, -1, 1, 1, 64, None) == -1         # negative N
    assert l.tab_quantize_launch(None, None, None, None, 2, 0, 5, 5, 64, None) == 0           # empty batch
    args = [None] * 6 + [0]
    assert l.tab_conv2d_launch(*args, 7, 1, 1, 1, 1, 1, 8, 8, 64, 4, 3, 3, None) == -1        # type out of range
    assert l.tab_conv2d_launch(*args, 0, 1, 1, 0, 1, 1, 8, 8, 64, 4, 3, 3, None) == -1        # stride 0
    assert l.tab_conv2d_launch(*args, 0, 0, 0, 1, 1, 1, 2, 2, 64, 4, 3, 3, None) == 0         # empty output
    assert l.tab_conv2d_launch(*args, 0, 1, 1, 1, 1, 1, 8, 8, 64, 4, 3, 3, None) == -2        # NULL pointers
    assert l.tab_conv2d_packed_launch(None, None, None, None, 3, 1, 1, 1, 1, 1, 8, 8, 64, 4, 3, 3, None) == -2
    assert l.tab_residual_threshold_launch(None, None, None, None, 0.7, -1, 4, None) == -1


def test_workspace_size():
    l = _cabi.lib()
    # bit-planes of the activations (N*H*W*PC words per plane) + byte weights (KN*KH*KW*PC*64), each rounded up to
    # 256 bytes, + 256 bytes for the completion counter of a chained call
    r = lambda b: (b + 255) // 256 * 256
    assert l.tab_conv2d_workspace_bytes(0, 0, 0, 1, 1, 2, 5, 5, 65, 4, 3, 3) == r(2 * 25 * 2 * 2 * 8) + r(4 * 9 * 128) + 256
    assert l.tab_conv2d_workspace_bytes(3, 1, 1, 1, 1, 2, 5, 5, 65, 4, 3, 3) == r(2 * 25 * 2 * 1 * 8) + r(4 * 9 * 128) + 256
    assert l.tab_conv2d_workspace_bytes(9, 1, 1, 1, 1, 2, 5, 5, 65, 4, 3, 3) == 0
    assert l.tab_conv2d_workspace_bytes(0, 1, 1, 0, 1, 2, 5, 5, 65, 4, 3, 3) == 0
    assert l.tab_conv2d_state_bytes(256) >= 256 * 8 + 4 and l.tab_conv2d_state_bytes(-1) == 0
    assert l.tab_conv2d_set_path(7) == -1
    assert l.tab_conv2d_set_path(2) == 0 and l.tab_conv2d_set_path(0) == 2


def test_static_entry_point_checks_before_any_launch():
    """Return codes of tab_conv2d_static_launch that need no device: a misaligned qw, y or btn is refused like
    tab_conv2d_launch refuses it, and sizes whose product would wrap around are refused, not wrapped."""
    l = _cabi.lib()
    base = 1 << 20                                                  # fake, aligned addresses: nothing dereferences them
    geom = (0, 1, 1, 1, 1, 1, 8, 8, 64, 4, 3, 3)
    for bad in range(5):
        ptrs = [base, base, base, base, base]
        ptrs[bad] += 1
        assert l.tab_conv2d_static_launch(*ptrs, *geom, None) == -6, bad
    big = 2 ** 31 - 1
    assert l.tab_conv2d_static_launch(base, base, base, base, base, 0, 1, 1, 1, 1, big, big, big, big, 4, 3, 3, None) == -5
    assert l.tab_conv2d_static_launch(base, base, base, base, base, 0, 1, 1, 1, 1, 65536, 65536, 4, 64, 4, 3, 3, None) == -5
    assert l.tab_conv2d_bits_launch(base + 1, base, base, *geom, None, None, None, 0.0, None) == -6
    assert l.tab_conv2d_bits_launch(base, base, base, *geom, None, None, base, 0.7, None) == -2     # thresholds need a state block


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", os.path.join(ROOT, "tab_b200", "no_such_lib.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _cabi.lib()
