"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from smallframework_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "small_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(small_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    assert "small_b200_conv2d_f32" in names and "small_b200_conv2d_u8" in names
    assert len(names) >= 35


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from smallframework_b200.build import build
        build()
    l = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared() if not hasattr(l, n)]
    assert not missing, missing


def test_binding_covers_the_header():
    assert sorted(_lib.exported_names()) == _declared()


def test_argument_errors_need_no_gpu():
    """Argument validation happens on the host before any CUDA call, with the reference's
    messages (interface_abstract.hpp:100, :218)."""
    l = _lib.lib()
    L = _lib.Layer(1, 16, 16, 8, 8, 3, 3, 3, 0, 0, 0, 0, 0, 0, 0.0, 0, 0, 0, 0, 0, 0)
    assert l.small_b200_conv2d_f32(ctypes.byref(L), None, None, None, None, None) == _lib.INVALID_ARGUMENT
    assert b"stride unsupported" in l.small_b200_last_error()
    L.stride = 1
    L.C = 5
    assert l.small_b200_conv2d_f32(ctypes.byref(L), None, None, None, None, None) == _lib.INVALID_ARGUMENT
    assert b"in_channels unsupported" in l.small_b200_last_error()
    with pytest.raises(ValueError):
        _lib.check(_lib.INVALID_ARGUMENT)
