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


def _layer(C_, K, H, W, Fh, Fw, s, pads, N=1):
    t, b, l, r = pads
    return _lib.Layer(N, C_, K, H, W, Fh, Fw, s, t, b, l, r, 0, 0, 0.0, 0, 0, 0, 0, 0, 0)


def test_shape_queries_need_no_gpu():
    """Which shapes the tensor-core convolution and the fused convolution + max pool cover is decided
    on the host (tiling and shared-memory plan), without touching a device."""
    l = _lib.lib()
    tc = lambda *a: bool(l.small_b200_conv2d_f32_tf32x3_supported(ctypes.byref(_layer(*a))))
    assert tc(1024, 1024, 13, 13, 3, 3, 1, (1, 1, 1, 1), 64)      # Tiny-YOLOv2 conv8: rows of the full width
    assert tc(32, 64, 104, 104, 3, 3, 1, (1, 1, 1, 1), 64)        # conv3: TH x TW pixel tiles
    assert tc(16, 32, 416, 416, 3, 3, 1, (1, 1, 1, 1))            # any width
    assert tc(1024, 128, 13, 13, 1, 1, 1, (0, 0, 0, 0))           # pointwise
    assert not tc(16, 32, 32, 32, 3, 3, 2, (0, 1, 0, 1))          # stride 2: CUDA-core kernel
    assert not tc(3, 16, 32, 32, 3, 3, 1, (1, 1, 1, 1))           # first layer
    assert not tc(16, 24, 32, 32, 3, 3, 1, (1, 1, 1, 1))          # 24 output channels: not a multiple of 16
    fused = lambda conv, pool: bool(l.small_b200_conv2d_maxpool_f32_supported(ctypes.byref(conv), ctypes.byref(pool)))
    conv = _layer(3, 16, 416, 416, 3, 3, 1, (1, 1, 1, 1), 4)
    assert fused(conv, _layer(16, 16, 416, 416, 2, 2, 2, (0, 0, 0, 0), 4))
    assert not fused(conv, _layer(16, 16, 416, 416, 2, 2, 1, (0, 1, 0, 1), 4))   # stride-1 pool
    assert not fused(conv, _layer(16, 16, 208, 208, 2, 2, 2, (0, 0, 0, 0), 4))   # pool of another tensor
