"""The allocation-free variant of the tensor-core convolution.

Some callers of this library may not allocate device memory at all (they run where cudaMalloc
is forbidden or would stall the GPU, or they are handed only input and output pointers), so
small_b200_conv2d_f32_tf32x3_noalloc keeps its scratch in a fixed array inside the library.
The test drives it through the C ABI twice in a row -- a larger call first, then a smaller one
with other data, so that anything left over in the shared scratch would show -- and compares
each result with the ordinary entry point fed with caller-provided scratch.  Both run the same
kernels on the same numbers, so the outputs must be identical bit for bit.  The file name sorts
last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle.bindings import same_pads
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P

pytestmark = pytest.mark.gpu


def _layer(N, Cn, K, H, W, Fh, Fw, pads, act=0, slope=0.0):
    t, b, l, r = pads
    return _lib.Layer(N, Cn, K, H, W, Fh, Fw, 1, t, b, l, r, 0, act, slope, 0, 0, 0, 0, 0, 0)


def _run_both(rng, N, Cn, K, H, W, Fh, Fw, with_bias):
    import torch
    pads = same_pads(H, W, Fh, Fw, 1)
    x = P.pack_activation(rng.uniform(-1, 1, (N, Cn, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, 0.1, (K, Cn, Fh, Fw)).astype(np.float32))
    bias = rng.uniform(-1, 1, K).astype(np.float32) if with_bias else None
    I, F = S.FloatBuffer(data=x), S.FloatBuffer(data=w)
    B = S.FloatBuffer(data=bias) if with_bias else None
    L = _layer(N, Cn, K, H, W, Fh, Fw, pads, S.ACT_LEAKY if with_bias else S.ACT_NONE, 0.1)
    n_out = N * K * L.out_hw()[0] * L.out_hw()[1]
    st = torch.cuda.current_stream().cuda_stream
    bp = B.ptr() if B is not None else None

    got = S.FloatBuffer(data=np.full(n_out, np.nan, np.float32))
    _lib.check(_lib.lib().small_b200_conv2d_f32_tf32x3_noalloc(C.byref(L), I.ptr(), F.ptr(), bp, got.ptr(), st))

    prep = S.FloatBuffer(2 * F.size())
    want = S.FloatBuffer(data=np.full(n_out, np.nan, np.float32))
    S.prepare_filter_3xTF32(Fh, Fw, K, Cn, F, prep)
    _lib.check(_lib.lib().small_b200_conv2d_f32_tf32x3(C.byref(L), I.ptr(), prep.ptr(), bp, want.ptr(), st))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return got.numpy(), want.numpy()


def test_no_alloc_matches_the_ordinary_entry_point_twice_in_a_row():
    rng = np.random.default_rng(2024)
    got, want = _run_both(rng, 3, 64, 128, 13, 13, 3, 3, with_bias=True)
    assert np.isfinite(want).all() and np.abs(want).max() > 0
    assert np.array_equal(got, want)
    # second call: smaller, different data, same shared scratch
    got, want = _run_both(rng, 1, 32, 32, 9, 7, 1, 1, with_bias=False)
    assert np.isfinite(want).all() and np.abs(want).max() > 0
    assert np.array_equal(got, want)


def test_no_alloc_refuses_what_does_not_fit():
    # two copies of 1024 x 1024 x 3 x 3 filter floats exceed the 4 Mi floats of built-in scratch
    L = _layer(64, 1024, 1024, 13, 13, 3, 3, (1, 1, 1, 1))
    rc = _lib.lib().small_b200_conv2d_f32_tf32x3_noalloc(C.byref(L), None, None, None, None, None)
    assert rc == _lib.INVALID_ARGUMENT
    msg = _lib.lib().small_b200_last_error().decode()
    assert "built-in scratch holds 16777216 bytes" in msg and "needs" in msg
    with pytest.raises(ValueError):
        _lib.check(rc)
