"""The bounded device-side waits of the tensor-core kernels: a wait that runs out is reported
once through small_b200_device_status(), the report clears it, and the kernels that follow work.
The wait is made to run out on the host's terms: a self-test kernel polls, with a limit of a few
dozen polls, a barrier nobody arrives on, then frees its tensor memory and returns."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.bindings import same_pads, shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, fbuf, rel_max_err

pytestmark = pytest.mark.gpu


def _conv_ok(oracle):
    rng = np.random.default_rng(5)
    Cn, K, H, W = 32, 128, 13, 13
    pads = same_pads(H, W, 3, 3, 1)
    x = P.pack_activation(rng.uniform(-1, 1, (1, Cn, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, 0.1, (K, Cn, 3, 3)).astype(np.float32))
    prep = S.FloatBuffer(2 * w.size)
    S.prepare_filter_3xTF32(3, 3, K, Cn, fbuf(w), prep)
    O = S.FloatBuffer(K * H * W)
    S.Conv2D_3xTF32(3, 3, 1, *pads, K, Cn, H, W, fbuf(x), prep, None, O)
    torch.cuda.synchronize()
    want = oracle.conv2d_f32(shape(Cn, K, H, W, 3, 3, 1, pads, CB), x[0], w)
    return rel_max_err(O.numpy(), want) <= 1e-5


def test_wait_that_runs_out_is_reported_once_and_cleared(oracle):
    assert _lib.device_status() == 0
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().small_b200_selftest_bounded_wait(48, st))
    v = C.c_int(0)
    rc = _lib.lib().small_b200_device_status(C.byref(v))
    assert rc == _lib.DEVICE_TIMEOUT and v.value == 99
    assert b"bounded device-side wait" in _lib.lib().small_b200_last_error()
    # reported once: the word is clear again, and a tensor-core convolution after it is correct
    assert _lib.device_status() == 0
    assert _conv_ok(oracle)
    assert _lib.device_status() == 0


def test_selftest_rejects_unbounded_limits():
    with pytest.raises(ValueError):
        _lib.check(_lib.lib().small_b200_selftest_bounded_wait(0, None))
    with pytest.raises(ValueError):
        _lib.check(_lib.lib().small_b200_selftest_bounded_wait(1 << 20, None))
