"""Weight preparation of a convolution layer (padding of output channels, packing, batch-normalisation
folding; include/small/Conv2DLayer.hpp:135-341): the oracle against the reference's own function
(compiled in oracle/_ref), and the CUDA kernel against the oracle, bit for bit."""
import ctypes as C

import numpy as np
import pytest

CASES = [
    # Keff, K, C, k, bias, batch norm
    (125, 128, 32, 1, True, True),     # the 125-channel head padded to 128
    (16, 16, 3, 3, False, True),       # first layer, 3 input channels
    (30, 32, 16, 3, True, False),
    (64, 64, 16, 3, False, False),
    (255, 256, 32, 1, False, True),
    (16, 16, 1, 3, True, True),
]


def _params(case):
    Keff, K, Cn, k, bias, bn = case
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    w = rng.normal(0, 1, (Keff, Cn, k, k)).astype(np.float32)
    b = rng.normal(0, 1, Keff).astype(np.float32) if bias else None
    g = [rng.uniform(0.5, 1.5, Keff).astype(np.float32), rng.normal(0, 1, Keff).astype(np.float32),
         rng.normal(0, 1, Keff).astype(np.float32), rng.uniform(0.1, 2, Keff).astype(np.float32)] if bn else None
    return w, b, g


def _reference(lib, K, w, b, g, eps):
    Keff, Cn, k, _ = w.shape
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    z = np.zeros(1, np.float32)
    rf, rb = np.zeros(K * Cn * k * k, np.float32), np.zeros(K, np.float32)
    rc = lib.ref_init_conv2d_buffers(K, Keff, Cn, k, k, p(w), p(b if b is not None else z), Keff if b is not None else 0,
                                     *(p(v) for v in (g if g is not None else [z] * 4)), Keff if g is not None else 0,
                                     C.c_float(eps), p(rf), p(rb))
    assert rc == 0, lib.ref_last_error()
    return rf, rb


@pytest.mark.parametrize("case", CASES, ids=lambda c: "Keff{}_K{}_C{}_k{}_bias{}_bn{}".format(*c))
def test_oracle_matches_the_reference_function(oracle, ref, zen2, case):
    """Packed filters against the reference built with a channel block of 16 (ZEN2); the bias against the
    REF build, whose arithmetic has no fused multiply-add (its block of 1 does not matter for a bias)."""
    Keff, K, Cn, k, _, _ = case
    w, b, g = _params(case)
    pf, pb = oracle.conv_weights_prepare_f32(K, w, b, g, 1e-5)
    rf, _ = _reference(zen2.lib, K, w, b, g, 1e-5)
    assert np.array_equal(pf, rf)
    if pb is not None:
        _, rb = _reference(ref.lib, Keff, w, b, g, 1e-5)
        assert np.array_equal(pb[:Keff], rb[:Keff]) and not pb[Keff:].any()


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=lambda c: "Keff{}_K{}_C{}_k{}_bias{}_bn{}".format(*c))
def test_gpu_weight_preparation_is_bit_identical(oracle, case):
    import torch
    from smallframework_b200 import _lib
    Keff, K, Cn, k, _, _ = case
    w, b, g = _params(case)
    want_f, want_b = oracle.conv_weights_prepare_f32(K, w, b, g, 1e-5)
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    ptr = lambda t: None if t is None else t.data_ptr()
    tw, tb = dev(w), dev(b)
    tg = [dev(v) for v in g] if g is not None else [None] * 4
    pf = torch.full((K * Cn * k * k,), 7.0, device="cuda")
    pb = torch.full((K,), 7.0, device="cuda") if want_b is not None else None
    _lib.check(_lib.lib().small_b200_conv_weights_prepare_f32(K, Keff, Cn, k, k, ptr(tw), ptr(tb), *(ptr(t) for t in tg),
                                                             1e-5, ptr(pf), ptr(pb),
                                                             torch.cuda.current_stream().cuda_stream))
    assert np.array_equal(pf.cpu().numpy(), want_f)
    if want_b is not None:
        assert np.array_equal(pb.cpu().numpy(), want_b)


def test_argument_errors_follow_the_reference():
    from smallframework_b200 import _lib
    l = _lib.lib()
    with pytest.raises(ValueError, match="invalid number of output channels"):
        _lib.check(l.small_b200_conv_weights_prepare_f32(24, 20, 16, 3, 3, None, None, None, None, None, None, 0.0, None, None, None))
    with pytest.raises(ValueError, match="BN buffers"):
        _lib.check(l.small_b200_conv_weights_prepare_f32(16, 16, 16, 3, 3, 1, None, 1, None, None, None, 0.0, 1, 1, None))
