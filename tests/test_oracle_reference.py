"""The CPU restatement against the UNMODIFIED reference compiled from its own headers
(oracle/_ref/libsmall_ref.so = REF platform, libsmall_zen2.so = ZEN2 platform).

With the REF blocking (C_ib = C_ob = 1) the restatement keeps the reference's order of
additions and is compiled without FMA contraction, so float results must be
BIT-IDENTICAL; uint8 results must be bit-identical always.  The ZEN2 platform uses
_mm256_fmadd_ps, so there the comparison carries a tolerance.  Shapes are sampled inside
the domain where the reference's own edge kernels are self-consistent
(tests/util.py:axis_defined_in_reference)."""
import numpy as np
import pytest

from oracle.bindings import Quant, same_pads, shape
from smallframework_b200 import packing as P
from tests.util import sample_window_cases

RNG_CASES = sample_window_cases(np.random.default_rng(7), 40)


def _id(c):
    C, H, W, Fh, Fw, s, pads = c
    return f"C{C}_{H}x{W}_k{Fh}x{Fw}_s{s}_p{''.join(map(str, pads))}"


@pytest.mark.parametrize("c", RNG_CASES, ids=_id)
def test_conv2d_f32_bit_exact(oracle, ref, c):
    C, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    K = 32
    x = P.pack_activation(rng.uniform(-1, 1, (C, H, W)).astype(np.float32), 1)
    w = P.pack_conv_filter(rng.normal(0, 0.3, (K, C, Fh, Fw)).astype(np.float32), 1, 1)
    sh = shape(C, K, H, W, Fh, Fw, s, pads, 1)
    assert np.array_equal(oracle.conv2d_f32(sh, x, w), ref.conv2d_f32(sh, x, w))
    seed = rng.uniform(-1, 1, K * sh.out_hw()[0] * sh.out_hw()[1]).astype(np.float32)
    assert np.array_equal(oracle.conv2d_f32(sh, x, w, out=seed), ref.conv2d_f32(sh, x, w, out=seed))


@pytest.mark.parametrize("c", RNG_CASES[:20], ids=_id)
def test_conv2d_f32_zen2_blocking(oracle, zen2, c):
    C, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    K, cb = 32, zen2.float_cb
    x = P.pack_activation(rng.uniform(-1, 1, (C, H, W)).astype(np.float32), cb)
    w = P.pack_conv_filter(rng.normal(0, 0.3, (K, C, Fh, Fw)).astype(np.float32), cb, cb)
    sh = shape(C, K, H, W, Fh, Fw, s, pads, cb)
    np.testing.assert_allclose(oracle.conv2d_f32(sh, x, w), zen2.conv2d_f32(sh, x, w),
                               rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("c", [c for c in RNG_CASES if c[0] >= 16][:20], ids=_id)
def test_dw_and_pools_f32_bit_exact(oracle, ref, c):
    C, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    x = P.pack_activation(rng.uniform(-1, 1, (C, H, W)).astype(np.float32), 1)
    w = P.pack_dw_filter(rng.normal(0, 0.3, (C, Fh, Fw)).astype(np.float32), 1)
    sh = shape(C, C, H, W, Fh, Fw, s, pads, 1)
    assert np.array_equal(oracle.conv2d_f32(sh, x, w, depthwise=True),
                          ref.conv2d_f32(sh, x, w, depthwise=True))
    assert np.array_equal(oracle.pool2d_f32(sh, x), ref.pool2d_f32(sh, x))
    assert np.array_equal(oracle.pool2d_f32(sh, x, average=True), ref.pool2d_f32(sh, x, average=True))


def test_elementwise_f32_bit_exact(oracle, ref):
    rng = np.random.default_rng(3)
    C, H, W = 16, 5, 7
    x = rng.uniform(-2, 2, C * H * W).astype(np.float32)
    y = rng.uniform(-2, 2, C * H * W).astype(np.float32)
    bias = rng.uniform(-1, 1, C).astype(np.float32)
    assert np.array_equal(oracle.relu_f32(x), ref.eltwise_f32("relu", C, H, W, x))
    assert np.array_equal(oracle.leaky_relu_f32(x, 0.1), ref.eltwise_f32("leaky", C, H, W, x, slope=0.1))
    assert np.array_equal(oracle.accum_f32(x, y), ref.eltwise_f32("accum", C, H, W, x, out=y))
    assert np.array_equal(oracle.upsample2d_f32(C, H, W, 1, 2, x), ref.eltwise_f32("upsample", C, H, W, x))
    assert np.array_equal(oracle.bias_f32(C, H, W, 1, bias), ref.bias_f32(C, H, W, bias))
    assert np.array_equal(oracle.bias_f32(C, H, W, 1, bias, out=y), ref.bias_f32(C, H, W, bias, out=y))
    np.testing.assert_allclose(oracle.softmax_f32(C, H, W, 1, x),
                               ref.eltwise_f32("softmax", C, H, W, x), rtol=1e-6, atol=0)


def _quants(rng, n):
    out = []
    for _ in range(n):
        out.append(Quant(int(rng.choice([128, 0, -128, 7])), int(rng.choice([128, 0, -128, -3])),
                         int(rng.choice([0, 0, 1])), int(rng.integers(0, 12)),
                         int(rng.integers(1 << 29, (1 << 31) - 1)), 0))
    return out


@pytest.mark.parametrize("c", RNG_CASES, ids=_id)
def test_uint8_bit_exact(oracle, ref, c):
    _, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    C, K = int(rng.choice([1, 3, 4, 8])), int(rng.choice([2, 5]))
    q = _quants(rng, 1)[0]
    x = P.pack_activation(rng.integers(0, 256, (C, H, W)).astype(np.uint8), 1)
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, Fh, Fw)).astype(np.uint8), 1, 1)
    wd = P.pack_dw_filter(rng.integers(0, 256, (C, Fh, Fw)).astype(np.uint8), 1)
    sh = shape(C, K, H, W, Fh, Fw, s, pads, 1)
    sd = shape(C, C, H, W, Fh, Fw, s, pads, 1)
    assert np.array_equal(oracle.conv2d_u8(sh, q, x, w), ref.conv2d_u8(sh, q, x, w))
    assert np.array_equal(oracle.conv2d_u8(sd, q, x, wd, depthwise=True),
                          ref.conv2d_u8(sd, q, x, wd, depthwise=True))
    assert np.array_equal(oracle.pool2d_u8(sd, q, x), ref.maxpool2d_u8(sd, q, x))
    assert np.array_equal(oracle.relu_u8(q, x), ref.relu_u8(C, H, W, q, x))


@pytest.mark.parametrize("c", RNG_CASES[:24], ids=_id)
def test_uint8_partial_forms_bit_exact(oracle, ref, c):
    """PartialConv2D / PartialDepthwiseConv2D<QUInt8Buffer>: int32 partial sums waiting in the output
    buffer, one block of output channels (the reference build's block is one channel, so K = 1 and a
    one-channel depthwise layer)."""
    _, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    C = int(rng.choice([1, 3, 4, 8]))
    q = _quants(rng, 1)[0]
    x = P.pack_activation(rng.integers(0, 256, (C, H, W)).astype(np.uint8), 1)
    w = P.pack_conv_filter(rng.integers(0, 256, (1, C, Fh, Fw)).astype(np.uint8), 1, 1)
    sh = shape(C, 1, H, W, Fh, Fw, s, pads, 1)
    ho, wo = sh.out_hw()
    part = rng.integers(-40000, 40000, ho * wo).astype(np.int32)
    got, want = oracle.partial_conv2d_u8(sh, q, x, w, part), ref.partial_conv2d_u8(sh, q, x, w, part)
    assert np.array_equal(got, want)
    x1 = x[:H * W]
    wd = P.pack_dw_filter(rng.integers(0, 256, (1, Fh, Fw)).astype(np.uint8), 1)
    sd = shape(1, 1, H, W, Fh, Fw, s, pads, 1)
    assert np.array_equal(oracle.partial_conv2d_u8(sd, q, x1, wd, part, depthwise=True),
                          ref.partial_conv2d_u8(sd, q, x1, wd, part, depthwise=True))


def test_uint8_default_quantisation(oracle, ref):
    """Buffers as the reference constructs them: zero 128, multiplier 1077952576,
    rshift 6 (QUInt8Buffer.hpp:234-272)."""
    rng = np.random.default_rng(11)
    q = Quant(128, 128, 0, 6, 1077952576, 0)
    C, K, H, W = 4, 2, 4, 5
    x = P.pack_activation(rng.integers(0, 256, (C, H, W)).astype(np.uint8), 1)
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, 3, 3)).astype(np.uint8), 1, 1)
    sh = shape(C, K, H, W, 3, 3, 1, same_pads(H, W, 3, 3, 1), 1)
    assert np.array_equal(oracle.conv2d_u8(sh, q, x, w), ref.conv2d_u8(sh, q, x, w))


def test_uint8_blocking_invariance(oracle):
    """The packed result must not depend on the channel block (REF 1, B200 16)."""
    rng = np.random.default_rng(5)
    C, K, H, W = 32, 16, 9, 6
    q = Quant(-128, -128, 0, 9, 1518500250, 0)
    x = rng.integers(0, 256, (C, H, W)).astype(np.uint8)
    w = rng.integers(0, 256, (K, C, 3, 3)).astype(np.uint8)
    outs = []
    for cb in (1, 16):
        sh = shape(C, K, H, W, 3, 3, 2, same_pads(H, W, 3, 3, 2), cb)
        ho, wo = sh.out_hw()
        y = oracle.conv2d_u8(sh, q, P.pack_activation(x, cb), P.pack_conv_filter(w, cb, cb))
        outs.append(P.unpack_activation(y, K, ho, wo, cb))
    assert np.array_equal(outs[0], outs[1])
    assert outs[0].min() < outs[0].max()


def test_requant_known_values(oracle):
    """Hand-checked values of the fixed-point tail (intrinsics_quint8.h:481-531): the
    rounding shift SUBTRACTS one when the remainder exceeds the threshold."""
    m = 1 << 30  # multiplier 0.5
    assert oracle.requant(200, 0, 0, m) == 100
    assert oracle.requant(201, 0, 0, m) == 101  # nudge rounds half up
    assert oracle.requant(4000, 0, 2, m) == 255  # clamp
    assert oracle.requant(-5, 0, 0, m) == 0
    # hi = 100 -> mask 3, mod 0 -> 100>>2 = 25; hi = 103 -> mod 3 > 1 -> 25 - 1 = 24
    assert oracle.requant(200, 0, 2, m) == 25
    assert oracle.requant(206, 0, 2, m) == 24
