"""uint8 parity of the CUDA path (through the C ABI) against the oracle: BIT-EXACT.

The oracle itself is pinned bit-for-bit to the compiled reference in
tests/test_oracle_reference.py; here it runs with the B200 blocking (16), which for integer
arithmetic gives the same numbers as the reference's blocking of 1
(test_uint8_blocking_invariance)."""
import numpy as np
import pytest

from oracle.bindings import Quant, same_pads, shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, qbuf
from tests.util import sample_window_cases

pytestmark = pytest.mark.gpu


def _out(n, q):
    O = S.QUInt8Buffer(n)
    O.lshift, O.rshift, O.multiplier = q.lshift, q.rshift, q.multiplier
    return O


def _quant(rng, taps_c, zero_points=None):
    """Zero points plus a multiplier / shift that spread the accumulator over 0..255 for a
    reduction of `taps_c` terms of uniform bytes."""
    zi = int(rng.choice([0, -128, 128, 5])); zf = int(rng.choice([-128, 0, 128, -7]))
    if zero_points is not None:
        zi, zf = zero_points
    ma, mw = 127.5 + zi, 127.5 + zf
    var = (74.0 ** 2 + ma ** 2) * (74.0 ** 2 + mw ** 2) - (ma * mw) ** 2
    top = abs(taps_c * ma * mw) + 2.0 * np.sqrt(taps_c * var)
    scale = 255.0 / top                      # = multiplier * 2^-31 * 2^-rshift
    rshift = int(np.clip(np.floor(-np.log2(scale)), 0, 30))
    mult = int(np.clip(scale * 2.0 ** (31 + rshift), 1 << 20, (1 << 31) - 1))
    return Quant(zi, zf, 0, rshift, mult, 0)


CONV_CASES = [
    # C, K, H, W, Fh, Fw, stride, pads, batch
    (64, 64, 25, 5, 1, 1, 1, "valid", 5),     # DS-CNN pointwise
    (1, 64, 49, 10, 10, 4, 2, "same", 3),     # DS-CNN stem (more than one padded row per side)
    (64, 16, 1, 1, 1, 1, 1, "valid", 7),      # DS-CNN dense head (12 padded to 16)
    (16, 32, 9, 11, 3, 3, 1, "same", 2),
    (32, 16, 12, 12, 3, 3, 2, "same", 2),
    (3, 16, 16, 16, 3, 3, 2, "same", 2),
    (128, 128, 6, 6, 1, 1, 1, "valid", 4),
    (16, 16, 7, 5, 5, 3, 1, (2, 2, 1, 1), 1),
    (256, 256, 3, 3, 1, 1, 1, "valid", 3),
]


_case_id = lambda c: "C{}_K{}_{}x{}_k{}x{}_s{}_{}_n{}".format(*[
    "".join(map(str, v)) if isinstance(v, tuple) else v for v in c])


@pytest.mark.parametrize("case", CONV_CASES, ids=_case_id)
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("path", [None, "cuda_cores", "tensor_core"], ids=["auto", "cuda_cores", "tensor_core"])
def test_conv2d_u8(oracle, case, with_bias, path):
    C, K, H, W, Fh, Fw, s, pm, N = case
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    rng = np.random.default_rng(abs(hash((case, with_bias))) % (1 << 31))
    q = _quant(rng, C * Fh * Fw)
    _check_conv(oracle, case, pads, q, rng, with_bias, path)


# Shapes for the implicit-GEMM kernel (every window / stride / padding / channel count on tcgen05
# kind::i8): odd numbers of channel blocks, more than 256 channels, first layers with 1..3 channels,
# windows larger than the image border, stride 2, several pixel tiles, several channel groups.
RING_CASES = [
    (16, 16, 24, 24, 1, 1, 1, "valid", 3),     # one channel block: half of every reduction step is zero
    (48, 32, 10, 7, 1, 1, 1, "valid", 2),      # odd number of blocks
    (512, 64, 5, 5, 1, 1, 1, "valid", 2),      # more channels than the pointwise kernel holds
    (16, 32, 48, 48, 3, 3, 2, "same", 2),      # MobileNet-like stride-2 layer
    (64, 128, 13, 13, 3, 3, 1, "same", 3),
    (32, 48, 9, 14, 5, 5, 1, "same", 2),       # K = 48: tiles of 16 channels
    (32, 192, 6, 6, 3, 3, 1, "same", 2),       # three channel groups of 64
    (3, 16, 96, 96, 3, 3, 2, "same", 2),       # MobileNet stem
    (3, 32, 20, 31, 5, 5, 1, "same", 1),       # first layer, more than two reduction steps
    (2, 16, 11, 9, 3, 3, 1, "valid", 2),
    (1, 16, 30, 30, 7, 7, 2, "same", 2),
    (16, 16, 3, 3, 7, 7, 1, (3, 3, 3, 3), 4),  # every pixel is a border pixel
    (80, 16, 17, 5, 2, 4, 2, "valid", 3),
]
ZERO_POINTS = [(0, -128), (-128, -128), (128, 128), (5, -7), (0, 0), (-128, 0), (3, -128)]


@pytest.mark.parametrize("case", RING_CASES, ids=_case_id)
@pytest.mark.parametrize("zp", ZERO_POINTS, ids=lambda z: "zi{}_zf{}".format(*z))
def test_conv2d_u8_implicit_gemm(oracle, case, zp):
    """Every zero-point class of the tensor-core kernel: shifted operands without correction
    (filter -128, activation 0 / -128), row sums through the extra accumulator columns (filter zero
    point not -128), per-tap channel sums at the border (activation zero point not 0)."""
    C, K, H, W, Fh, Fw, s, pm, N = case
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    rng = np.random.default_rng(abs(hash((case, zp))) % (1 << 31))
    q = _quant(rng, C * Fh * Fw, zp)
    _check_conv(oracle, case, pads, q, rng, True, "tensor_core")


# Reductions of at most 32 bytes (a 1x1 layer on 16 channels, small windows on 1..3 channels) with the
# zero points of the quantised networks run the one-step dp4a kernel; the 3x3x3 window has a path of its
# own (aligned word loads), with the byte path at the left border and at the end of the buffer.
ONESTEP_CASES = [
    (3, 16, 15, 17, 3, 3, 1, "same", 3),
    (3, 16, 96, 96, 3, 3, 2, "same", 2),
    (3, 32, 9, 5, 3, 3, 2, "valid", 2),
    (3, 16, 7, 7, 3, 3, 1, (0, 1, 0, 1), 1),
    (3, 16, 5, 4, 3, 3, 1, "same", 4),
    (3, 16, 3, 3, 3, 3, 1, "valid", 5),      # one output pixel per image: the run ends at the buffer's end
    (16, 16, 24, 24, 1, 1, 1, "valid", 3),
    (16, 16, 9, 9, 1, 1, 2, "valid", 2),
    (2, 16, 11, 9, 3, 3, 1, "valid", 2),
    (1, 16, 8, 8, 5, 5, 1, "same", 2),
    (3, 48, 10, 10, 2, 2, 2, "valid", 2),
]


@pytest.mark.parametrize("case", ONESTEP_CASES, ids=_case_id)
@pytest.mark.parametrize("zp", [(0, -128), (-128, -128)], ids=lambda z: "zi{}_zf{}".format(*z))
def test_conv2d_u8_single_step_reductions(oracle, case, zp):
    C, K, H, W, Fh, Fw, s, pm, N = case
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    rng = np.random.default_rng(abs(hash((case, zp))) % (1 << 31))
    q = _quant(rng, C * Fh * Fw, zp)
    _check_conv(oracle, case, pads, q, rng, True, "cuda_cores")


def _check_conv(oracle, case, pads, q, rng, with_bias, path):
    C, K, H, W, Fh, Fw, s, pm, N = case
    x = P.pack_activation(rng.integers(0, 256, (N, C, H, W)).astype(np.uint8))
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, Fh, Fw)).astype(np.uint8))
    bias = rng.integers(-1024, 1025, K).astype(np.int32) if with_bias else None
    sh = shape(C, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    I, F, O = qbuf(x, q.zero_in), qbuf(w, q.zero_filt), _out(N * K * ho * wo, q)
    if with_bias:
        import torch
        S.Conv2D_Bias_Activation(Fh, Fw, s, *pads, K, C, H, W, I, F,
                                 torch.from_numpy(bias).cuda(), O, batch=N, path=path)
    else:
        S.Conv2D(Fh, Fw, s, *pads, K, C, H, W, I, F, O, batch=N, path=path)
    want = np.stack([oracle.conv2d_u8(sh, q, x[n], w, bias=bias) for n in range(N)])
    got = O.numpy().reshape(N, -1)
    assert _lib.device_status() == 0  # no tensor-core kernel gave up on a bounded wait
    assert np.array_equal(got, want)
    assert want.min() < want.max()  # the case is not degenerate (all clamped)


WIN_CASES = sample_window_cases(np.random.default_rng(33), 16, channels=(16, 64), first_layer=False,
                                max_hw=16)


@pytest.mark.parametrize("c", WIN_CASES, ids=lambda c: "C{}_{}x{}_k{}x{}_s{}_p{}".format(
    *c[:6], "".join(map(str, c[6]))))
def test_depthwise_pools_relu_u8(oracle, c):
    C, H, W, Fh, Fw, s, pads = c
    N = 2
    rng = np.random.default_rng(abs(hash(c)) % (1 << 31))
    q = _quant(rng, Fh * Fw)
    x = P.pack_activation(rng.integers(0, 256, (N, C, H, W)).astype(np.uint8))
    w = P.pack_dw_filter(rng.integers(0, 256, (C, Fh, Fw)).astype(np.uint8))
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    I, F, O = qbuf(x, q.zero_in), qbuf(w, q.zero_filt), _out(N * C * ho * wo, q)
    S.DepthwiseConv2D(Fh, Fw, s, *pads, C, H, W, I, F, O, batch=N)
    want = np.stack([oracle.conv2d_u8(sh, q, x[n], w, depthwise=True) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    qp = Quant(q.zero_in, 0, 0, 1, 1 << 30, 0)  # spreads a + zero over the output range
    O = _out(N * C * ho * wo, qp)
    S.MaxPool2D(Fh, Fw, s, *pads, C, H, W, I, O, batch=N)
    want = np.stack([oracle.pool2d_u8(sh, qp, x[n]) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    qa = Quant(q.zero_in, 0, 0, int(np.ceil(np.log2(Fh * Fw))) + 1, 1 << 30, 0)
    O = _out(N * C * ho * wo, qa)
    S.AveragePool2D(Fh, Fw, min(s, 3), *pads, C, H, W, I, O, batch=N)
    want = np.stack([oracle.pool2d_u8(sh, qa, x[n], average=True) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    O = _out(x.size, qp)
    S.ReLUActivation(C, H, W, I, O, batch=N)
    assert np.array_equal(O.numpy(), oracle.relu_u8(qp, x.ravel()))


def test_default_constructed_buffers_match_the_reference_defaults(oracle):
    """zero 128, multiplier 1077952576, rshift 6 (QUInt8Buffer.hpp:234-272)."""
    b = S.QUInt8Buffer(16)
    assert (b.zero(), b.multiplier, b.lshift, b.rshift) == (128, 1077952576, 0, 6)
    rng = np.random.default_rng(3)
    C, K, H, W = 16, 16, 6, 7
    x = P.pack_activation(rng.integers(0, 256, (C, H, W)).astype(np.uint8))
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, 3, 3)).astype(np.uint8))
    pads = same_pads(H, W, 3, 3, 1)
    I, F, O = S.QUInt8Buffer(data=x), S.QUInt8Buffer(data=w), S.QUInt8Buffer(K * H * W)
    S.Conv2D(3, 3, 1, *pads, K, C, H, W, I, F, O)
    q = Quant(128, 128, 0, 6, 1077952576, 0)
    assert np.array_equal(O.numpy(), oracle.conv2d_u8(shape(C, K, H, W, 3, 3, 1, pads, CB), q, x, w))


def test_full_batch_pointwise_matches_single_images(oracle):
    """DS-CNN pointwise layer at the benchmark's batch (4096): spot-check images against the
    oracle and check that the batched result equals per-image calls."""
    rng = np.random.default_rng(12)
    C = K = 64; H, W, N = 25, 5, 4096
    q = Quant(0, -128, 0, 7, 1400000000, 0)
    x = rng.integers(0, 256, (N, C * H * W)).astype(np.uint8)
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, 1, 1)).astype(np.uint8))
    sh = shape(C, K, H, W, 1, 1, 1, (0, 0, 0, 0), CB)
    I, F, O = qbuf(x, q.zero_in), qbuf(w, q.zero_filt), _out(N * K * H * W, q)
    S.Conv2D(1, 1, 1, 0, 0, 0, 0, K, C, H, W, I, F, O, batch=N)
    got = O.numpy().reshape(N, -1)
    for n in (0, 1, 777, 4095):
        assert np.array_equal(got[n], oracle.conv2d_u8(sh, q, x[n], w))
    O1 = _out(K * H * W, q)
    S.Conv2D(1, 1, 1, 0, 0, 0, 0, K, C, H, W, qbuf(x[2048], q.zero_in), F, O1)
    assert np.array_equal(O1.numpy(), got[2048])


# The dp4a fast paths (filter zero point -128, input zero point 0 or -128) against the oracle.
FAST_DW_CASES = [
    # C, H, W, Fh, Fw, stride, pads
    (64, 25, 5, 3, 3, 1, "same"),        # DS-CNN depthwise
    (16, 9, 12, 3, 3, 2, "same"),
    (32, 11, 7, 5, 5, 1, (2, 2, 2, 2)),  # 25 taps: 7 groups of four, the last one partial
    (48, 6, 6, 2, 2, 1, (0, 1, 0, 1)),
    (16, 8, 8, 1, 1, 1, "valid"),
    (128, 6, 6, 3, 3, 1, "same"),
]


@pytest.mark.parametrize("c", FAST_DW_CASES, ids=lambda c: "C{}_{}x{}_k{}x{}_s{}".format(*c[:6]))
@pytest.mark.parametrize("zero_in", [0, -128])
@pytest.mark.parametrize("with_bias", [False, True])
def test_depthwise_u8_dp4a_path(oracle, c, zero_in, with_bias):
    import torch
    C, H, W, Fh, Fw, s, pm = c
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    N = 3
    rng = np.random.default_rng(abs(hash((c, zero_in, with_bias))) % (1 << 31))
    top = Fh * Fw * 128.0 * 128.0 * 0.6
    rshift = int(np.clip(np.floor(-np.log2(255.0 / top)), 0, 30))
    q = Quant(zero_in, -128, 0, rshift, int(255.0 / top * 2.0 ** (31 + rshift)), 0)
    x = P.pack_activation(rng.integers(0, 256, (N, C, H, W)).astype(np.uint8))
    w = P.pack_dw_filter(rng.integers(0, 256, (C, Fh, Fw)).astype(np.uint8))
    bias = rng.integers(-4096, 4097, C).astype(np.int32) if with_bias else None
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    I, F, O = qbuf(x, zero_in), qbuf(w, -128), _out(N * C * ho * wo, q)
    if with_bias:
        S.DepthwiseConv2D_Bias_Activation(Fh, Fw, s, *pads, C, H, W, I, F, torch.from_numpy(bias).cuda(), O, batch=N)
    else:
        S.DepthwiseConv2D(Fh, Fw, s, *pads, C, H, W, I, F, O, batch=N)
    want = np.stack([oracle.conv2d_u8(sh, q, x[n], w, bias=bias, depthwise=True) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    assert 0 < want.mean() < 255 and want.min() < want.max()


FAST_C1_CASES = [
    # K, H, W, Fh, Fw, stride, pads, batch
    (64, 49, 10, 10, 4, 2, "same", 9),    # DS-CNN stem; 9 images = two full CTAs of 4 and one of 1
    (16, 12, 10, 3, 3, 1, "same", 2),
    (32, 9, 14, 5, 7, 2, "same", 5),      # 7 taps per row: two words, the second partial
    (16, 8, 8, 1, 1, 1, "valid", 1),
    (16, 7, 9, 2, 5, 1, (1, 0, 2, 2), 4),
]


@pytest.mark.parametrize("c", FAST_C1_CASES, ids=lambda c: "K{}_{}x{}_k{}x{}_s{}_n{}".format(*c[:6], c[7]))
@pytest.mark.parametrize("zero_in", [0, -128])
def test_conv2d_u8_one_channel_dp4a_path(oracle, c, zero_in):
    import torch
    K, H, W, Fh, Fw, s, pm, N = c
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    rng = np.random.default_rng(abs(hash((c, zero_in))) % (1 << 31))
    top = Fh * Fw * 128.0 * 128.0 * 0.5
    rshift = int(np.clip(np.floor(-np.log2(255.0 / top)), 0, 30))
    q = Quant(zero_in, -128, 0, rshift, int(255.0 / top * 2.0 ** (31 + rshift)), 0)
    x = P.pack_activation(rng.integers(0, 256, (N, 1, H, W)).astype(np.uint8))
    w = P.pack_conv_filter(rng.integers(0, 256, (K, 1, Fh, Fw)).astype(np.uint8))
    bias = rng.integers(-4096, 4097, K).astype(np.int32)
    sh = shape(1, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    I, F, O = qbuf(x, zero_in), qbuf(w, -128), _out(N * K * ho * wo, q)
    S.Conv2D_Bias_Activation(Fh, Fw, s, *pads, K, 1, H, W, I, F, torch.from_numpy(bias).cuda(), O, batch=N)
    want = np.stack([oracle.conv2d_u8(sh, q, x[n], w, bias=bias) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    assert want.min() < want.max()


@pytest.mark.parametrize("shape_", [(64, 25, 5), (16, 3, 3), (256, 7, 9)])
@pytest.mark.parametrize("zero_in", [0, -128, 7])
def test_global_average_pool_u8(oracle, shape_, zero_in):
    C, H, W = shape_
    N = 5
    rng = np.random.default_rng(C * H + W + zero_in + 1000)
    x = P.pack_activation(rng.integers(0, 256, (N, C, H, W)).astype(np.uint8))
    rshift = int(np.floor(np.log2(H * W)))  # multiplier = 2^(31 + rshift) / taps lies in [2^30, 2^31)
    q = Quant(zero_in, 0, 0, rshift, int(2.0 ** (31 + rshift) / (H * W) * 0.99), 0)
    sh = shape(C, C, H, W, H, W, 1, (0, 0, 0, 0), CB)
    I, O = qbuf(x, zero_in), _out(N * C, q)
    S.AveragePool2D(H, W, 1, 0, 0, 0, 0, C, H, W, I, O, batch=N)
    want = np.stack([oracle.pool2d_u8(sh, q, x[n], average=True) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    assert want.min() < want.max()


PARTIAL_CASES = [
    # C, H, W, Fh, Fw, stride, pads
    (16, 9, 11, 3, 3, 1, "same"),
    (64, 40, 37, 1, 1, 1, "valid"),     # more than one block of 1024 pixels in the in-place pass
    (48, 12, 12, 3, 3, 2, "same"),
    (3, 16, 16, 3, 3, 2, "same"),       # first layer
    (32, 7, 5, 5, 3, 1, (2, 2, 1, 1)),
]


@pytest.mark.parametrize("case", PARTIAL_CASES, ids=lambda c: "C{}_{}x{}_k{}x{}_s{}_{}".format(*[
    "".join(map(str, v)) if isinstance(v, tuple) else v for v in c]))
def test_partial_forms_u8(oracle, case):
    """PartialConv2D / PartialDepthwiseConv2D<quint8>: int32 partial sums waiting at
    the start of the output buffer, 16 output channels, one image -- where the reference's in-buffer
    int32 storage does not overlap itself.  The oracle's form is pinned to the compiled reference in
    tests/test_oracle_reference.py."""
    import torch
    C, H, W, Fh, Fw, s, pm = case
    K = 16
    pads = same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    q = _quant(rng, C * Fh * Fw)
    x = P.pack_activation(rng.integers(0, 256, (1, C, H, W)).astype(np.uint8))
    w = P.pack_conv_filter(rng.integers(0, 256, (K, C, Fh, Fw)).astype(np.uint8))
    sh = shape(C, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    part = rng.integers(-30000, 30000, ho * wo * K).astype(np.int32)
    O = _out(4 * K * ho * wo, q)
    O.data()[:] = torch.from_numpy(part.view(np.uint8)).cuda()
    S.PartialConv2D(Fh, Fw, s, *pads, K, C, H, W, qbuf(x, q.zero_in), qbuf(w, q.zero_filt), O)
    want = oracle.partial_conv2d_u8(sh, q, x[0], w, part)
    assert np.array_equal(O.numpy()[:K * ho * wo], want)
    assert want.min() < want.max()
    if C != 16:
        return
    # depthwise on the same 16 channels
    qd = _quant(rng, Fh * Fw)
    wd = P.pack_dw_filter(rng.integers(0, 256, (C, Fh, Fw)).astype(np.uint8))
    sd = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    partd = rng.integers(-3000, 3000, ho * wo * C).astype(np.int32)
    want = oracle.partial_conv2d_u8(sd, qd, x[0], wd, partd, depthwise=True)
    O = _out(4 * C * ho * wo, qd)
    O.data()[:] = torch.from_numpy(partd.view(np.uint8)).cuda()
    S.PartialDepthwiseConv2D(Fh, Fw, s, *pads, C, H, W, qbuf(x, qd.zero_in), qbuf(wd, qd.zero_filt), O)
    assert np.array_equal(O.numpy()[:C * ho * wo], want)


def test_partial_forms_u8_refuse_overlapping_blocks():
    rng = np.random.default_rng(4)
    x = qbuf(P.pack_activation(rng.integers(0, 256, (1, 16, 6, 6)).astype(np.uint8)), 0)
    w = qbuf(P.pack_conv_filter(rng.integers(0, 256, (32, 16, 1, 1)).astype(np.uint8)), -128)
    O = S.QUInt8Buffer(4 * 32 * 36)
    with pytest.raises(Exception, match="overlap"):
        S.PartialConv2D(1, 1, 1, 0, 0, 0, 0, 32, 16, 6, 6, x, w, O)
    g = qbuf(rng.integers(0, 256, 16 * 16 * 36).astype(np.uint8), 0)
    wg = qbuf(rng.integers(0, 256, 16 * 16 * 16).astype(np.uint8), -128)
    with pytest.raises(Exception, match="overlap"):
        S.PartialGroupConv2D(1, 1, 1, 16, 0, 0, 0, 0, 16, 6, 6, g, wg, S.QUInt8Buffer(4 * 16 * 16 * 36))
