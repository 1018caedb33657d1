"""fp32 parity of the CUDA path (through the C ABI) against the oracle, the reference's
golden vectors and, at benchmark sizes, size-independent properties.

Gate for contractions: max|x - ref| / max|ref| <= 1e-5 against the oracle run with the same
blocking (16), i.e. the same order of additions; the only difference left is fused
multiply-add on the GPU versus separate multiply and add in the reference's REF build.
Pools, ReLU, LeakyReLU, Accum, Bias, UpSample and Concat must be bit-exact."""
import numpy as np
import pytest
import torch

from oracle.bindings import same_pads, shape
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, fbuf, oracle_conv_batch, rel_max_err
from tests.util import (case_id, case_pads, golden_cases, read_bin, reference_close,
                        sample_window_cases)

pytestmark = pytest.mark.gpu
TOL = 1e-5

CONV_CASES = [
    # C, K, H, W, Fh, Fw, stride, pads, batch
    (16, 16, 8, 8, 3, 3, 1, "same", 1),
    (16, 32, 13, 13, 3, 3, 1, "same", 3),
    (32, 64, 26, 20, 3, 3, 1, "same", 2),
    (64, 128, 13, 13, 3, 3, 1, "same", 2),
    (128, 64, 7, 9, 1, 1, 1, "valid", 2),
    (16, 16, 32, 32, 3, 3, 2, "same", 2),
    (32, 64, 16, 16, 1, 1, 2, "valid", 2),
    (16, 48, 9, 17, 5, 3, 1, (2, 2, 1, 1), 1),
    (48, 16, 11, 6, 2, 4, 2, "valid", 2),
    (3, 16, 20, 24, 3, 3, 1, "same", 2),
    (3, 32, 33, 17, 3, 3, 2, "same", 2),
    (1, 16, 12, 10, 3, 3, 1, "same", 1),
    (2, 16, 9, 9, 1, 1, 1, "valid", 1),
    (256, 16, 1, 1, 1, 1, 1, "valid", 4),   # dense head: Conv2D 1x1 on a 1x1 image
    (16, 16, 17, 40, 7, 7, 1, "same", 1),   # falls back to the narrow channel tile
]


def _pads(H, W, Fh, Fw, s, mode):
    if mode == "same":
        return same_pads(H, W, Fh, Fw, s)
    if mode == "valid":
        return (0, 0, 0, 0)
    return mode


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "C{}_K{}_{}x{}_k{}x{}_s{}_{}_n{}".format(*[
    "".join(map(str, v)) if isinstance(v, tuple) else v for v in c]))
@pytest.mark.parametrize("mode", ["plain", "partial", "bias_relu", "bias_leaky"])
def test_conv2d(oracle, case, mode):
    C, K, H, W, Fh, Fw, s, pm, N = case
    pads = _pads(H, W, Fh, Fw, s, pm)
    rng = np.random.default_rng(abs(hash((case, mode))) % (1 << 31))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (C * Fh * Fw)), (K, C, Fh, Fw)).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, K).astype(np.float32)
    sh = shape(C, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    xp, wp = P.pack_activation(x), P.pack_conv_filter(w)
    seed = rng.uniform(-1, 1, (N, K * ho * wo)).astype(np.float32)
    I, F = fbuf(xp), fbuf(wp)
    if mode == "plain":
        O = S.FloatBuffer(N * K * ho * wo)
        S.Conv2D(Fh, Fw, s, *pads, K, C, H, W, I, F, O, batch=N)
        want = oracle_conv_batch(oracle, sh, xp, wp)
    elif mode == "partial":
        O = fbuf(seed)
        S.PartialConv2D(Fh, Fw, s, *pads, K, C, H, W, I, F, O, batch=N)
        want = oracle_conv_batch(oracle, sh, xp, wp, seed=seed)
    else:
        act, slope = (S.ACT_RELU, 0.0) if mode == "bias_relu" else (S.ACT_LEAKY, 0.1)
        O = S.FloatBuffer(N * K * ho * wo)
        S.Conv2D_Bias_Activation(Fh, Fw, s, *pads, K, C, H, W, I, F, fbuf(bias), O,
                                 activation=act, negative_slope=slope, batch=N)
        want = oracle_conv_batch(oracle, sh, xp, wp, bias=bias, act=act, slope=slope)
    got = O.numpy().reshape(N, -1)
    assert rel_max_err(got, want) <= TOL


def test_fused_equals_unfused_chain(oracle):
    """Conv2D_Bias_Activation against the reference's unfused chain Bias -> PartialConv2D ->
    LeakyReLUActivation run through the same library: identical bits."""
    rng = np.random.default_rng(1)
    C, K, H, W, N = 32, 64, 13, 13, 2
    pads = same_pads(H, W, 3, 3, 1)
    x = P.pack_activation(rng.uniform(0, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, 0.05, (K, C, 3, 3)).astype(np.float32))
    b = rng.uniform(-1, 1, K).astype(np.float32)
    I, F, B = fbuf(x), fbuf(w), fbuf(b)
    O1, O2 = S.FloatBuffer(N * K * H * W), S.FloatBuffer(N * K * H * W)
    S.Conv2D_Bias_Activation(3, 3, 1, *pads, K, C, H, W, I, F, B, O1, activation=S.ACT_LEAKY,
                             negative_slope=0.1, batch=N)
    S.Bias(K, H, W, B, O2, batch=N)
    S.PartialConv2D(3, 3, 1, *pads, K, C, H, W, I, F, O2, batch=N)
    S.LeakyReLUActivation(K, H, W, O2, 0.1, O2, batch=N)
    assert np.array_equal(O1.numpy(), O2.numpy())


@pytest.mark.parametrize("tensor_core", [False, True])
@pytest.mark.parametrize("act,slope", [(0, 0.0), (2, 0.1)])
def test_special_values_pass_through_a_convolution(oracle, tensor_core, act, slope):
    """Infinities and NaN in the input reach the output as in the reference, with no activation and
    with LeakyReLU.  Two documented differences are left out: the fused ReLU of a -inf / NaN
    accumulator gives NaN where the reference's separate ReLU pass gives 0, and the 3xTF32 split of an
    infinity is (inf, inf - inf = NaN), so on the tensor-core path infinite inputs give NaN."""
    rng = np.random.default_rng(5)
    C, K, H, W, N = 32, 32, 12, 12, 1
    x = rng.uniform(0.1, 1, (N, C, H, W)).astype(np.float32)
    if not tensor_core:
        x[0, 3, 2, 2] = -np.inf
        x[0, 5, 9, 3] = np.inf
    x[0, 7, 6, 8] = np.nan
    w = np.abs(rng.normal(0, 0.1, (K, C, 1, 1))).astype(np.float32) + 0.01
    bias = rng.uniform(-0.5, 0.5, K).astype(np.float32)
    sh = shape(C, K, H, W, 1, 1, 1, (0, 0, 0, 0), CB)
    xp, wp = P.pack_activation(x), P.pack_conv_filter(w)
    O = S.FloatBuffer(N * K * H * W)
    if tensor_core:
        FP = S.FloatBuffer(2 * wp.size)
        S.prepare_filter_3xTF32(1, 1, K, C, fbuf(wp), FP)
        S.Conv2D_3xTF32(1, 1, 1, 0, 0, 0, 0, K, C, H, W, fbuf(xp), FP, fbuf(bias), O, activation=act,
                        negative_slope=slope, batch=N)
    else:
        S.Conv2D_Bias_Activation(1, 1, 1, 0, 0, 0, 0, K, C, H, W, fbuf(xp), fbuf(wp), fbuf(bias), O,
                                 activation=act, negative_slope=slope, batch=N)
    want = oracle_conv_batch(oracle, sh, xp, wp, bias=bias, act=act, slope=slope)
    got = O.numpy().reshape(N, -1)
    special = ~np.isfinite(want)
    assert special.sum() >= K
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[special & ~np.isnan(want)], want[special & ~np.isnan(want)])
    fin = np.isfinite(want)
    assert rel_max_err(got[fin], want[fin]) <= TOL


def test_conv2d_is_deterministic():
    rng = np.random.default_rng(2)
    C, K, H, W, N = 64, 64, 26, 26, 4
    pads = same_pads(H, W, 3, 3, 1)
    I = fbuf(P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)))
    F = fbuf(P.pack_conv_filter(rng.normal(0, 0.05, (K, C, 3, 3)).astype(np.float32)))
    outs = []
    for _ in range(3):
        O = S.FloatBuffer(N * K * H * W)
        S.Conv2D(3, 3, 1, *pads, K, C, H, W, I, F, O, batch=N)
        outs.append(O.numpy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


@pytest.mark.parametrize("c", [pytest.param(c, id=case_id(c)) for c in golden_cases("conv2d")])
def test_conv2d_golden(c):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    w = read_bin(c["w"]).reshape(c["K"], c["C"], c["k"], c["k"])
    pads = case_pads(c)
    sh = shape(c["C"], c["K"], c["H"], c["W"], c["k"], c["k"], c["s"], pads, CB)
    ho, wo = sh.out_hw()
    y = read_bin(c["y"]).reshape(c["K"], ho, wo)
    O = S.FloatBuffer(c["K"] * ho * wo)
    S.Conv2D(c["k"], c["k"], c["s"], *pads, c["K"], c["C"], c["H"], c["W"],
             fbuf(P.pack_activation(x)), fbuf(P.pack_conv_filter(w)), O)
    assert reference_close(P.unpack_activation(O.numpy(), c["K"], ho, wo), y)


@pytest.mark.parametrize("c", [pytest.param(c, id=case_id(c)) for c in golden_cases("dw_conv")])
def test_dw_conv_golden(c):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    w = read_bin(c["w"]).reshape(c["C"], c["k"], c["k"])
    pads = case_pads(c)
    sh = shape(c["C"], c["C"], c["H"], c["W"], c["k"], c["k"], c["s"], pads, CB)
    ho, wo = sh.out_hw()
    y = read_bin(c["y"]).reshape(c["C"], ho, wo)
    O = S.FloatBuffer(c["C"] * ho * wo)
    S.DepthwiseConv2D(c["k"], c["k"], c["s"], *pads, c["C"], c["H"], c["W"],
                      fbuf(P.pack_activation(x)), fbuf(P.pack_dw_filter(w)), O)
    assert reference_close(P.unpack_activation(O.numpy(), c["C"], ho, wo), y)


@pytest.mark.parametrize("kind", ["maxpool", "averagepool"])
def test_pool_golden(kind):
    for c in golden_cases(kind):
        x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
        pads = case_pads(c)
        sh = shape(c["C"], c["C"], c["H"], c["W"], c["k"], c["k"], c["s"], pads, CB)
        ho, wo = sh.out_hw()
        y = read_bin(c["y"]).reshape(c["C"], ho, wo)
        O = S.FloatBuffer(c["C"] * ho * wo)
        fn = S.MaxPool2D if kind == "maxpool" else S.AveragePool2D
        fn(c["k"], c["k"], c["s"], *pads, c["C"], c["H"], c["W"], fbuf(P.pack_activation(x)), O)
        got = P.unpack_activation(O.numpy(), c["C"], ho, wo)
        if kind == "maxpool":
            assert np.array_equal(got, y), case_id(c)  # test/test_maxpool.cpp:101 compares exactly
        else:
            assert reference_close(got, y), case_id(c)


def test_relu_softmax_partial_bias_golden():
    for c in golden_cases("relu"):
        x, y = read_bin(c["x"]), read_bin(c["y"])
        O = S.FloatBuffer(x.size)
        S.ReLUActivation(c["C"], c["H"], c["W"], fbuf(x), O)
        assert np.array_equal(O.numpy(), y)
    for c in golden_cases("softmax"):
        x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
        y = read_bin(c["y"]).reshape(c["C"], c["H"], c["W"])
        O = S.FloatBuffer(x.size)
        S.SoftMax(c["C"], c["H"], c["W"], fbuf(P.pack_activation(x)), O)
        assert reference_close(P.unpack_activation(O.numpy(), c["C"], c["H"], c["W"]), y)
    for c in golden_cases("partial_bias"):
        x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
        y = read_bin(c["y"]).reshape(c["C"], c["H"], c["W"])
        O = fbuf(P.pack_activation(x))
        S.PartialBias(c["C"], c["H"], c["W"], fbuf(np.arange(c["C"], dtype=np.float32)), O)
        assert reference_close(P.unpack_activation(O.numpy(), c["C"], c["H"], c["W"]), y)


WIN_CASES = sample_window_cases(np.random.default_rng(21), 24, channels=(16, 48), first_layer=False,
                                max_hw=20)


@pytest.mark.parametrize("c", WIN_CASES, ids=lambda c: "C{}_{}x{}_k{}x{}_s{}_p{}".format(
    *c[:6], "".join(map(str, c[6]))))
def test_depthwise_and_pools_vs_oracle(oracle, c):
    C, H, W, Fh, Fw, s, pads = c
    N = 2
    rng = np.random.default_rng(abs(hash(c)) % (1 << 31))
    x = P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_dw_filter(rng.normal(0, 0.3, (C, Fh, Fw)).astype(np.float32))
    bias = rng.uniform(-1, 1, C).astype(np.float32)
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    I = fbuf(x)
    O = S.FloatBuffer(N * C * ho * wo)
    S.DepthwiseConv2D(Fh, Fw, s, *pads, C, H, W, I, fbuf(w), O, batch=N)
    want = oracle_conv_batch(oracle, sh, x, w, depthwise=True)
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= TOL
    S.DepthwiseConv2D_Bias_Activation(Fh, Fw, s, *pads, C, H, W, I, fbuf(w), fbuf(bias), O,
                                      activation=S.ACT_RELU, batch=N)
    want = oracle_conv_batch(oracle, sh, x, w, bias=bias, act=1, depthwise=True)
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= TOL
    S.MaxPool2D(Fh, Fw, s, *pads, C, H, W, I, O, batch=N)
    want = np.stack([oracle.pool2d_f32(sh, x[n]) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    S.AveragePool2D(Fh, Fw, s, *pads, C, H, W, I, O, batch=N)
    want = np.stack([oracle.pool2d_f32(sh, x[n], average=True) for n in range(N)])
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= 1e-6


def test_elementwise_vs_oracle(oracle):
    rng = np.random.default_rng(5)
    N, C, H, W = 3, 32, 7, 5
    x = rng.uniform(-2, 2, (N, C * H * W)).astype(np.float32)
    y = rng.uniform(-2, 2, (N, C * H * W)).astype(np.float32)
    bias = rng.uniform(-1, 1, C).astype(np.float32)
    I = fbuf(x)
    O = S.FloatBuffer(x.size)
    S.ReLUActivation(C, H, W, I, O, batch=N)
    assert np.array_equal(O.numpy(), oracle.relu_f32(x.ravel()))
    S.LeakyReLUActivation(C, H, W, I, fbuf(np.array([0.1], np.float32)), O, batch=N)
    assert np.array_equal(O.numpy(), oracle.leaky_relu_f32(x.ravel(), 0.1))
    O = fbuf(y)
    S.Accum(C, H, W, I, O, batch=N)
    assert np.array_equal(O.numpy(), oracle.accum_f32(x.ravel(), y.ravel()))
    S.Bias(C, H, W, fbuf(bias), O, batch=N)
    assert np.array_equal(O.numpy().reshape(N, -1)[1], oracle.bias_f32(C, H, W, CB, bias))
    O = fbuf(y)
    S.PartialBias(C, H, W, fbuf(bias), O, batch=N)
    assert np.array_equal(O.numpy().reshape(N, -1)[2], oracle.bias_f32(C, H, W, CB, bias, out=y[2]))
    O = S.FloatBuffer(4 * x.size)
    S.UpSample2D(2, C, H, W, I, O, batch=N)
    assert np.array_equal(O.numpy().reshape(N, -1)[1], oracle.upsample2d_f32(C, H, W, CB, 2, x[1]))
    with pytest.raises(ValueError):
        S.UpSample2D(3, C, H, W, I, O)
    O = S.FloatBuffer(x.size)
    S.SoftMax(C, H, W, I, O, batch=N)
    for n in range(N):
        np.testing.assert_allclose(O.numpy().reshape(N, -1)[n], oracle.softmax_f32(C, H, W, CB, x[n]),
                                   rtol=2e-6, atol=0)
    # in-place ReLU, as demo/tinyyolov2.cpp:274-276 uses it
    Z = fbuf(x)
    S.ReLUActivation(C, H, W, Z, Z, batch=N)
    assert np.array_equal(Z.numpy(), oracle.relu_f32(x.ravel()))
    # Concat: two packed buffers become one with the channels appended
    a = rng.uniform(-1, 1, (N, 16, H, W)).astype(np.float32)
    b = rng.uniform(-1, 1, (N, 32, H, W)).astype(np.float32)
    O = S.FloatBuffer(N * 48 * H * W)
    S.Concat(16, 32, H, W, fbuf(P.pack_activation(a)), fbuf(P.pack_activation(b)), O, batch=N)
    got = P.unpack_activation(O.numpy().reshape(N, -1), 48, H, W)
    assert np.array_equal(got, np.concatenate([a, b], axis=1))


def test_errors_match_the_reference():
    """std::invalid_argument cases of interface_abstract.hpp:100, :218 surface as ValueError."""
    I, F, O = S.FloatBuffer(16 * 64), S.FloatBuffer(16 * 16 * 9), S.FloatBuffer(16 * 64)
    with pytest.raises(ValueError, match="stride unsupported"):
        S.Conv2D(3, 3, 3, 0, 0, 0, 0, 16, 16, 8, 8, I, F, O)
    with pytest.raises(ValueError, match="in_channels unsupported"):
        S.Conv2D(3, 3, 1, 0, 0, 0, 0, 16, 5, 8, 8, I, F, O)
    with pytest.raises(ValueError, match="in_channels unsupported"):
        S.MaxPool2D(2, 2, 2, 0, 0, 0, 0, 3, 8, 8, I, O)
    with pytest.raises(ValueError, match="stride unsupported"):
        S.AveragePool2D(2, 2, 4, 0, 0, 0, 0, 16, 8, 8, I, O)
    with pytest.raises(ValueError, match="in_channels unsupported"):
        S.ReLUActivation(8, 2, 2, I, O)


def test_full_size_tiny_yolo_layer_linearity(oracle):
    """A Tiny-YOLOv2 sized layer (128 -> 256 channels at 26x26, batch 8) on the CUDA-core kernel:
    against the oracle for two of the images, plus two properties over the whole batch:
    conv(x1 + x2) = conv(x1) + conv(x2) within fp32 rounding, and every image of a batch equals
    the same image run alone."""
    rng = np.random.default_rng(9)
    C, K, H, W, N = 128, 256, 26, 26, 8
    pads = same_pads(H, W, 3, 3, 1)
    x1 = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
    x2 = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
    wp = P.pack_conv_filter(rng.normal(0, np.sqrt(2 / (C * 9)), (K, C, 3, 3)).astype(np.float32))
    F = fbuf(wp)
    def run(x, n):
        O = S.FloatBuffer(n * K * H * W)
        S.Conv2D(3, 3, 1, *pads, K, C, H, W, fbuf(P.pack_activation(x)), F, O, batch=n)
        return O.numpy().reshape(n, -1)
    y1, y2, y12 = run(x1, N), run(x2, N), run(x1 + x2, N)
    assert rel_max_err(y12, y1 + y2) <= 1e-5
    assert np.array_equal(run(x1[5:6], 1)[0], y1[5])
    sh = shape(C, K, H, W, 3, 3, 1, pads, CB)
    xp = P.pack_activation(x1)
    for n in (0, 7):
        assert rel_max_err(y1[n], oracle.conv2d_f32(sh, xp[n], wp)) <= TOL


FUSED_POOL_CASES = [
    # C, K, H, W, Fh, Fw, conv pads, batch
    (3, 16, 20, 24, 3, 3, "same", 2),     # first layer (HWC image), 4 x 16 accumulators per thread
    (3, 64, 32, 32, 3, 3, "same", 1),
    (1, 32, 12, 10, 3, 3, "same", 2),
    (16, 32, 24, 40, 3, 3, "same", 2),    # staged kernel, 32-channel CTA (Tiny-YOLOv2 conv2 shape class)
    (32, 64, 16, 16, 3, 3, "same", 2),    # staged kernel, 64-channel CTA
    (16, 32, 10, 22, 3, 3, "valid", 1),   # output 8 x 20: tiles that overhang the image
    (16, 64, 18, 18, 1, 1, "valid", 1),
]


@pytest.mark.parametrize("case", FUSED_POOL_CASES, ids=lambda c: "C{}_K{}_{}x{}_k{}x{}_{}_n{}".format(*c))
@pytest.mark.parametrize("mode", ["plain", "bias_relu", "bias_leaky"])
def test_conv2d_maxpool_fused(oracle, case, mode):
    """Conv2D(+bias)(+activation) -> MaxPool2D 2x2 / 2 as ONE kernel (the reference's
    Conv2D_Bias_ReLU_Maxpool2D family, fused_interface_abstract.hpp:463-1418) against the oracle's
    convolution followed by its max pool."""
    C, K, H, W, Fh, Fw, pm, N = case
    pads = _pads(H, W, Fh, Fw, 1, pm)
    rng = np.random.default_rng(abs(hash((case, mode))) % (1 << 31))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (C * Fh * Fw)), (K, C, Fh, Fw)).astype(np.float32)
    bias = None if mode == "plain" else rng.uniform(-0.5, 0.5, K).astype(np.float32)
    act, slope = {"plain": (0, 0.0), "bias_relu": (S.ACT_RELU, 0.0), "bias_leaky": (S.ACT_LEAKY, 0.1)}[mode]
    sh = shape(C, K, H, W, Fh, Fw, 1, pads, CB)
    ho, wo = sh.out_hw()
    shp = shape(K, K, ho, wo, 2, 2, 2, (0, 0, 0, 0), CB)
    assert S.conv2d_maxpool_supported(Fh, Fw, 1, pads, 2, 2, 2, (0, 0, 0, 0), K, C, H, W)
    xp, wp = P.pack_activation(x), P.pack_conv_filter(w)
    O = S.FloatBuffer(N * K * (ho // 2) * (wo // 2))
    S.Conv2D_Bias_Activation_Maxpool2D(Fh, Fw, 1, pads, 2, 2, 2, (0, 0, 0, 0), K, C, H, W, fbuf(xp), fbuf(wp),
                                       None if bias is None else fbuf(bias), O, activation=act,
                                       negative_slope=slope, batch=N)
    got = O.numpy().reshape(N, -1)
    conv = oracle_conv_batch(oracle, sh, xp, wp, bias=bias, act=act, slope=slope)
    want = np.stack([oracle.pool2d_f32(shp, conv[n]) for n in range(N)])
    assert rel_max_err(got, want) <= TOL
    if C >= CB:
        # the staged kernel adds in the same order with or without the pool: bit-identical to
        # the two-kernel path
        mid, two = S.FloatBuffer(N * K * ho * wo), S.FloatBuffer(N * K * (ho // 2) * (wo // 2))
        S.Conv2D_Bias_Activation(Fh, Fw, 1, *pads, K, C, H, W, fbuf(xp), fbuf(wp),
                                 None if bias is None else fbuf(bias), mid, activation=act,
                                 negative_slope=slope, batch=N)
        S.MaxPool2D(2, 2, 2, 0, 0, 0, 0, K, ho, wo, mid, two, batch=N)
        assert np.array_equal(got, two.numpy().reshape(N, -1))


def test_conv2d_maxpool_fused_refuses_other_pools():
    assert not S.conv2d_maxpool_supported(3, 3, 1, (1, 1, 1, 1), 2, 2, 1, (0, 1, 0, 1), 32, 16, 13, 13)  # stride-1 pool
    assert not S.conv2d_maxpool_supported(3, 3, 1, (1, 1, 1, 1), 3, 3, 2, (0, 0, 0, 0), 32, 16, 16, 16)  # 3x3 pool
    assert not S.conv2d_maxpool_supported(3, 3, 1, (1, 1, 1, 1), 2, 2, 2, (0, 0, 0, 0), 32, 16, 13, 13)  # odd output
    assert not S.conv2d_maxpool_supported(3, 3, 2, (0, 1, 0, 1), 2, 2, 2, (0, 0, 0, 0), 32, 16, 16, 16)  # stride-2 conv
    assert not S.conv2d_maxpool_supported(3, 3, 1, (1, 1, 1, 1), 2, 2, 2, (0, 0, 0, 0), 16, 16, 16, 16)  # 16 channels


def test_first_layer_filters_in_constant_memory_slots(oracle):
    """The 3-channel 3x3 first layer with 16 output channels keeps its filter in one of four
    constant-memory slots (one per filter buffer, refreshed on every call); further filter buffers run
    the shared-memory form.  Six filter buffers, each used twice in alternation, all against the oracle."""
    rng = np.random.default_rng(12)
    C, K, H, W, N = 3, 16, 32, 40, 2
    pads = same_pads(H, W, 3, 3, 1)
    sh = shape(C, K, H, W, 3, 3, 1, pads, CB)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    xp = P.pack_activation(x)
    I = fbuf(xp)
    filters = [P.pack_conv_filter(rng.normal(0, 0.2, (K, C, 3, 3)).astype(np.float32)) for _ in range(6)]
    bufs = [fbuf(w) for w in filters]
    want = [oracle_conv_batch(oracle, sh, xp, w, act=1) for w in filters]
    for rep in range(2):
        for w, F, ref in zip(filters, bufs, want):
            O = S.FloatBuffer(N * K * H * W)
            S.Conv2D_ReLU(3, 3, 1, *pads, K, C, H, W, I, F, O, batch=N)
            assert rel_max_err(O.numpy().reshape(N, -1), ref) <= TOL
    # a filter buffer whose contents change between calls: the slot is refreshed every time
    F = bufs[0]
    F.data().copy_(bufs[5].data())
    O = S.FloatBuffer(N * K * H * W)
    S.Conv2D_ReLU(3, 3, 1, *pads, K, C, H, W, I, F, O, batch=N)
    assert rel_max_err(O.numpy().reshape(N, -1), want[5]) <= TOL


@pytest.mark.parametrize("c", [(16, 9, 11, 3, 3, 1, "same"), (64, 12, 12, 3, 3, 2, "same"),
                               (32, 7, 5, 5, 3, 1, (2, 2, 1, 1)), (128, 6, 6, 1, 1, 1, "valid")],
                         ids=lambda c: "C{}_{}x{}_k{}x{}_s{}_{}".format(*[
                             "".join(map(str, v)) if isinstance(v, tuple) else v for v in c]))
def test_partial_depthwise_conv2d_f32(oracle, c):
    """small::PartialDepthwiseConv2D<FloatBuffer> (interface_abstract.hpp:1127): the depthwise
    convolution accumulated onto the existing output."""
    C, H, W, Fh, Fw, s, pm = c
    N = 2
    pads = _pads(H, W, Fh, Fw, s, pm)
    rng = np.random.default_rng(abs(hash(c)) % (1 << 31))
    x = P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_dw_filter(rng.normal(0, 0.3, (C, Fh, Fw)).astype(np.float32))
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    seed = rng.uniform(-1, 1, (N, C * ho * wo)).astype(np.float32)
    O = fbuf(seed)
    S.PartialDepthwiseConv2D(Fh, Fw, s, *pads, C, H, W, fbuf(x), fbuf(w), O, batch=N)
    want = oracle_conv_batch(oracle, sh, x, w, seed=seed, depthwise=True)
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= TOL


@pytest.mark.parametrize("io", [(64, 16, 5), (256, 16, 300), (1024, 32, 7), (3, 16, 4)],
                         ids=lambda v: "in{}_out{}_n{}".format(*v))
def test_dense_wrapper(oracle, io):
    """Dense() = Conv2D 1x1 on a 1x1 image (the way the reference's models build their heads,
    include/small/models/DSCNNTiny.hpp:255-263), at batches that take the CUDA-core kernel and the
    tensor-core kernel with the batch as the pixel axis."""
    cin, cout, N = io
    rng = np.random.default_rng(cin * 7 + cout)
    x = P.pack_activation(rng.uniform(-1, 1, (N, cin, 1, 1)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, 0.1, (cout, cin, 1, 1)).astype(np.float32))
    O = S.FloatBuffer(N * cout)
    S.Dense(cout, cin, fbuf(x), fbuf(w), O, batch=N)
    sh = shape(cin, cout, 1, 1, 1, 1, 1, (0, 0, 0, 0), CB)
    want = oracle_conv_batch(oracle, sh, x, w)
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= TOL
