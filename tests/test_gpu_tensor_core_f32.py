"""fp32 convolution on the tensor cores (tcgen05 kind::tf32, 3xTF32 split) against the oracle:
max|x - ref| / max|ref| <= 1e-5, the same gate as the CUDA-core kernel."""
import numpy as np
import pytest

from oracle.bindings import same_pads, shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, fbuf, oracle_conv_batch, rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-5

CASES = [
    # C, K, H, W, Fh, Fw, pads, batch
    (16, 16, 13, 13, 3, 3, "same", 1),      # one 16-channel block, 128+64-row tiles
    (32, 64, 13, 13, 3, 3, "same", 2),
    (64, 256, 13, 13, 3, 3, "same", 2),     # 256 output channels per CTA: all of tensor memory
    (32, 128, 26, 26, 3, 3, "same", 2),     # several M tiles per image
    (32, 32, 52, 52, 3, 3, "same", 1),
    (16, 64, 104, 104, 3, 3, "same", 1),
    (128, 128, 13, 13, 1, 1, "valid", 3),   # pointwise: no junk columns
    (32, 16, 9, 20, 5, 3, (2, 2, 1, 1), 1),
    (48, 32, 11, 7, 2, 4, "valid", 2),
    (32, 48, 8, 8, 3, 3, (0, 1, 0, 1), 2),  # unequal pads
    (512, 128, 13, 13, 3, 3, "same", 1),    # long reduction: 32 channel blocks
    (1024, 128, 13, 13, 3, 3, "same", 1),   # the longest reduction of the configurations (9216 terms)
    (1024, 128, 13, 13, 1, 1, "valid", 2),
    # pointwise layers fetch their patches with plain asynchronous copies: several pixel tiles per
    # image with a partial last one, a plane smaller than a patch, many tiles per CTA
    (256, 256, 26, 26, 1, 1, "valid", 2),
    (64, 128, 7, 5, 1, 1, "valid", 5),
    (32, 144, 13, 13, 1, 1, "valid", 160),
    # pointwise layers on small images: the batch becomes the rows of one image, tiles run across images
    (128, 256, 3, 3, 1, 1, "valid", 37),
    (64, 128, 6, 6, 1, 1, "valid", 10),
    (32, 64, 4, 4, 1, 1, "valid", 70),
    (48, 32, 8, 8, 1, 1, "valid", 3),
    (256, 128, 1, 1, 1, 1, "valid", 300),
    # wide images: TH x TW pixel tiles (partial tiles at the right and bottom edges)
    (16, 32, 40, 130, 3, 3, "same", 2),
    (32, 64, 70, 90, 3, 3, "same", 1),
    (16, 16, 9, 300, 1, 1, "valid", 1),
    (32, 48, 33, 75, 5, 3, (2, 2, 1, 1), 1),
    (16, 32, 50, 64, 3, 3, "valid", 2),
    # small tiles: four accumulator buffers in tensor memory (128 or 64 pixels per tile)
    (32, 128, 8, 8, 3, 3, "same", 3),
    (64, 256, 6, 6, 3, 3, "same", 2),
    (32, 144, 10, 10, 3, 3, "same", 2),     # partial last channel tile (16 of 128 rows)
    # 32 or 64 output channels: pixels on the tensor core's M (one or two blocks of 128 pixels)
    (16, 32, 8, 8, 3, 3, "same", 5),
    (256, 64, 13, 13, 3, 3, "same", 2),
    (32, 64, 26, 26, 1, 1, "valid", 2),
    (48, 32, 20, 20, 5, 5, (2, 2, 2, 2), 1),
    # 16 output channels: the narrowest MMA (N = 16), 16-column accumulator buffers
    (16, 16, 32, 32, 3, 3, "same", 4),
    (32, 16, 13, 13, 3, 3, "same", 3),
    (64, 16, 8, 8, 1, 1, "valid", 9),
    (256, 16, 1, 1, 1, 1, "valid", 500),
    # pixel-major persistent tiles whose whole filter stays in shared memory (one stage per group of a
    # tile: 1, 3, 5 and 6 stages), with more tiles than CTAs, so that every issuing thread meets stages
    # another thread used first
    (16, 16, 26, 26, 1, 1, "valid", 96),
    (48, 32, 26, 26, 1, 1, "valid", 64),
    (80, 64, 20, 20, 1, 1, "valid", 64),
    (16, 32, 32, 32, 3, 3, "same", 48),
    (32, 64, 26, 26, 3, 3, "same", 48),
    # 64 output channels, two blocks of 128 pixels per tile: two accumulator buffers of 256 columns and two
    # issuing threads, more tiles than CTAs (buffer phases run on over many groups)
    (32, 64, 104, 104, 3, 3, "same", 4),
    (64, 64, 20, 20, 3, 3, "same", 80),
    # one 16-channel block, 16 / 32 output channels: the whole window is one group (2x3, 3x1 and 1x3 windows too)
    (16, 32, 20, 24, 2, 3, "valid", 3),
    (16, 16, 30, 18, 3, 1, (1, 1, 0, 0), 40),
    (16, 32, 18, 90, 1, 3, (0, 0, 1, 1), 2),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "C{}_K{}_{}x{}_k{}x{}_{}_n{}".format(*[
    "".join(map(str, v)) if isinstance(v, tuple) else v for v in c]))
@pytest.mark.parametrize("mode", ["plain", "partial_bias_leaky"])
def test_conv2d_3xtf32(oracle, case, mode):
    C, K, H, W, Fh, Fw, pm, N = case
    pads = same_pads(H, W, Fh, Fw, 1) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    assert S.tf32x3_supported(Fh, Fw, 1, *pads, K, C, H, W)
    rng = np.random.default_rng(abs(hash((case, mode))) % (1 << 31))
    x = P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, np.sqrt(2.0 / (C * Fh * Fw)), (K, C, Fh, Fw)).astype(np.float32))
    bias = rng.uniform(-0.5, 0.5, K).astype(np.float32)
    sh = shape(C, K, H, W, Fh, Fw, 1, pads, CB)
    ho, wo = sh.out_hw()
    I, F = fbuf(x), fbuf(w)
    Fp = S.FloatBuffer(2 * F.size())
    S.prepare_filter_3xTF32(Fh, Fw, K, C, F, Fp)
    if mode == "plain":
        O = S.FloatBuffer(N * K * ho * wo)
        S.Conv2D_3xTF32(Fh, Fw, 1, *pads, K, C, H, W, I, Fp, None, O, batch=N)
        want = oracle_conv_batch(oracle, sh, x, w)
    else:
        seed = rng.uniform(-1, 1, (N, K * ho * wo)).astype(np.float32)
        O = fbuf(seed)
        S.Conv2D_3xTF32(Fh, Fw, 1, *pads, K, C, H, W, I, Fp, fbuf(bias), O, partial=True,
                        activation=S.ACT_LEAKY, negative_slope=0.1, batch=N)
        want = oracle_conv_batch(oracle, sh, x, w, bias=bias, act=2, slope=0.1, seed=seed)
    got = O.numpy().reshape(N, -1)
    assert _lib.device_status() == 0
    assert rel_max_err(got, want) <= TOL


POOLED_CASES = [
    # C, K, H, W, Fh, Fw, pads, batch: images wider than 64 pixels, even output sizes
    (16, 32, 40, 130, 3, 3, "same", 2),    # merged-operand kernel, partial tiles at the right edge
    (32, 64, 70, 90, 3, 3, "same", 2),     # 64 output channels
    (16, 32, 208, 208, 3, 3, "same", 1),   # Tiny-YOLOv2 conv2 + maxpool2: more tiles than CTAs
    (32, 64, 104, 104, 3, 3, "same", 3),   # conv3 + maxpool3
    (16, 32, 12, 100, 1, 1, "valid", 2),
    (32, 32, 52, 68, 5, 3, (2, 2, 1, 1), 1),
]


@pytest.mark.parametrize("case", POOLED_CASES, ids=lambda c: "C{}_K{}_{}x{}_k{}x{}_{}_n{}".format(*[
    "".join(map(str, v)) if isinstance(v, tuple) else v for v in c]))
@pytest.mark.parametrize("mode", ["plain", "bias_leaky"])
def test_conv2d_maxpool_3xtf32(oracle, case, mode):
    """Conv2D(+bias)(+activation) -> MaxPool2D 2x2 / 2 in the epilogue of the tensor-core kernel (the
    reference's Conv2D_Bias_ReLU_Maxpool2D family, fused_interface_abstract.hpp:463-1418) against the
    oracle's convolution followed by its max pool, and bit-identical to the two-call path."""
    C, K, H, W, Fh, Fw, pm, N = case
    pads = same_pads(H, W, Fh, Fw, 1) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm
    assert S.conv2d_maxpool_3xTF32_supported(Fh, Fw, pads, K, C, H, W)
    rng = np.random.default_rng(abs(hash((case, mode, "pool"))) % (1 << 31))
    x = P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, np.sqrt(2.0 / (C * Fh * Fw)), (K, C, Fh, Fw)).astype(np.float32))
    bias = None if mode == "plain" else rng.uniform(-0.5, 0.5, K).astype(np.float32)
    act, slope = (0, 0.0) if mode == "plain" else (S.ACT_LEAKY, 0.1)
    sh = shape(C, K, H, W, Fh, Fw, 1, pads, CB)
    ho, wo = sh.out_hw()
    shp = shape(K, K, ho, wo, 2, 2, 2, (0, 0, 0, 0), CB)
    I, F = fbuf(x), fbuf(w)
    B = None if bias is None else fbuf(bias)
    Fp = S.FloatBuffer(2 * F.size())
    S.prepare_filter_3xTF32(Fh, Fw, K, C, F, Fp)
    O = S.FloatBuffer(N * K * (ho // 2) * (wo // 2))
    S.Conv2D_Maxpool2D_3xTF32(Fh, Fw, pads, K, C, H, W, I, Fp, B, O, activation=act, negative_slope=slope, batch=N)
    got = O.numpy().reshape(N, -1)
    assert _lib.device_status() == 0
    conv = oracle_conv_batch(oracle, sh, x, w, bias=bias, act=act, slope=slope)
    want = np.stack([oracle.pool2d_f32(shp, conv[n]) for n in range(N)])
    assert rel_max_err(got, want) <= TOL
    # same sums in the same order with or without the pool
    mid, two = S.FloatBuffer(N * K * ho * wo), S.FloatBuffer(N * K * (ho // 2) * (wo // 2))
    S.Conv2D_3xTF32(Fh, Fw, 1, *pads, K, C, H, W, I, Fp, B, mid, activation=act, negative_slope=slope, batch=N)
    S.MaxPool2D(2, 2, 2, 0, 0, 0, 0, K, ho, wo, mid, two, batch=N)
    assert np.array_equal(got, two.numpy().reshape(N, -1))


def test_pooled_epilogue_refuses_other_shapes():
    assert not S.conv2d_maxpool_3xTF32_supported(3, 3, (1, 1, 1, 1), 32, 16, 52, 52)     # narrow image: row-range tiles
    assert not S.conv2d_maxpool_3xTF32_supported(3, 3, (1, 1, 1, 1), 128, 64, 104, 104)  # channel-major kernel
    assert not S.conv2d_maxpool_3xTF32_supported(3, 3, (1, 1, 1, 1), 32, 16, 101, 101)   # odd output
    assert not S.conv2d_maxpool_3xTF32_supported(2, 2, (0, 0, 0, 0), 32, 16, 101, 101)   # even filter width
    assert not S.conv2d_maxpool_3xTF32_supported(3, 3, (1, 1, 1, 1), 16, 16, 104, 104)   # 16 output channels


def test_unsupported_shapes_are_refused():
    assert not S.tf32x3_supported(3, 3, 2, 0, 1, 0, 1, 16, 16, 32, 32)   # stride 2
    assert not S.tf32x3_supported(3, 3, 1, 1, 1, 1, 1, 16, 3, 32, 32)    # first layer
    assert S.tf32x3_supported(3, 3, 1, 1, 1, 1, 1, 16, 16, 416, 416)     # wide images: 2-D pixel tiles
