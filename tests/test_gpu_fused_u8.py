"""The one-kernel uint8 blocks (csrc/block_u8_tc.cu) through the C ABI against the oracle's
layer-by-layer result, bit-exact: 1x1 convolution -> 3x3 depthwise convolution, one-channel first
layer -> depthwise convolution, and 1x1 convolution -> global average pool -> dense layer.
Image sizes up to the 128-pixel limit, batches that give a CTA none, one and several images,
both zero points of the input and of the intermediate, with and without biases."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.bindings import Quant, same_pads, shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB

pytestmark = pytest.mark.gpu


def _quant_for(acc_top):
    """(lshift, rshift, multiplier) mapping accumulators up to acc_top onto 0..255."""
    import math
    scale = 255.0 / max(acc_top, 1.0)
    rshift = int(np.clip(math.floor(-math.log2(scale)), 0, 30))
    mult = int(np.clip(round(scale * 2.0 ** (31 + rshift)), 1, (1 << 31) - 1))
    return 0, rshift, mult


def _qbuf(data, zero, q=None):
    b = S.QUInt8Buffer(data=np.ascontiguousarray(data, np.uint8))
    b.m_zero = zero
    if q is not None:
        b.lshift, b.rshift, b.multiplier = q
    return b


PW_DW_CASES = [
    # C, K, H, W, batch, zero_in, zero_mid, biases
    (64, 64, 25, 5, 5, 0, 0, True),        # the keyword-spotting block
    (64, 64, 25, 5, 700, 0, 0, True),      # several images per CTA
    (32, 32, 8, 8, 3, -128, 0, False),
    (128, 64, 16, 8, 2, 0, -128, True),    # exactly 128 pixels; signed intermediate
    (64, 32, 11, 11, 1, -128, -128, True),
    (32, 64, 1, 7, 4, 0, 0, False),        # one row
    (64, 64, 9, 1, 4, 0, 0, True),         # one column
    (32, 32, 1, 1, 3, 0, 0, True),         # one pixel
    (128, 64, 10, 10, 3, -128, 0, "huge"),  # biases too large for the in-accumulator form of the constants
]


@pytest.mark.parametrize("case", PW_DW_CASES, ids=lambda c: "C{}_K{}_{}x{}_n{}_zi{}_zm{}_b{}".format(*c))
def test_pointwise_then_depthwise_one_kernel(oracle, case):
    Cn, K, H, W, N, zi, zm, with_bias = case
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    x = rng.integers(0, 256, (N, Cn, H, W), dtype=np.uint8)
    w1 = rng.integers(0, 256, (K, Cn, 1, 1), dtype=np.uint8)
    w2 = rng.integers(0, 256, (K, 3, 3), dtype=np.uint8)
    top = 1025 if with_bias != "huge" else 3_000_000
    b1 = rng.integers(-top + 1, top, K).astype(np.int32) if with_bias else None
    b2 = rng.integers(-top + 1, top, K).astype(np.int32) if with_bias else None
    q1 = _quant_for(Cn * 128 * 100 + (top if top > 2000 else 0))
    q2 = _quant_for(9 * 128 * 100 + (top if top > 2000 else 0))
    xp, w1p, w2p = P.pack_activation(x), P.pack_conv_filter(w1), P.pack_dw_filter(w2)
    I, F1, F2 = _qbuf(xp, zi), _qbuf(w1p, -128), _qbuf(w2p, -128)
    mid = _qbuf(np.zeros(N * K * H * W, np.uint8), zm, q1)
    O = _qbuf(np.zeros(N * K * H * W, np.uint8), 0, q2)
    tb = lambda b: None if b is None else torch.from_numpy(b).cuda()
    one_kernel = S.Conv2D_ReLU_DepthwiseConv2D_ReLU(1, 1, 1, 0, 0, 0, 0, 3, 3, 1, 1, 1, 1, 1, K, Cn, H, W, I, F1, mid, F2, O,
                                                   conv_bias=tb(b1), dw_bias=tb(b2), batch=N)
    assert one_kernel
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = O.numpy().reshape(N, -1)
    s1 = shape(Cn, K, H, W, 1, 1, 1, (0, 0, 0, 0), CB)
    s2 = shape(K, K, H, W, 3, 3, 1, (1, 1, 1, 1), CB)
    for n in sorted(set([0, N // 2, N - 1] + list(range(min(N, 3))))):
        m = oracle.conv2d_u8(s1, Quant(zi, -128, *q1, 0), xp[n], w1p, bias=b1)
        want = oracle.conv2d_u8(s2, Quant(zm, -128, *q2, 0), m, w2p, bias=b2, depthwise=True)
        assert np.array_equal(got[n], want), (case, n, int(np.count_nonzero(got[n] != want)))
    assert got.min() < got.max()


STEM_DW_CASES = [
    # H, W, Fh, Fw, stride, K, batch, zero_in
    (49, 10, 10, 4, 2, 64, 5, -128),   # the keyword-spotting stem
    (49, 10, 10, 4, 2, 64, 601, -128),
    (12, 10, 3, 3, 1, 32, 3, 0),
    (20, 6, 5, 2, 2, 64, 2, -128),
]


@pytest.mark.parametrize("case", STEM_DW_CASES, ids=lambda c: "{}x{}_k{}x{}_s{}_K{}_n{}_zi{}".format(*c))
def test_first_layer_then_depthwise_one_kernel(oracle, case):
    H, W, Fh, Fw, s, K, N, zi = case
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    pads = same_pads(H, W, Fh, Fw, s)
    x = rng.integers(0, 256, (N, 1, H, W), dtype=np.uint8)
    w1 = rng.integers(0, 256, (K, 1, Fh, Fw), dtype=np.uint8)
    w2 = rng.integers(0, 256, (K, 3, 3), dtype=np.uint8)
    b1 = rng.integers(-1024, 1025, K).astype(np.int32)
    b2 = rng.integers(-1024, 1025, K).astype(np.int32)
    q1 = _quant_for(Fh * Fw * 128 * 60)
    q2 = _quant_for(9 * 128 * 100)
    s1 = shape(1, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = s1.out_hw()
    s2 = shape(K, K, ho, wo, 3, 3, 1, (1, 1, 1, 1), CB)
    xp, w1p, w2p = P.pack_activation(x), P.pack_conv_filter(w1), P.pack_dw_filter(w2)
    I, F1, F2 = _qbuf(xp, zi), _qbuf(w1p, -128), _qbuf(w2p, -128)
    mid = _qbuf(np.zeros(N * K * ho * wo, np.uint8), 0, q1)
    O = _qbuf(np.zeros(N * K * ho * wo, np.uint8), 0, q2)
    one_kernel = S.Conv2D_ReLU_DepthwiseConv2D_ReLU(Fh, Fw, s, *pads, 3, 3, 1, 1, 1, 1, 1, K, 1, H, W, I, F1, mid, F2, O,
                                                   conv_bias=torch.from_numpy(b1).cuda(),
                                                   dw_bias=torch.from_numpy(b2).cuda(), batch=N)
    assert one_kernel
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = O.numpy().reshape(N, -1)
    for n in sorted(set([0, N // 2, N - 1])):
        m = oracle.conv2d_u8(s1, Quant(zi, -128, *q1, 0), xp[n], w1p, bias=b1)
        want = oracle.conv2d_u8(s2, Quant(0, -128, *q2, 0), m, w2p, bias=b2, depthwise=True)
        assert np.array_equal(got[n], want), (case, n)


def test_pairs_outside_the_one_kernel_form_run_as_two_calls(oracle):
    """A 14x14 image has more than 128 pixels: the same function gives the same bytes through two kernels."""
    Cn = K = 32; H = W = 14; N = 2
    rng = np.random.default_rng(3)
    x = rng.integers(0, 256, (N, Cn, H, W), dtype=np.uint8)
    w1 = rng.integers(0, 256, (K, Cn, 1, 1), dtype=np.uint8)
    w2 = rng.integers(0, 256, (K, 3, 3), dtype=np.uint8)
    q1, q2 = _quant_for(Cn * 128 * 100), _quant_for(9 * 128 * 100)
    xp, w1p, w2p = P.pack_activation(x), P.pack_conv_filter(w1), P.pack_dw_filter(w2)
    mid = _qbuf(np.zeros(N * K * H * W, np.uint8), 0, q1)
    O = _qbuf(np.zeros(N * K * H * W, np.uint8), 0, q2)
    one_kernel = S.Conv2D_ReLU_DepthwiseConv2D_ReLU(1, 1, 1, 0, 0, 0, 0, 3, 3, 1, 1, 1, 1, 1, K, Cn, H, W, _qbuf(xp, 0),
                                                   _qbuf(w1p, -128), mid, _qbuf(w2p, -128), O, batch=N)
    assert not one_kernel
    got = O.numpy().reshape(N, -1)
    s1 = shape(Cn, K, H, W, 1, 1, 1, (0, 0, 0, 0), CB)
    s2 = shape(K, K, H, W, 3, 3, 1, (1, 1, 1, 1), CB)
    for n in range(N):
        m = oracle.conv2d_u8(s1, Quant(0, -128, *q1, 0), xp[n], w1p)
        assert np.array_equal(got[n], oracle.conv2d_u8(s2, Quant(0, -128, *q2, 0), m, w2p, depthwise=True))


@pytest.mark.parametrize("case", [(64, 64, 25, 5, 12, 7), (64, 64, 25, 5, 12, 900), (32, 32, 6, 6, 32, 3), (128, 64, 16, 8, 2, 2)],
                         ids=lambda c: "C{}_K{}_{}x{}_Kd{}_n{}".format(*c))
def test_pointwise_pool_dense_one_kernel(oracle, case):
    Cn, K, H, W, Kd, N = case
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    x = rng.integers(0, 256, (N, Cn, H, W), dtype=np.uint8)
    w1 = rng.integers(0, 256, (K, Cn, 1, 1), dtype=np.uint8)
    kdp = -(-Kd // CB) * CB
    wd = np.full((kdp, K, 1, 1), 128, np.uint8)
    wd[:Kd] = rng.integers(0, 256, (Kd, K, 1, 1), dtype=np.uint8)
    b1 = rng.integers(-1024, 1025, K).astype(np.int32)
    bd = np.zeros(kdp, np.int32); bd[:Kd] = rng.integers(-1024, 1025, Kd)
    q1, qp, qd = _quant_for(Cn * 128 * 100), _quant_for(H * W * 255), _quant_for(K * 128 * 60)
    xp, w1p, wdp = P.pack_activation(x), P.pack_conv_filter(w1), P.pack_conv_filter(wd)
    Lc = S._qlayer(N, Cn, K, H, W, 1, 1, 1, (0, 0, 0, 0), 0, -128, q1)
    Lp = S._qlayer(N, K, K, H, W, H, W, 1, (0, 0, 0, 0), 0, 0, qp)
    Ld = S._qlayer(N, K, kdp, 1, 1, 1, 1, 1, (0, 0, 0, 0), 0, -128, qd)
    l = _lib.lib()
    assert l.small_b200_conv2d_avgpool_dense_u8_supported(C.byref(Lc), C.byref(Lp), C.byref(Ld))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tx, t1, td, tb1, tbd = dev(xp.ravel()), dev(w1p), dev(wdp), dev(b1), dev(bd)
    o = torch.zeros(N * kdp, dtype=torch.uint8, device="cuda")
    _lib.check(l.small_b200_conv2d_avgpool_dense_u8(C.byref(Lc), C.byref(Lp), C.byref(Ld), tx.data_ptr(), t1.data_ptr(),
                                                    tb1.data_ptr(), td.data_ptr(), tbd.data_ptr(), o.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = o.cpu().numpy().reshape(N, kdp)
    s1 = shape(Cn, K, H, W, 1, 1, 1, (0, 0, 0, 0), CB)
    sp = shape(K, K, H, W, H, W, 1, (0, 0, 0, 0), CB)
    sd = shape(K, kdp, 1, 1, 1, 1, 1, (0, 0, 0, 0), CB)
    for n in sorted(set([0, N // 2, N - 1])):
        m = oracle.conv2d_u8(s1, Quant(0, -128, *q1, 0), xp[n], w1p, bias=b1)
        pl = oracle.pool2d_u8(sp, Quant(0, 0, *qp, 0), m, average=True)
        want = oracle.conv2d_u8(sd, Quant(0, -128, *qd, 0), pl, wdp, bias=bd)
        assert np.array_equal(got[n], want), (case, n, got[n], want)
