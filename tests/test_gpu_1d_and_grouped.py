"""The 1-D family (2-D layers with a window height of 1 and a row stride of 1), the grouped
convolution of the fused interface (block-diagonal 16 -> 16 convolutions) and Dropout, through the
C ABI against the oracle.  A 1-D layer over [C/16][batch][W][16] is checked row by row: every batch
entry is a 1 x W image for the oracle (include/small/abstract_layer.hpp:1838-1846)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.bindings import shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, rel_max_err

pytestmark = pytest.mark.gpu


def _layer(N, C_, K, H, W, Fh, Fw, stride, pads, stride_h=0, accumulate=0, act=0):
    L = _lib.Layer(N, C_, K, H, W, Fh, Fw, stride, *pads, accumulate, act, 0.0, 0, 0, 0, 0, 0, 0)
    L.stride_h = stride_h
    return L


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("case", [(16, 32, 7, 40, 3, 2, (1, 1)), (32, 16, 5, 33, 5, 2, (2, 2)), (16, 16, 4, 24, 3, 1, (1, 1)),
                                  (3, 16, 6, 50, 7, 2, (3, 3)), (64, 64, 3, 16, 1, 2, (0, 0))],
                         ids=lambda c: "C{}_K{}_b{}_W{}_k{}_s{}".format(*c[:6]))
@pytest.mark.parametrize("partial", [False, True])
def test_conv1d_with_its_own_row_stride(oracle, case, partial):
    """small::Conv1D / PartialConv1D (interface_abstract_1D.hpp:47, :415), strides 1 and 2."""
    Cn, K, B, W, k, s, (l, r) = case
    rng = np.random.default_rng(abs(hash(case)) % (1 << 31))
    x = rng.uniform(-1, 1, (Cn, B, W)).astype(np.float32)           # [C][batch][W]
    w = rng.normal(0, 0.2, (K, Cn, 1, k)).astype(np.float32)
    xp, wp = P.pack_activation(x[None])[0], P.pack_conv_filter(w)
    L = _layer(1, Cn, K, B, W, 1, k, s, (0, 0, l, r), stride_h=1, accumulate=int(partial))
    ho, wo = L.out_hw()
    assert ho == B
    seed = rng.uniform(-1, 1, K * B * wo).astype(np.float32)
    tx, tw, to = _dev(xp), _dev(wp), _dev(seed)
    _lib.check(_lib.lib().small_b200_conv2d_f32(C.byref(L), tx.data_ptr(), tw.data_ptr(), None, to.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    got = P.unpack_activation(to.cpu().numpy()[None], K, B, wo)[0]    # [K][batch][Wo]
    seed_u = P.unpack_activation(seed[None], K, B, wo)[0]
    sh = shape(Cn, K, 1, W, 1, k, s, (0, 0, l, r), CB)
    for b in range(B):
        row = P.pack_activation(x[None, :, b:b + 1, :])[0]
        out0 = P.pack_activation(seed_u[None, :, b:b + 1, :])[0] if partial else None
        want = P.unpack_activation(oracle.conv2d_f32(sh, row, wp, out=out0)[None], K, 1, wo)[0][:, 0]
        assert rel_max_err(got[:, b], want) <= 1e-5, (case, b)


@pytest.mark.parametrize("average", [False, True])
def test_pool1d_with_its_own_row_stride(oracle, average):
    Cn, B, W, k, s = 32, 6, 41, 3, 2
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, (Cn, B, W)).astype(np.float32)
    xp = P.pack_activation(x[None])[0]
    L = _layer(1, Cn, Cn, B, W, 1, k, s, (0, 0, 1, 1), stride_h=1)
    ho, wo = L.out_hw()
    tx, to = _dev(xp), torch.zeros(Cn * B * wo, device="cuda")
    fn = _lib.lib().small_b200_avgpool2d_f32 if average else _lib.lib().small_b200_maxpool2d_f32
    _lib.check(fn(C.byref(L), tx.data_ptr(), to.data_ptr(), torch.cuda.current_stream().cuda_stream))
    got = P.unpack_activation(to.cpu().numpy()[None], Cn, B, wo)[0]
    sh = shape(Cn, Cn, 1, W, 1, k, s, (0, 0, 1, 1), CB)
    for b in range(B):
        row = P.pack_activation(x[None, :, b:b + 1, :])[0]
        want = P.unpack_activation(oracle.pool2d_f32(sh, row, average=average)[None], Cn, 1, wo)[0][:, 0]
        assert np.array_equal(got[:, b], want) if not average else rel_max_err(got[:, b], want) <= 1e-6


def test_upsample1d():
    Cn, B, W = 32, 5, 9
    rng = np.random.default_rng(6)
    x = rng.uniform(-1, 1, (Cn, B, W)).astype(np.float32)
    tx, to = _dev(P.pack_activation(x[None])[0]), torch.zeros(Cn * B * W * 2, device="cuda")
    _lib.check(_lib.lib().small_b200_upsample1d_f32(1, Cn, B, W, tx.data_ptr(), to.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream))
    got = P.unpack_activation(to.cpu().numpy()[None], Cn, B, 2 * W)[0]
    assert np.array_equal(got, np.repeat(x, 2, axis=2))


def test_row_stride_is_refused_where_it_is_not_provided():
    L = _layer(1, 32, 32, 8, 8, 1, 3, 2, (0, 0, 1, 1), stride_h=1)
    assert not _lib.lib().small_b200_conv2d_f32_tf32x3_supported(C.byref(L))
    with pytest.raises(ValueError, match="stride unsupported"):
        _lib.check(_lib.lib().small_b200_conv2d_u8(C.byref(L), None, None, None, None, None))


@pytest.mark.parametrize("case", [(4, 10, 12, 3, 1, (1, 1, 1, 1), 2), (3, 9, 9, 3, 2, (0, 1, 0, 1), 1), (8, 6, 6, 1, 1, (0, 0, 0, 0), 3)],
                         ids=lambda c: "G{}_{}x{}_k{}_s{}_n{}".format(c[0], c[1], c[2], c[3], c[4], c[6]))
@pytest.mark.parametrize("mode", ["plain", "bias_relu", "partial"])
def test_block_diagonal_grouped_convolution(oracle, case, mode):
    """The grouped convolution of the reference's fused interface (fused_interface_abstract.hpp:2740-2760):
    group g is a dense 16 -> 16 convolution on channel block g, i.e. the oracle's dense convolution with
    C = K = 16 applied block by block with that group's filter."""
    G, H, W, k, s, pads, N = case
    rng = np.random.default_rng(abs(hash((case, mode))) % (1 << 31))
    x = rng.uniform(-1, 1, (N, G * 16, H, W)).astype(np.float32)
    w = rng.normal(0, 0.2, (G, 16, 16, k, k)).astype(np.float32)    # [g][k][c][kh][kw]
    bias = rng.uniform(-0.5, 0.5, G * 16).astype(np.float32) if mode == "bias_relu" else None
    xp = P.pack_activation(x)
    wp = np.concatenate([P.pack_conv_filter(w[g]) for g in range(G)])
    L = _layer(N, 16, 16, H, W, k, k, s, pads, accumulate=int(mode == "partial"), act=1 if mode == "bias_relu" else 0)
    ho, wo = L.out_hw()
    seed = rng.uniform(-1, 1, (N, G * 16 * ho * wo)).astype(np.float32)
    tx, tw, to = _dev(xp.ravel()), _dev(wp), _dev(seed.ravel())
    tb = None if bias is None else _dev(bias)
    _lib.check(_lib.lib().small_b200_blockconv2d_f32(C.byref(L), G, tx.data_ptr(), tw.data_ptr(),
                                                     None if tb is None else tb.data_ptr(), to.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream))
    got = to.cpu().numpy().reshape(N, G, -1)
    sh = shape(16, 16, H, W, k, k, s, pads, CB)
    for n in range(N):
        for g in range(G):
            blk = xp[n].reshape(G, -1)[g]
            out0 = seed[n].reshape(G, -1)[g] if mode == "partial" else None
            want = oracle.conv2d_f32(sh, blk, P.pack_conv_filter(w[g]), bias=None if bias is None else bias[g * 16:(g + 1) * 16],
                                     act=1 if mode == "bias_relu" else 0, out=out0)
            assert rel_max_err(got[n, g], want) <= 1e-5, (case, mode, n, g)


def test_dropout_scales():
    rng = np.random.default_rng(8)
    x = rng.uniform(-1, 1, (2, 32, 5, 7)).astype(np.float32)
    I, O = S.FloatBuffer(data=P.pack_activation(x)), S.FloatBuffer(x.size)
    S.Dropout(32, 5, 7, I, 0.625, O, batch=2)
    assert np.array_equal(O.numpy(), (P.pack_activation(x).ravel() * np.float32(0.625)))
    with pytest.raises(ValueError, match="in_channels unsupported"):
        S.Dropout(8, 5, 7, I, 0.5, O)
