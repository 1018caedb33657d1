"""Packed-layout index math against the formulas of include/small/buffers.hpp:33-120."""
import numpy as np
import pytest

from smallframework_b200 import packing as P


def packed_buffer_index(C, H, W, cb, c, h, w):
    cb = P.effective_block(C, cb)
    return (c // cb) * H * W * cb + h * W * cb + w * cb + c % cb


def packed_weight_index(K, C, Fh, Fw, cob, cib, k, c, kh, kw):
    cib = P.effective_block(C, cib)
    return ((k // cob) * (C // cib) * Fh * Fw * cib * cob + (c // cib) * Fh * Fw * cib * cob
            + kh * Fw * cib * cob + kw * cib * cob + (c % cib) * cob + k % cob)


@pytest.mark.parametrize("C,cb", [(3, 16), (16, 16), (96, 16), (32, 1), (1, 16), (2, 16)])
def test_activation_layout(C, cb):
    H, W = 5, 7
    x = np.arange(C * H * W, dtype=np.float32).reshape(C, H, W)
    p = P.pack_activation(x, cb)
    for c, h, w in [(0, 0, 0), (C - 1, H - 1, W - 1), (C // 2, 2, 3)]:
        assert p[packed_buffer_index(C, H, W, cb, c, h, w)] == x[c, h, w]
    assert np.array_equal(P.unpack_activation(p, C, H, W, cb), x)


@pytest.mark.parametrize("K,C", [(16, 3), (32, 16), (96, 96), (16, 1)])
def test_filter_layout(K, C):
    Fh, Fw = 3, 2
    w = np.arange(K * C * Fh * Fw, dtype=np.float32).reshape(K, C, Fh, Fw)
    p = P.pack_conv_filter(w, 16, 16)
    for k, c, kh, kw in [(0, 0, 0, 0), (K - 1, C - 1, Fh - 1, Fw - 1), (K // 2, C // 2, 1, 1)]:
        assert p[packed_weight_index(K, C, Fh, Fw, 16, 16, k, c, kh, kw)] == w[k, c, kh, kw]
    assert np.array_equal(P.unpack_conv_filter(p, K, C, Fh, Fw), w)


def test_batch_is_image_major():
    x = np.random.default_rng(0).normal(size=(3, 32, 4, 4)).astype(np.float32)
    p = P.pack_activation(x)
    assert p.shape == (3, 32 * 16)
    for n in range(3):
        assert np.array_equal(p[n], P.pack_activation(x[n]))


def test_bad_channel_counts_raise():
    with pytest.raises(RuntimeError):
        P.pack_activation(np.zeros((5, 2, 2), np.float32))
    with pytest.raises(RuntimeError):
        P.pack_activation(np.zeros((20, 2, 2), np.float32))


def test_padding_rules():
    # include/small/utils.hpp:43-64; examples: 3x3 s2 on 32 -> (0,1); 10x4 s2 on 49x10
    assert P.calc_padding(32, 3, 2) == (0, 1)
    assert P.calc_padding(49, 10, 2) == (4, 5)
    assert P.calc_padding(10, 4, 2) == (1, 1)
    assert P.output_dim(49, 4, 5, 10, 2) == 25 and P.output_dim(10, 1, 1, 4, 2) == 5
    assert P.calc_padding(416, 3, 1) == (1, 1)
