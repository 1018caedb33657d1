"""Grouped convolution (small::GroupConv2D / PartialGroupConv2D,
include/small/interface_abstract.hpp:1265-1530).

CPU part: the restatement with a group block of 1 against the UNMODIFIED reference on its REF
platform, bit for bit (float, Partial float, quint8), and the block-16 restatement against the
block-1 one after re-packing (the block only changes where a group's numbers lie).
GPU part: the CUDA path through the C ABI against the block-16 restatement: float within the
1e-5 gate of the other fp32 contractions, quint8 bit-exact.

Layouts (abstract_layer.hpp:1419-1432 with K_b = F_cb = 1):
    I [G/gb][C][H][W][gb]   F [G/gb][K][C][Fh][Fw][gb]   O [G/gb][K][Ho][Wo][gb]
"""
import numpy as np
import pytest

from oracle.bindings import Quant, same_pads, shape

CB = 16

# groups, channels per group, H, W, Fh, Fw, stride, pads  (inside the domain where the
# reference's edge kernels are self-consistent: 3x3 with pad <= 1, 1x1 unpadded)
REF_CASES = [
    (4, 3, 7, 9, 3, 3, 1, (1, 1, 1, 1)),
    (2, 5, 8, 8, 3, 3, 2, (0, 1, 0, 1)),
    (6, 2, 6, 5, 1, 1, 1, (0, 0, 0, 0)),
    (3, 4, 9, 9, 3, 3, 1, (0, 0, 0, 0)),
    (16, 16, 6, 6, 3, 3, 1, (1, 1, 1, 1)),
    (1, 8, 10, 7, 3, 3, 2, (0, 0, 0, 0)),
]


def pack_groups(a, gb):
    """[G][planes][h][w] -> [G/gb][planes][h][w][gb]"""
    G = a.shape[0]
    return np.ascontiguousarray(
        a.reshape(G // gb, gb, *a.shape[1:]).transpose(0, 2, 3, 4, 1)).ravel()


def unpack_groups(a, G, planes, h, w, gb):
    return a.reshape(G // gb, planes, h, w, gb).transpose(0, 4, 1, 2, 3).reshape(G, planes, h, w)


def _id(c):
    G, C, H, W, Fh, Fw, s, pads = c
    return f"G{G}_C{C}_{H}x{W}_k{Fh}x{Fw}_s{s}_p{''.join(map(str, pads))}"


@pytest.mark.parametrize("c", REF_CASES, ids=_id)
def test_oracle_block1_is_the_reference(oracle, ref, c):
    G, C, H, W, Fh, Fw, s, pads = c
    rng = np.random.default_rng(hash(c) & 0xFFFF)
    sh = shape(C, C, H, W, Fh, Fw, s, pads, 1)
    ho, wo = sh.out_hw()
    x = rng.uniform(-1, 1, G * C * H * W).astype(np.float32)
    w = rng.normal(0, 0.3, G * C * C * Fh * Fw).astype(np.float32)
    assert np.array_equal(oracle.groupconv2d_f32(sh, G, x, w), ref.groupconv2d_f32(sh, G, x, w))
    seed = rng.uniform(-1, 1, G * C * ho * wo).astype(np.float32)
    assert np.array_equal(oracle.groupconv2d_f32(sh, G, x, w, out=seed),
                          ref.groupconv2d_f32(sh, G, x, w, out=seed))
    q = Quant(int(rng.choice([0, -128, 5])), int(rng.choice([-128, 0, -7])), 0, 9, 1515870810, 0)
    xu = rng.integers(0, 256, G * C * H * W).astype(np.uint8)
    wu = rng.integers(0, 256, G * C * C * Fh * Fw).astype(np.uint8)
    assert np.array_equal(oracle.groupconv2d_u8(sh, q, G, xu, wu), ref.groupconv2d_u8(sh, q, G, xu, wu))


def test_oracle_block16_is_block1_repacked(oracle):
    rng = np.random.default_rng(3)
    G, C, K, H, W, Fh, Fw, s, pads = 32, 3, 5, 7, 6, 3, 3, 1, (1, 1, 1, 1)
    x = rng.uniform(-1, 1, (G, C, H, W)).astype(np.float32)
    w = rng.normal(0, 0.3, (G, K * C, Fh, Fw)).astype(np.float32)
    b = rng.uniform(-1, 1, (G, K, 1, 1)).astype(np.float32)
    s1, s16 = shape(C, K, H, W, Fh, Fw, s, pads, 1), shape(C, K, H, W, Fh, Fw, s, pads, CB)
    ho, wo = s1.out_hw()
    o1 = oracle.groupconv2d_f32(s1, G, x.ravel(), w.ravel(), bias=b.ravel(), act=2, slope=0.1)
    o16 = oracle.groupconv2d_f32(s16, G, pack_groups(x, CB), pack_groups(w, CB), bias=pack_groups(b, CB),
                                 act=2, slope=0.1)
    assert np.array_equal(unpack_groups(o16, G, K, ho, wo, CB), o1.reshape(G, K, ho, wo))
    q = Quant(-128, -128, 0, 11, 1300000000, 0)
    xu = rng.integers(0, 256, (G, C, H, W)).astype(np.uint8)
    wu = rng.integers(0, 256, (G, K * C, Fh, Fw)).astype(np.uint8)
    u1 = oracle.groupconv2d_u8(s1, q, G, xu.ravel(), wu.ravel())
    u16 = oracle.groupconv2d_u8(s16, q, G, pack_groups(xu, CB), pack_groups(wu, CB))
    assert np.array_equal(unpack_groups(u16, G, K, ho, wo, CB), u1.reshape(G, K, ho, wo))
    assert u1.min() < u1.max()


# ------------------------------------------------------------------------------- GPU
GPU_CASES = [
    # groups, C (= K) per group, H, W, Fh, Fw, stride, pads, batch
    (16, 16, 9, 11, 3, 3, 1, "same", 2),
    (32, 16, 8, 8, 3, 3, 2, "same", 3),
    (48, 32, 5, 7, 1, 1, 1, "valid", 1),
    (16, 16, 12, 6, 5, 3, 2, (2, 1, 0, 2), 2),
    (64, 16, 13, 13, 3, 3, 1, "valid", 1),
]


def _pads(c):
    G, C, H, W, Fh, Fw, s, pm, N = c
    return same_pads(H, W, Fh, Fw, s) if pm == "same" else (0, 0, 0, 0) if pm == "valid" else pm


@pytest.mark.gpu
@pytest.mark.parametrize("c", GPU_CASES, ids=lambda c: "G{}_C{}_{}x{}_k{}x{}_s{}".format(*c[:7]))
def test_groupconv_f32_vs_oracle(oracle, c):
    from smallframework_b200 import interface as S
    from tests.gpu_util import fbuf, rel_max_err
    G, C, H, W, Fh, Fw, s, pm, N = c
    pads = _pads(c)
    rng = np.random.default_rng(abs(hash(c)) % (1 << 31))
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    x = rng.uniform(-1, 1, (N, G * C * H * W)).astype(np.float32)
    w = rng.normal(0, 0.2, G * C * C * Fh * Fw).astype(np.float32)
    I, F, O = fbuf(x), fbuf(w), S.FloatBuffer(N * G * C * ho * wo)
    S.GroupConv2D(Fh, Fw, s, G, *pads, C, H, W, I, F, O, batch=N)
    want = np.stack([oracle.groupconv2d_f32(sh, G, x[n], w) for n in range(N)])
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= 1e-5
    seed = rng.uniform(-1, 1, (N, G * C * ho * wo)).astype(np.float32)
    O = fbuf(seed)
    S.PartialGroupConv2D(Fh, Fw, s, G, *pads, C, H, W, I, F, O, batch=N)
    want = np.stack([oracle.groupconv2d_f32(sh, G, x[n], w, out=seed[n]) for n in range(N)])
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= 1e-5
    bias = rng.uniform(-1, 1, G * C).astype(np.float32)
    S.GroupConv2D(Fh, Fw, s, G, *pads, C, H, W, I, F, O, bias_buf=fbuf(bias), activation=S.ACT_LEAKY,
                  negative_slope=0.1, batch=N)
    want = np.stack([oracle.groupconv2d_f32(sh, G, x[n], w, bias=bias, act=2, slope=0.1) for n in range(N)])
    assert rel_max_err(O.numpy().reshape(N, -1), want) <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("c", GPU_CASES, ids=lambda c: "G{}_C{}_{}x{}_k{}x{}_s{}".format(*c[:7]))
@pytest.mark.parametrize("zeros", [(-128, -128), (0, -128), (5, -7)])
def test_groupconv_u8_bit_exact(oracle, c, zeros):
    from smallframework_b200 import interface as S
    from tests.gpu_util import qbuf
    G, C, H, W, Fh, Fw, s, pm, N = c
    pads = _pads(c)
    rng = np.random.default_rng(abs(hash((c, zeros))) % (1 << 31))
    zi, zf = zeros
    ma, mw = 127.5 + zi, 127.5 + zf
    t = C * Fh * Fw
    top = abs(t * ma * mw) + 2.0 * np.sqrt(t * ((74.0 ** 2 + ma ** 2) * (74.0 ** 2 + mw ** 2) - (ma * mw) ** 2))
    scale = 255.0 / top
    rshift = int(np.clip(np.floor(-np.log2(scale)), 0, 30))
    q = Quant(zi, zf, 0, rshift, int(np.clip(scale * 2.0 ** (31 + rshift), 1 << 20, (1 << 31) - 1)), 0)
    sh = shape(C, C, H, W, Fh, Fw, s, pads, CB)
    ho, wo = sh.out_hw()
    x = rng.integers(0, 256, (N, G * C * H * W)).astype(np.uint8)
    w = rng.integers(0, 256, G * C * C * Fh * Fw).astype(np.uint8)
    O = S.QUInt8Buffer(N * G * C * ho * wo)
    O.lshift, O.rshift, O.multiplier = q.lshift, q.rshift, q.multiplier
    S.GroupConv2D(Fh, Fw, s, G, *pads, C, H, W, qbuf(x, zi), qbuf(w, zf), O, batch=N)
    want = np.stack([oracle.groupconv2d_u8(sh, q, G, x[n], w) for n in range(N)])
    assert np.array_equal(O.numpy().reshape(N, -1), want)
    assert want.min() < want.max()


@pytest.mark.gpu
def test_groupconv_argument_errors():
    from smallframework_b200 import interface as S
    I, F, O = S.FloatBuffer(16 * 16 * 16), S.FloatBuffer(16 * 16 * 16 * 9), S.FloatBuffer(16 * 16 * 16)
    with pytest.raises(ValueError, match="in_channels unsupported"):
        S.GroupConv2D(3, 3, 1, 16, 1, 1, 1, 1, 3, 4, 4, I, F, O)
    with pytest.raises(ValueError, match="stride unsupported"):
        S.GroupConv2D(3, 3, 3, 16, 1, 1, 1, 1, 16, 4, 4, I, F, O)
    with pytest.raises(ValueError, match="output_groups unsupported"):
        S.GroupConv2D(3, 3, 1, 5, 1, 1, 1, 1, 16, 4, 4, I, F, O)
