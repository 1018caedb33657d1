"""How far each fp32 convolution path is from the exact result.  The reference's loop nest (the
oracle restates it bit for bit), the CUDA-core kernel and the 3xTF32 tensor-core kernel are
compared with an fp64 recomputation on the deepest reduction of the benchmark networks
(1024 input channels x 3x3 = 9216 terms, Tiny-YOLOv2 conv8) and on the reference's own golden
convolutions, in the two norms in use:
  * max norm, max|x - exact| / max|exact|  (the 1e-5 gate of the GPU parity tests);
  * the reference's element-wise almost_equal, |x - y| <= 1e-5 + 5e-3 |y| (test/test_utils.hpp:41-46),
    reported as the worst |x - y| / (1e-5 + 5e-3 |y|): at most 1 passes.
The numbers are printed (run with -s) and bounded."""
import numpy as np
import pytest
import torch

from oracle.bindings import same_pads, shape
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, fbuf
from tests.util import case_id, case_pads, golden_cases, read_bin

pytestmark = pytest.mark.gpu


def conv_fp64(x, w, pads, stride=1):
    """x [C,H,W], w [K,C,Fh,Fw] -> [K,Ho,Wo] in float64 (im2col + one matrix product)."""
    t, b, l, r = pads
    Cn, H, W = x.shape
    K, _, Fh, Fw = w.shape
    xp = np.zeros((Cn, H + t + b, W + l + r), np.float64)
    xp[:, t:t + H, l:l + W] = x
    Ho, Wo = (H + t + b - Fh) // stride + 1, (W + l + r - Fw) // stride + 1
    cols = np.empty((Cn, Fh, Fw, Ho, Wo), np.float64)
    for kh in range(Fh):
        for kw in range(Fw):
            cols[:, kh, kw] = xp[:, kh:kh + stride * Ho:stride, kw:kw + stride * Wo:stride]
    return (w.reshape(K, -1).astype(np.float64) @ cols.reshape(Cn * Fh * Fw, Ho * Wo)).reshape(K, Ho, Wo)


def norms(got, exact):
    d = np.abs(got.astype(np.float64) - exact)
    return float(d.max() / np.abs(exact).max()), float((d / (1e-5 + 5e-3 * np.abs(exact))).max())


def gpu_paths(x, w, pads, stride=1):
    """(CUDA-core result, tensor-core result or None), unpacked [K,Ho,Wo]."""
    Cn, H, W = x.shape
    K, _, Fh, Fw = w.shape
    xp, wp = P.pack_activation(x[None]), P.pack_conv_filter(w)
    sh = shape(Cn, K, H, W, Fh, Fw, stride, pads, CB)
    ho, wo = sh.out_hw()
    O = S.FloatBuffer(K * ho * wo)
    S.Conv2D(Fh, Fw, stride, *pads, K, Cn, H, W, fbuf(xp), fbuf(wp), O)
    ffma = P.unpack_activation(O.numpy()[None], K, ho, wo)[0]
    tc = None
    if S.tf32x3_supported(Fh, Fw, stride, *pads, K, Cn, H, W):
        prep = S.FloatBuffer(2 * wp.size)
        S.prepare_filter_3xTF32(Fh, Fw, K, Cn, fbuf(wp), prep)
        O2 = S.FloatBuffer(K * ho * wo)
        S.Conv2D_3xTF32(Fh, Fw, stride, *pads, K, Cn, H, W, fbuf(xp), prep, None, O2)
        tc = P.unpack_activation(O2.numpy()[None], K, ho, wo)[0]
    torch.cuda.synchronize()
    return ffma, tc, (sh, xp[0], wp, ho, wo)


@pytest.mark.parametrize("dist", ["relu_like", "signed"])
def test_error_against_fp64_at_9216_terms(oracle, dist):
    rng = np.random.default_rng(64)
    Cn = K = 1024; H = W = 13
    pads = same_pads(H, W, 3, 3, 1)
    x = rng.random((Cn, H, W), dtype=np.float32) if dist == "relu_like" else rng.uniform(-1, 1, (Cn, H, W)).astype(np.float32)
    w = rng.normal(0, np.sqrt(2 / (Cn * 9)), (K, Cn, 3, 3)).astype(np.float32)
    exact = conv_fp64(x, w, pads)
    ffma, tc, (sh, xp, wp, ho, wo) = gpu_paths(x, w, pads)
    ref = P.unpack_activation(oracle.conv2d_f32(sh, xp, wp)[None], K, ho, wo)[0]
    rows = {"reference loop nest (oracle)": norms(ref, exact), "CUDA-core kernel": norms(ffma, exact),
            "3xTF32 tensor-core kernel": norms(tc, exact)}
    for name, (mx, ew) in rows.items():
        print(f"\n{dist:9s} 1024->1024 3x3 @13, vs fp64: {name:30s} max-norm {mx:.2e}  element-wise worst {ew:.2e}")
    # each path is inside the 1e-5 gate against the exact result, not only against each other
    for name, (mx, ew) in rows.items():
        assert mx <= 1e-5, (name, mx)


@pytest.mark.parametrize("case", golden_cases("conv2d"), ids=case_id)
def test_golden_convolutions_both_paths_in_both_norms(case):
    """The reference's own golden convolutions (PyTorch outputs): where each device path stands
    against the golden data in the reference's element-wise norm and in the max norm."""
    Cn, K, H, W, k, s = case["C"], case["K"], case["H"], case["W"], case["k"], case["s"]
    if Cn % CB or K % CB:
        pytest.skip("golden case with an odd channel count is a first-layer case")
    pads = case_pads(case)
    x = read_bin(case["x"]).reshape(Cn, H, W)
    w = read_bin(case["w"]).reshape(K, Cn, k, k)
    sh = shape(Cn, K, H, W, k, k, s, pads, CB)
    ho, wo = sh.out_hw()
    y = read_bin(case["y"]).reshape(K, ho, wo).astype(np.float64)
    ffma, tc, _ = gpu_paths(x, w, pads, s)
    mx, ew = norms(ffma, y)
    print(f"\n{case_id(case)}: CUDA cores max-norm {mx:.2e} element-wise {ew:.2e}", end="")
    assert ew <= 1.0 and mx <= 1e-5
    if tc is not None:
        mx, ew = norms(tc, y)
        print(f"; tensor cores max-norm {mx:.2e} element-wise {ew:.2e}", end="")
        assert mx <= 1e-5
