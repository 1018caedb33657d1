"""One process, two devices: kernels that need more than 48 KB of shared memory set their function
attribute per device, the status word and the constant-memory slots are per device.  Skipped where
fewer than two GPUs are visible."""
import numpy as np
import pytest
import torch

from oracle.bindings import Quant, same_pads, shape
from smallframework_b200 import _lib
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P
from tests.gpu_util import CB, oracle_conv_batch, rel_max_err

pytestmark = pytest.mark.gpu


def _on(dev, a, dtype=np.float32):
    cls = S.FloatBuffer if dtype == np.float32 else S.QUInt8Buffer
    return cls(device=f"cuda:{dev}", data=np.ascontiguousarray(a, dtype))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_same_process_two_devices(oracle):
    rng = np.random.default_rng(21)
    # fp32 on the tensor cores (200 KB of shared memory), the first layer (constant-memory slots), and
    # the uint8 pointwise kernel, each on device 0, then device 1, then device 0 again
    C, K, H, W, N = 64, 128, 13, 13, 3
    pads = same_pads(H, W, 3, 3, 1)
    sh = shape(C, K, H, W, 3, 3, 1, pads, CB)
    x = P.pack_activation(rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32))
    w = P.pack_conv_filter(rng.normal(0, 0.05, (K, C, 3, 3)).astype(np.float32))
    want = oracle_conv_batch(oracle, sh, x, w, act=1)
    sh1 = shape(3, 16, 32, 32, 3, 3, 1, same_pads(32, 32, 3, 3, 1), CB)
    x1 = P.pack_activation(rng.uniform(-1, 1, (N, 3, 32, 32)).astype(np.float32))
    w1 = P.pack_conv_filter(rng.normal(0, 0.2, (16, 3, 3, 3)).astype(np.float32))
    want1 = oracle_conv_batch(oracle, sh1, x1, w1, act=1)
    q = Quant(0, -128, 0, 9, 1518500250, 0)
    shq = shape(64, 64, 25, 5, 1, 1, 1, (0, 0, 0, 0), CB)
    xq = P.pack_activation(rng.integers(0, 256, (N, 64, 25, 5)).astype(np.uint8))
    wq = P.pack_conv_filter(rng.integers(0, 256, (64, 64, 1, 1)).astype(np.uint8))
    wantq = np.stack([oracle.conv2d_u8(shq, q, xq[n], wq) for n in range(N)])
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().small_b200_set_device(dev))
            FP = S.FloatBuffer(2 * w.size, device=f"cuda:{dev}")
            S.prepare_filter_3xTF32(3, 3, K, C, _on(dev, w), FP)
            O = S.FloatBuffer(N * K * H * W, device=f"cuda:{dev}")
            S.Conv2D_3xTF32(3, 3, 1, *pads, K, C, H, W, _on(dev, x), FP, None, O, activation=S.ACT_RELU, batch=N)
            assert rel_max_err(O.numpy().reshape(N, -1), want) <= 1e-5
            O1 = S.FloatBuffer(N * 16 * 32 * 32, device=f"cuda:{dev}")
            S.Conv2D_ReLU(3, 3, 1, *same_pads(32, 32, 3, 3, 1), 16, 3, 32, 32, _on(dev, x1), _on(dev, w1), O1, batch=N)
            assert rel_max_err(O1.numpy().reshape(N, -1), want1) <= 1e-5
            I, F = _on(dev, xq, np.uint8), _on(dev, wq, np.uint8)
            I.m_zero, F.m_zero = q.zero_in, q.zero_filt
            Oq = S.QUInt8Buffer(N * 64 * 125, device=f"cuda:{dev}")
            Oq.lshift, Oq.rshift, Oq.multiplier = q.lshift, q.rshift, q.multiplier
            S.Conv2D(1, 1, 1, 0, 0, 0, 0, 64, 64, 25, 5, I, F, Oq, batch=N)
            assert np.array_equal(Oq.numpy().reshape(N, -1), wantq)
            assert _lib.device_status() == 0
    _lib.check(_lib.lib().small_b200_set_device(0))
