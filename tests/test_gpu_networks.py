"""Whole layer chains (smallframework_b200.networks.Chain, one CUDA graph) against the oracle's
chain: fast cases at reduced image sizes on both fp32 paths, DS-CNN uint8, bit-exact.  The same
networks at the sizes the benchmark runs are in test_gpu_full_size.py."""
import numpy as np
import pytest
import torch

from smallframework_b200 import _lib, networks
from smallframework_b200 import packing as P
from tests.gpu_util import oracle_chain, rel_max_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tensor_core", [False, True, "auto"])
def test_tiny_yolov2_chain(oracle, tensor_core):
    layers = networks.tiny_yolov2(seed=4, size=64)
    N = 3
    rng = np.random.default_rng(0)
    x = P.pack_activation(rng.random((N, 3, 64, 64), dtype=np.float32))
    chain = networks.Chain(layers, N, "f32", tensor_core=tensor_core)
    chain.x.copy_(torch.from_numpy(x.ravel()))
    chain.capture()
    for _ in range(2):  # a replayed graph gives the same bits
        chain.launch()
    chain.stream.synchronize()
    assert _lib.device_status() == 0
    got = chain.y.cpu().numpy().reshape(N, -1)
    used_tc = sum(p is not None for p in chain.prepared)
    assert (used_tc > 0) == bool(tensor_core)
    for n in range(N):
        want = oracle_chain(oracle, layers, x[n])
        # nine convolutions deep: the gate is applied to the network output
        assert rel_max_err(got[n], want) <= 2e-5, (tensor_core, n)
    k, ho, wo = networks.output_shape(layers)
    assert (k, ho, wo) == (125, 2, 2)
    # padded output channels (125 -> 128) hold zeros
    y = P.unpack_activation(got, 128, ho, wo)
    assert np.all(y[:, 125:] == 0)


def test_ds_cnn_chain_bit_exact(oracle):
    layers = networks.ds_cnn(seed=1)
    N = 5
    rng = np.random.default_rng(1)
    x = P.pack_activation(rng.integers(0, 256, (N, 1, 49, 10), dtype=np.uint8))
    chain = networks.Chain(layers, N, "u8")
    chain.x.copy_(torch.from_numpy(x.ravel()))
    chain.capture()
    chain.launch()
    chain.stream.synchronize()
    assert _lib.device_status() == 0
    got = chain.y.cpu().numpy().reshape(N, -1)
    for n in range(N):
        want = oracle_chain(oracle, layers, x[n], "u8")
        assert np.array_equal(got[n], want)
    assert got[:, :12].min() < got[:, :12].max()


def test_work_totals():
    """Algorithmic work per image of the two benchmark networks (hand-computed from the layer shapes)."""
    ly = networks.tiny_yolov2()
    assert abs(sum(networks.algorithmic_work(L, 4)[0] for L in ly if L["op"] == "conv") - 6.971e9) < 1e7
    ld = networks.ds_cnn(calib_images=1)
    assert abs(sum(networks.algorithmic_work(L, 1)[0] for L in ld) - 5.3e6) < 1e5


def _run_chain(layers, x, dtype, **kw):
    N = x.shape[0]
    chain = networks.Chain(layers, N, dtype, **kw)
    chain.x.copy_(torch.from_numpy(x.ravel()))
    chain.capture()
    chain.launch()
    chain.stream.synchronize()
    assert _lib.device_status() == 0
    return chain, chain.y.cpu().numpy().reshape(N, -1)


@pytest.mark.parametrize("tensor_core", [False, "auto"])
def test_resnet8_chain(oracle, tensor_core):
    """ResNet-8: residual stages as PartialConv2D onto the shortcut's buffer
    (include/small/models/Resnet8Tiny.hpp:284-288), stride-2 convolutions, global average pool,
    dense head, softmax."""
    layers = networks.resnet8(seed=0)
    N = 3
    rng = np.random.default_rng(10)
    x = P.pack_activation(rng.random((N, 3, 32, 32), dtype=np.float32))
    chain, got = _run_chain(layers, x, "f32", tensor_core=tensor_core)
    for n in range(N):
        want = oracle_chain(oracle, layers, x[n])
        assert rel_max_err(got[n], want) <= 2e-5
    # 16 padded classes of which 10 are real: probabilities sum to one over all of them
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)


def test_mobilenet_v1_025_chain_fp32(oracle):
    """MobileNet-v1 x0.25 fp32: 13 depthwise-separable blocks with stride-2 depthwise layers."""
    layers = networks.mobilenet_v1_025(seed=2, dtype="f32")
    N = 2
    rng = np.random.default_rng(11)
    x = P.pack_activation(rng.random((N, 3, 96, 96), dtype=np.float32))
    chain, got = _run_chain(layers, x, "f32")
    for n in range(N):
        want = oracle_chain(oracle, layers, x[n])
        assert rel_max_err(got[n], want) <= 2e-5


def test_mobilenet_v1_025_chain_uint8_bit_exact(oracle):
    """MobileNet-v1 x0.25 uint8: every layer requantised, bit-exact through 28 layers."""
    layers = networks.mobilenet_v1_025(seed=2, dtype="u8")
    N = 2
    rng = np.random.default_rng(12)
    x = P.pack_activation(rng.integers(0, 256, (N, 3, 96, 96), dtype=np.uint8))
    chain, got = _run_chain(layers, x, "u8")
    for n in range(N):
        want = oracle_chain(oracle, layers, x[n], "u8")
        assert np.array_equal(got[n], want)
    assert got[:, :2].min() < got[:, :2].max() or got[:, :2].max() > 0


@pytest.mark.parametrize("idx", range(13))
def test_yolov3_tiny_layer(oracle, idx):
    """The 13 convolution shapes of YOLOv3-tiny, each alone, at a reduced image size (channel
    counts, kernel sizes and the 255 -> 256 padding are the real ones); the 416x416 layers are in
    test_gpu_full_size.py."""
    layers = networks.yolov3_tiny_convs(seed=3, size=64)[idx]
    L = layers[0]
    N = 2
    rng = np.random.default_rng(100 + idx)
    x = P.pack_activation(rng.uniform(-1, 1, (N, L["C"], L["H"], L["W"])).astype(np.float32))
    for tc in (False, True):
        if tc and idx == 0:
            continue  # 3 input channels: CUDA-core first-layer kernel only
        chain, got = _run_chain(layers, x, "f32", tensor_core=tc)
        for n in range(N):
            want = oracle_chain(oracle, layers, x[n])
            assert rel_max_err(got[n], want) <= 1e-5, (idx, tc)
