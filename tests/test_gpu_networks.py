"""Whole layer chains (smallframework_b200.networks.Chain, one CUDA graph) against the oracle
run layer by layer: Tiny-YOLOv2 at a reduced image size (the oracle needs seconds per image at
416x416) on both fp32 paths, DS-CNN uint8 at full size, bit-exact."""
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
    """Algorithmic work per image of the two benchmark networks."""
    ly = networks.tiny_yolov2()
    assert abs(sum(networks.algorithmic_work(L, 4)[0] for L in ly if L["op"] == "conv") - 6.971e9) < 1e7
    ld = networks.ds_cnn(calib_images=1)
    assert abs(sum(networks.algorithmic_work(L, 1)[0] for L in ld) - 5.3e6) < 1e5
