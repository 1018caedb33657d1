"""Parity at the sizes the benchmark runs, layer by layer, against the oracle (which is
bit-identical to the reference's REF build): Tiny-YOLOv2 at 416x416 on both fp32 paths (two
images alone, and two sampled images of a 64-image launch, which is what takes the persistent
multi-tile loops, the wide-image tiling and the two-CTA split reduction through several
waves), the 13 YOLOv3-tiny convolutions at 416x416, DS-CNN uint8 at batch 4096 and
MobileNet-v1 x0.25 uint8 at batch 2048 with sampled images, bit-exact.

Every layer is compared on the input the device kernel itself read, so the 1e-5 gate
(max|x - ref| / max|ref|) applies to each layer on its own; the error of the whole network
against the oracle's own chain is reported and held to 1e-4."""
import numpy as np
import pytest
import torch

from smallframework_b200 import _lib, networks
from smallframework_b200 import packing as P
from tests.gpu_util import oracle_chain, rel_max_err, run_layers_checked

pytestmark = pytest.mark.gpu


def _fill(chain, x):
    chain.x.copy_(torch.from_numpy(np.ascontiguousarray(x).reshape(-1)))


def _show(title, report):
    print("\n" + title + ": " + ", ".join(f"{n} {e:.2e}" for n, e in report))


@pytest.mark.parametrize("tensor_core", [False, "auto"])
def test_tiny_yolov2_416_two_images_per_layer(oracle, tensor_core):
    """include/small/models/TinyYoloV2.hpp:92-135 at its real size; the reference holds its own
    model to its function chain the same way (test/test_tinyyolov2.cpp:624-747)."""
    layers = networks.tiny_yolov2(seed=4, size=416)
    N = 2
    rng = np.random.default_rng(40)
    x = P.pack_activation(rng.random((N, 3, 416, 416), dtype=np.float32))
    chain = networks.Chain(layers, N, "f32", tensor_core=tensor_core)
    _fill(chain, x)
    report = run_layers_checked(oracle, chain, layers, range(N))
    _show(f"Tiny-YOLOv2 416x416 tensor_core={tensor_core} per-layer error", report)
    # the whole network as one CUDA graph against the oracle's own chain
    chain.capture()
    chain.launch()
    chain.stream.synchronize()
    assert _lib.device_status() == 0
    got = chain.y.cpu().numpy().reshape(N, -1)
    errs = [rel_max_err(got[n], oracle_chain(oracle, layers, x[n])) for n in range(N)]
    print(f"network output error tensor_core={tensor_core}: {max(errs):.2e}")
    assert max(errs) <= 1e-4
    assert networks.output_shape(layers) == (125, 13, 13)


@pytest.mark.parametrize("tensor_core", [False, "auto"])
def test_tiny_yolov2_416_batch64_sampled_images(oracle, tensor_core):
    """The launch the benchmark times: 64 images per GPU.  conv8 then is 512 tiles = 1024 CTAs in
    clusters of two over several waves, conv2/conv3 walk many tiles per persistent CTA."""
    layers = networks.tiny_yolov2(seed=4, size=416)
    N = 64
    g = torch.Generator(device="cuda").manual_seed(41)
    chain = networks.Chain(layers, N, "f32", tensor_core=tensor_core)
    chain.x.copy_(torch.rand(chain.x.numel(), device="cuda", generator=g))
    report = run_layers_checked(oracle, chain, layers, (0, 37, 63))
    _show(f"Tiny-YOLOv2 416x416 batch 64 tensor_core={tensor_core} per-layer error", report)


@pytest.mark.parametrize("idx", range(13))
def test_yolov3_tiny_layer_416(oracle, idx):
    """The 13 convolution shapes of YOLOv3-tiny at 416x416 (test/cfg_data/yolov3-tiny.cfg), each
    alone, on the CUDA cores and (where covered) on the tensor cores."""
    layers = networks.yolov3_tiny_convs(seed=3, size=416)[idx]
    L = layers[0]
    N = 2
    rng = np.random.default_rng(300 + idx)
    x = P.pack_activation(rng.uniform(-1, 1, (N, L["C"], L["H"], L["W"])).astype(np.float32))
    for tc in (False, True):
        if tc and idx == 0:
            continue  # 3 input channels: CUDA-core first-layer kernel only
        chain = networks.Chain(layers, N, "f32", tensor_core=tc)
        assert (chain.prepared[0] is not None) == tc
        _fill(chain, x)
        report = run_layers_checked(oracle, chain, layers, range(N))
        _show(f"y3t{idx} {L['C']}->{L['K']} {L['Fh']}x{L['Fw']} @{L['H']} tensor_core={tc}", report)


def test_conv_1024_to_1024_13x13_many_clusters(oracle):
    """The split reduction (two CTAs per tile) with far more clusters than SMs: 40 images x 8
    channel tiles = 320 tiles = 640 CTAs."""
    L = dict(op="conv", name="deep", C=1024, K=1024, H=13, W=13, Fh=3, Fw=3, stride=1, pads=(1, 1, 1, 1),
             act=2, slope=0.1)
    rng = np.random.default_rng(77)
    L["w"] = rng.normal(0, np.sqrt(2 / (1024 * 9)), (1024, 1024, 3, 3)).astype(np.float32)
    L["b"] = rng.uniform(-0.1, 0.1, 1024).astype(np.float32)
    N = 40
    chain = networks.Chain([L], N, "f32", tensor_core=True)
    assert chain.prepared[0] is not None
    g = torch.Generator(device="cuda").manual_seed(78)
    chain.x.copy_(torch.rand(chain.x.numel(), device="cuda", generator=g) * 2 - 1)
    report = run_layers_checked(oracle, chain, [L], (0, 19, 39))
    _show("1024->1024 3x3 @13 batch 40", report)


def test_ds_cnn_batch4096_sampled_images_bit_exact(oracle):
    """DS-CNN uint8 at the benchmark's batch: the persistent tensor-core kernels walk many tiles
    per CTA; sampled images, every layer, bit-exact."""
    layers = networks.ds_cnn(seed=1)
    N = 4096
    g = torch.Generator(device="cuda").manual_seed(42)
    chain = networks.Chain(layers, N, "u8")
    chain.x.copy_(torch.randint(0, 256, (chain.x.numel(),), device="cuda", generator=g, dtype=torch.uint8))
    xin = chain.x.cpu().numpy().reshape(N, -1)
    sample = (0, 1, 127, 128, 2047, 3000, 4095)
    report = run_layers_checked(oracle, chain, layers, sample, dtype="u8")
    _show("DS-CNN batch 4096 differing bytes per layer", report)
    chain.capture()
    chain.launch()
    chain.stream.synchronize()
    assert _lib.device_status() == 0
    got = chain.y.cpu().numpy().reshape(N, -1)
    for n in sample:
        assert np.array_equal(got[n], oracle_chain(oracle, layers, xin[n], "u8")), n


def test_mobilenet_u8_batch2048_sampled_images_bit_exact(oracle):
    """MobileNet-v1 x0.25 uint8 (include/small/models/MobileNetTiny.hpp) at batch 2048."""
    layers = networks.mobilenet_v1_025(seed=2, dtype="u8")
    N = 2048
    g = torch.Generator(device="cuda").manual_seed(43)
    chain = networks.Chain(layers, N, "u8")
    chain.x.copy_(torch.randint(0, 256, (chain.x.numel(),), device="cuda", generator=g, dtype=torch.uint8))
    report = run_layers_checked(oracle, chain, layers, (0, 1023, 2047), dtype="u8")
    _show("MobileNet-v1 x0.25 uint8 batch 2048 differing bytes per layer", report)


def test_mobilenet_f32_batch2048_sampled_images(oracle):
    """MobileNet-v1 x0.25 fp32 at batch 2048: the 1x1 layers on small images run with the batch as
    the rows of one image (tiles that span images)."""
    layers = networks.mobilenet_v1_025(seed=2, dtype="f32")
    N = 2048
    g = torch.Generator(device="cuda").manual_seed(44)
    chain = networks.Chain(layers, N, "f32")
    chain.x.copy_(torch.rand(chain.x.numel(), device="cuda", generator=g))
    report = run_layers_checked(oracle, chain, layers, (0, 1023, 2047))
    _show("MobileNet-v1 x0.25 fp32 batch 2048 per-layer error", report)


def test_resnet8_batch1024_sampled_images(oracle):
    """ResNet-8 (include/small/models/Resnet8Tiny.hpp) at batch 1024, residual stages as
    PartialConv2D onto the shortcut's buffer."""
    layers = networks.resnet8(seed=0)
    N = 1024
    g = torch.Generator(device="cuda").manual_seed(45)
    chain = networks.Chain(layers, N, "f32")
    chain.x.copy_(torch.rand(chain.x.numel(), device="cuda", generator=g))
    report = run_layers_checked(oracle, chain, layers, (0, 511, 1023))
    _show("ResNet-8 batch 1024 per-layer error", report)
