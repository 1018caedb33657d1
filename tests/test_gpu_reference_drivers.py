"""The reference's own test drivers (test/test_*.cpp of the reference, compiled UNCHANGED
against include/small/platforms/b200 by tests/reference_drivers/Makefile) run on the GPU.

Each driver packs its data with BufferT::C_ib / C_ob = 16, calls the small:: functions (which
on this platform forward to libsmall_b200.so) and compares with the reference's golden
vectors or closed forms.  The binaries and the data travel in tests/reference_drivers/_build
(built where the reference tree is mounted); without them the tests are skipped, not passed.
"""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "reference_drivers", "_build")

DRIVERS = ["test_buffer", "test_tensor", "test_packing", "test_conv2d", "test_conv2d_rect",
           "test_partial_conv2d", "test_dw_conv", "test_maxpool", "test_averagepool", "test_relu",
           "test_leaky", "test_softmax", "test_partial_bias", "test_shortcut", "test_upsample2d",
           "test_route_concat", "test_tinyyolov2", "test_resnet8", "test_dscnn",
           "test_dscnn_square", "test_mobilenet", "test_autoencoder", "test_conv1d"]

# Sub-tests that need files the reference's own checkout lacks (its .MISSING_LARGE_BLOBS);
# they fail on every platform, the CPU ones included.
SKIP = {"test_conv2d": ["conv2d_batchnorm"]}  # needs out__conv2d_Ci3_H416_W416_k3_s1_f_Co16_2768896.bin


@pytest.mark.parametrize("name", DRIVERS)
def test_reference_driver(name):
    exe = os.path.join(BUILD, "bin", name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    cmd = [exe]
    if name in SKIP:
        cmd += ["--skip"] + SKIP[name]
    env = dict(os.environ, OMP_NUM_THREADS="4")
    r = subprocess.run(cmd, cwd=os.path.join(BUILD, "run"), env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=900)
    tail = "\n".join(r.stdout.splitlines()[-25:])
    assert r.returncode == 0, f"{name} failed:\n{tail}"


# The platform runs fp32 convolutions on the tensor cores by default; the drivers that contain fp32
# convolutions are run once more with every convolution kept on the CUDA cores.
CONV_DRIVERS = ["test_conv2d", "test_conv2d_rect", "test_partial_conv2d", "test_tinyyolov2", "test_resnet8",
                "test_autoencoder", "test_mobilenet", "test_dscnn", "test_dscnn_square", "test_conv1d"]


@pytest.mark.parametrize("name", CONV_DRIVERS)
def test_reference_driver_on_cuda_cores_only(name):
    exe = os.path.join(BUILD, "bin", name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    cmd = [exe]
    if name in SKIP:
        cmd += ["--skip"] + SKIP[name]
    env = dict(os.environ, OMP_NUM_THREADS="4", SMALL_B200_TENSOR_CORE="0")
    r = subprocess.run(cmd, cwd=os.path.join(BUILD, "run"), env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=900)
    tail = "\n".join(r.stdout.splitlines()[-25:])
    assert r.returncode == 0, f"{name} failed with SMALL_B200_TENSOR_CORE=0:\n{tail}"


def _tiny_yolov2_model_on_the_oracle(oracle, size, filters, image):
    """include/small/models/TinyYoloV2.hpp:161-240 layer by layer on the CPU restatement: six blocks of
    Conv2D 3x3 'same' + ReLU and MaxPool2D 2x2 'same' (strides 2,2,2,2,2,1), two Conv2D 3x3 + ReLU to
    1024 channels, one Conv2D 1x1 + ReLU to 16 channels.  Filters arrive packed."""
    import numpy as np
    from oracle.bindings import same_pads, shape
    chans = [3, 16, 32, 64, 128, 256, 512, 1024, 1024, 16]
    cur, h = image, size
    for l in range(9):
        k = 1 if l == 8 else 3
        sh = shape(chans[l], chans[l + 1], h, h, k, k, 1, same_pads(h, h, k, k, 1), 16)
        cur = oracle.conv2d_f32(sh, cur, filters[l], act=1)
        if l < 6:
            s = 2 if l < 5 else 1
            shp = shape(chans[l + 1], chans[l + 1], h, h, 2, 2, s, same_pads(h, h, 2, 2, s), 16)
            cur = oracle.pool2d_f32(shp, cur)
            h = shp.out_hw()[0]
    return cur


@pytest.mark.parametrize("tensor_core", ["0", "1"])
def test_model_classes_as_cuda_graph(oracle, tensor_core, tmp_path):
    """tests/drivers/model_graph.cpp: the reference's TinyYoloV2 Model class run eagerly, recorded with
    small::b200::InferenceGraph and replayed (bit-identical), and batched with BatchScope (every image
    equals its single-image result).  The model's output for one 416x416 image is then recomputed from
    the driver's own filters and image on the oracle (bit-identical to the reference's REF build)."""
    import numpy as np
    exe = os.path.join(BUILD, "bin", "model_graph")
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    env = dict(os.environ, OMP_NUM_THREADS="4", SMALL_B200_TENSOR_CORE=tensor_core)
    r = subprocess.run([exe, "416", "3", "10", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=900)
    tail = "\n".join(l for l in r.stdout.splitlines() if not l.startswith("Model::dtor"))[-2000:]
    print(tail)
    assert r.returncode == 0, f"model_graph failed (SMALL_B200_TENSOR_CORE={tensor_core}):\n{tail}"
    load = lambda name: np.fromfile(os.path.join(tmp_path, name), dtype=np.float32)
    want = _tiny_yolov2_model_on_the_oracle(oracle, 416, [load(f"f{l}.bin") for l in range(9)], load("image.bin"))
    got = load("out.bin")
    assert got.shape == want.shape
    err = float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())
    print(f"TinyYoloV2 Model class vs the oracle, SMALL_B200_TENSOR_CORE={tensor_core}: {err:.2e}")
    assert err <= 1e-4
