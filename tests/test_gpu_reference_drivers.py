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


# ---- the reference's demo programs (demo/CMakeLists.txt:26-78), built unchanged
FUSED_DRIVERS = ["conv_fused_MAX_POOL", "conv_fused_MAX_POOL_n_bias", "conv_fused_MAX_POOL_n_bias_n_relu",
                 "conv_fused_DW_CONV", "conv_fused_DW_CONV_n_bias", "conv_fused_DW_CONV_n_bias_n_relu"]
# <C_i> <H> <W>  conv <k> <stride> <pad>  <C_o>  second layer <k> <stride> <pad> <C_o>
FUSED_ARGS = {
    "MAX_POOL": [["16", "32", "32", "3", "1", "f", "32", "2", "2", "v", "32"],      # one kernel (pool in registers)
                 ["32", "13", "13", "3", "1", "f", "64", "3", "2", "v", "64"],      # 3x3 pool: two kernels
                 ["3", "64", "64", "3", "1", "f", "16", "2", "2", "v", "16"]],      # first layer
    "DW_CONV": [["16", "24", "24", "1", "1", "v", "32", "3", "1", "f", "32"],
                ["32", "12", "12", "3", "1", "f", "64", "3", "2", "f", "64"]],
}


@pytest.mark.parametrize("name", FUSED_DRIVERS)
def test_reference_fused_block_driver(name):
    """demo/fused_block_driver.cpp (conv_fused_*.exe of the reference's build): a fused call
    (Conv2D[_Bias][_ReLU]_Maxpool2D / ..._DepthwiseConv2D...) against the unfused pair of calls, with the
    driver's own element-wise check (it asserts)."""
    exe = os.path.join(BUILD, "bin", name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    for argv in FUSED_ARGS["MAX_POOL" if "MAX_POOL" in name else "DW_CONV"]:
        r = subprocess.run([exe] + argv, cwd=os.path.join(BUILD, "run"), env=dict(os.environ, OMP_NUM_THREADS="4"),
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
        tail = "\n".join(r.stdout.splitlines()[-15:])
        assert r.returncode == 0, f"{name} {' '.join(argv)} failed (rc {r.returncode}):\n{tail}"


MODEL_DEMOS = ["model_mobilenet", "model_mobilenet_reshuffled", "model_resnet", "model_resnet_1D", "model_dscnn",
               "model_dscnn_square", "model_autoencoder", "model_tinyyolov2"]


@pytest.mark.parametrize("name", MODEL_DEMOS)
def test_reference_model_demo(name):
    """The reference's model demos (model_*.exe): each builds its network from the functional interface
    and from the Layer classes, compares the two and times them."""
    exe = os.path.join(BUILD, "bin", name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    r = subprocess.run([exe], cwd=os.path.join(BUILD, "run"), env=dict(os.environ, OMP_NUM_THREADS="4"),
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1800)
    tail = "\n".join(r.stdout.splitlines()[-15:])
    assert r.returncode == 0, f"{name} failed (rc {r.returncode}):\n{tail}"


def test_every_fused_form_through_the_small_boundary():
    """tests/drivers/fused_forms.cpp: the 15 fused 2-D functions, the 1-D family with stride 2, UpSample1D
    and Dropout through the small:: headers, each against the unfused composition or a direct loop."""
    exe = os.path.join(BUILD, "bin", "fused_forms")
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (run make -C tests/reference_drivers where the reference is mounted)")
    r = subprocess.run([exe], env=dict(os.environ, OMP_NUM_THREADS="4"), stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=900)
    print(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-3000:]
