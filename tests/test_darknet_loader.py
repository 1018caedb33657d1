"""The Darknet loader (smallframework_b200/darknet.py): configuration parsing and weight-file offsets
on the CPU; the whole path -- weight upload, device-side padding / packing / batch-norm folding, the
layer DAG with routes, upsampling, a shortcut and two detection heads, box decoding and NMS -- on the
GPU against the same network walked with the oracle's functions."""
import numpy as np
import pytest

from smallframework_b200 import darknet
from smallframework_b200 import packing as P

CFG = """
[net]
# a two-headed detector in the shape of YOLOv3-tiny, reduced: every section type the loader knows
width=64
height=64
channels=3

[convolutional]
batch_normalize=1
filters=16
size=3
stride=1
pad=1
activation=leaky

[maxpool]
size=2
stride=2

[convolutional]
batch_normalize=1
filters=32
size=3
stride=1
pad=1
activation=leaky

[maxpool]
size=2
stride=2

[convolutional]
batch_normalize=1
filters=32
size=3
stride=1
pad=1
activation=leaky

[shortcut]
from=-2
activation=linear

[maxpool]
size=2
stride=1

[convolutional]
batch_normalize=1
filters=64
size=3
stride=2
pad=1
activation=leaky

[convolutional]
filters=21
size=1
stride=1
pad=1
activation=linear

[yolo]
mask = 3,4,5
anchors = 10,14,  23,27,  37,58,  81,82,  135,169,  344,319
classes=2
num=6

[route]
layers = -3

[convolutional]
batch_normalize=1
filters=16
size=1
stride=1
pad=1
activation=leaky

[upsample]
stride=2

[route]
layers = -1, 6

[convolutional]
filters=21
size=1
stride=1
pad=1
activation=linear

[yolo]
mask = 0,1,2
anchors = 10,14,  23,27,  37,58,  81,82,  135,169,  344,319
classes=2
num=6
"""


def test_plan_shapes_and_weight_offsets():
    shape, plan, total = darknet.build_plan(CFG)
    assert shape == (3, 64, 64)
    ops = [r["op"] for r in plan]
    assert ops == ["conv", "maxpool", "conv", "maxpool", "conv", "shortcut", "maxpool", "conv", "conv", "yolo",
                   "route", "conv", "upsample", "route", "conv", "yolo"]
    assert (plan[0]["Cp"], plan[0]["K"], plan[0]["Ho"]) == (3, 16, 64)
    assert plan[6]["pads"] == (0, 1, 0, 1) and plan[6]["Ho"] == 16          # size 2 stride 1 'same'
    assert (plan[7]["stride"], plan[7]["Ho"]) == (2, 8)
    assert (plan[8]["K"], plan[8]["Kp"]) == (21, 32)                        # 3 anchors x (5 + 2), padded to the block
    assert plan[9]["anchors"] == [(81, 82), (135, 169), (344, 319)] and plan[9]["preds"] == 3 * 8 * 8
    assert plan[10]["parents"] == [7] and plan[13]["parents"] == [12, 6] and plan[13]["K"] == 16 + 32
    assert plan[5]["parents"] == [4, 3]
    offs = [r["w_off"] for r in plan if r["op"] == "conv"]
    sizes = [4 * 16 + 16 * 3 * 9, 4 * 32 + 32 * 16 * 9, 4 * 32 + 32 * 32 * 9, 4 * 64 + 64 * 32 * 9, 21 + 21 * 64, 4 * 16 + 16 * 64,
             21 + 21 * 48]
    assert offs == list(np.cumsum([0] + sizes[:-1])) and total == sum(sizes)
    assert len(darknet.random_weights(CFG)) == darknet.HEADER_BYTES + 4 * total


def test_plan_refuses_what_the_reference_refuses():
    with pytest.raises(ValueError, match="route layer must have only 1 or 2"):
        darknet.build_plan(CFG.replace("layers = -1, 6", "layers = -1, 6, 2"))
    with pytest.raises(ValueError, match="unsupported section"):
        darknet.build_plan(CFG + "\n[dropout]\nprobability=.5\n")
    with pytest.raises(ValueError, match="incorrect input buffer shape"):
        darknet.build_plan(CFG.replace("classes=2", "classes=3"))


def oracle_walk(oracle, cfg, weights, x_packed):
    """The network of `cfg` for ONE packed image, layer by layer on the oracle."""
    from oracle.bindings import shape
    _, plan, n = darknet.build_plan(cfg)
    w = np.frombuffer(weights, np.float32, offset=darknet.HEADER_BYTES, count=n)
    outs, heads = [], []
    src = lambda i: x_packed if i < 0 else outs[i]
    for r in plan:
        a = src(r["parents"][0])
        if r["op"] == "conv":
            k, c, f, o = r["K"], r["C"], r["size"], r["w_off"]
            if r["bn"]:
                beta, gamma, mean, var = (w[o + j * k:o + (j + 1) * k] for j in range(4))
                filt = w[o + 4 * k:o + 4 * k + k * c * f * f].reshape(k, c, f, f)
                pf, pb = oracle.conv_weights_prepare_f32(r["Kp"], filt, None, (gamma, beta, mean, var), darknet.BN_EPS)
            else:
                filt = w[o + k:o + k + k * c * f * f].reshape(k, c, f, f)
                pf, pb = oracle.conv_weights_prepare_f32(r["Kp"], filt, w[o:o + k], None, 0.0)
            sh = shape(r["Cp"], r["Kp"], r["H"], r["W"], f, f, r["stride"], r["pads"], 16)
            outs.append(oracle.conv2d_f32(sh, a, pf, bias=pb, act=r["act"], slope=darknet.LEAKY_SLOPE))
        elif r["op"] == "maxpool":
            sh = shape(r["Cp"], r["Kp"], r["H"], r["W"], r["size"], r["size"], r["stride"], r["pads"], 16)
            outs.append(oracle.pool2d_f32(sh, a))
        elif r["op"] == "upsample":
            outs.append(oracle.upsample2d_f32(r["Cp"], r["H"], r["W"], 16, 2, a))
        elif r["op"] == "route":
            outs.append(a if len(r["parents"]) == 1 else np.concatenate([a, src(r["parents"][1])]))
        elif r["op"] == "shortcut":
            outs.append(oracle.accum_f32(src(r["parents"][1]), a))
        elif r["op"] == "yolo":
            outs.append(oracle.yolo_decode_f32(r["Cp"], r["H"], r["W"], 16, r["anchors"], r["classes"], r["img"] // r["H"], a))
            heads.append(outs[-1])
    return heads


@pytest.mark.gpu
@pytest.mark.parametrize("tensor_core", [False, "auto"])
def test_loaded_network_matches_the_oracle_walk(oracle, tensor_core):
    import torch
    from tests.gpu_util import rel_max_err
    weights = darknet.random_weights(CFG, seed=3)
    N = 3
    rng = np.random.default_rng(5)
    x = P.pack_activation(rng.random((N, 3, 64, 64), dtype=np.float32))
    model = darknet.DarknetModel(CFG, weights, batch=N, tensor_core=tensor_core)
    heads = [h.cpu().numpy() for h in model.inference(x)]
    torch.cuda.synchronize()
    assert [h.shape for h in heads] == [(N, 192, 7), (N, 768, 7)]
    for n in range(N):
        want = oracle_walk(oracle, CFG, weights, x[n])
        for got, ref in zip(heads, want):
            assert rel_max_err(got[n], ref) <= 2e-5, (tensor_core, n)
    # detections: the device pipeline on its own records against the oracle's NMS on the same records
    dets = model.detect(x, confidence_threshold=0.5, iou_threshold=0.45)
    for n in range(N):
        rec = np.concatenate([h[n] for h in heads])
        want, cand = oracle.nms_f32(rec, 2, 0.5, 0.45)
        assert cand > 0 and np.array_equal(dets[n], want)
