"""Box decoding and non-maximum suppression: the oracle against the reference's golden vectors
(CPU), and the CUDA kernels against the oracle and the goldens (GPU)."""
import os

import numpy as np
import pytest

from smallframework_b200 import packing as P
from tests.util import REFDATA, read_bin, reference_close

ANCHORS_19 = [(116, 90), (156, 198), (373, 326)]   # test/test_yolo.cpp:158, mask 6,7,8


def _golden_19():
    n = 255 * 19 * 19
    x = read_bin(os.path.join(REFDATA, f"in__yolo_Ci255_H19_W19_k0_s0_f_{n}.bin")).reshape(255, 19, 19)
    y = read_bin(os.path.join(REFDATA, f"out__yolo_Ci255_H19_W19_k0_s0_f_{n}.bin")).reshape(3 * 19 * 19, 85)
    xu = np.zeros((1, 256, 19, 19), np.float32)    # 255 channels padded to the block, as the layer before does
    xu[0, :255] = x
    return P.pack_activation(xu)[0], y


def synthetic_predictions(rng, P_, classes, clusters=12, conf=0.25):
    """Records like a YOLO layer's: a few clusters of heavily overlapping boxes with high scores among
    many low-confidence ones; some exactly equal objectness values (the ordering of ties is defined)."""
    pred = np.zeros((P_, classes + 5), np.float32)
    pred[:, 4] = rng.uniform(0, conf * 0.9, P_)
    pred[:, 5:] = rng.uniform(0, conf * 0.9, (P_, classes))
    pred[:, 0:2] = rng.uniform(0, 608, (P_, 2))
    pred[:, 2:4] = rng.uniform(8, 200, (P_, 2))
    for c in range(clusters):
        members = rng.choice(P_, size=int(rng.integers(3, 30)), replace=False)
        centre, size = rng.uniform(50, 550, 2), rng.uniform(30, 250, 2)
        for m in members:
            pred[m, 0:2] = centre + rng.normal(0, size * 0.08)
            pred[m, 2:4] = size * rng.uniform(0.8, 1.25, 2)
            pred[m, 4] = np.float32(rng.uniform(0.3, 1.0)) if rng.random() < 0.8 else np.float32(0.5)
            for cls in rng.choice(classes, size=int(rng.integers(1, 3)), replace=False):
                pred[m, 5 + cls] = rng.uniform(0.3, 1.0)
    return pred


def test_oracle_box_decoding_reproduces_the_reference_golden(oracle):
    xp, y = _golden_19()
    got = oracle.yolo_decode_f32(256, 19, 19, 16, ANCHORS_19, 80, 608 // 19, xp)
    assert reference_close(got, y)            # the reference's own almost_equal (test/test_yolo.cpp:117)
    assert np.abs(got - y).max() <= 1e-4


def test_oracle_nms_keeps_what_a_direct_restatement_keeps(oracle):
    """so_nms_f32 against a few lines of numpy that follow non_max_suppression.hpp:98-155 literally."""
    rng = np.random.default_rng(0)
    pred = synthetic_predictions(rng, 600, 20)
    kept, cand = oracle.nms_f32(pred, 20, 0.25, 0.45)
    dets = [(p, c) for p in range(600) if pred[p, 4] > 0.25 for c in range(20) if pred[p, 5 + c] > 0.25]
    assert cand == len(dets) > 20
    order = sorted(range(len(dets)), key=lambda i: -pred[dets[i][0], 4])   # stable: ties keep collection order
    def iou(a, b):
        f = np.float32
        def ov(x1, w1, x2, w2):
            return min(f(x1 + w1 / f(2)), f(x2 + w2 / f(2))) - max(f(x1 - w1 / f(2)), f(x2 - w2 / f(2)))
        wo, ho = ov(a[0], a[2], b[0], b[2]), ov(a[1], a[3], b[1], b[3])
        inter = f(0) if (wo < 0 or ho < 0) else f(wo * ho)
        return inter / f(f(a[2] * a[3]) + f(b[2] * b[3]) - inter)
    alive, want = [True] * len(order), []
    for i, di in enumerate(order):
        if not alive[i]:
            continue
        want.append(di)
        for j in range(i + 1, len(order)):
            dj = order[j]
            if alive[j] and dets[dj][1] == dets[di][1] and not iou(pred[dets[di][0]], pred[dets[dj][0]]) < 0.45:
                alive[j] = False
    assert len(kept) == len(want) < cand
    for row, di in zip(kept, want):
        p, c = dets[di]
        assert np.array_equal(row[:5], pred[p, :5]) and row[5] == pred[p, 5 + c] and int(row[6]) == c


@pytest.mark.gpu
def test_gpu_box_decoding(oracle):
    import torch
    from smallframework_b200 import interface as S
    xp, y = _golden_19()
    N = 3
    I = S.FloatBuffer(data=np.stack([xp, xp * np.float32(0.5), -xp]))
    O = S.FloatBuffer(N * 3 * 19 * 19 * 85)
    S.YOLODecode(ANCHORS_19, 80, 608, 256, 19, 19, I, O, batch=N)
    torch.cuda.synchronize()
    got = O.numpy().reshape(N, 3 * 19 * 19, 85)
    assert reference_close(got[0], y)
    for n, xin in enumerate((xp, xp * np.float32(0.5), -xp)):
        want = oracle.yolo_decode_f32(256, 19, 19, 16, ANCHORS_19, 80, 608 // 19, xin)
        assert np.abs(got[n] - want).max() <= 2e-6 * max(1.0, float(np.abs(want).max())), n


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(2535, 80, 12, 0), (600, 20, 30, 1), (50, 3, 2, 2), (4000, 80, 60, 3)],
                         ids=lambda c: "P{}_classes{}_clusters{}".format(*c[:3]))
def test_gpu_nms_keeps_exactly_what_the_oracle_keeps(oracle, case):
    from smallframework_b200 import interface as S
    P_, classes, clusters, seed = case
    pred = synthetic_predictions(np.random.default_rng(seed), P_, classes, clusters)
    want, cand = oracle.nms_f32(pred, classes, 0.25, 0.45)
    got = S.NonMaxSuppression(S.FloatBuffer(data=pred), P_, classes, 0.25, 0.45, max_detections=4096)
    assert cand > len(want) > 0
    assert got.shape == want.shape and np.array_equal(got, want)


@pytest.mark.gpu
def test_gpu_nms_reports_overflow_and_empty_input():
    from smallframework_b200 import _lib, interface as S
    pred = synthetic_predictions(np.random.default_rng(4), 600, 20, 30)
    with pytest.raises(_lib.SmallB200Error, match="candidates"):
        S.NonMaxSuppression(S.FloatBuffer(data=pred), 600, 20, 0.25, 0.45, max_candidates=8)
    assert S.NonMaxSuppression(S.FloatBuffer(data=pred), 600, 20, 2.0, 0.45).shape == (0, 7)
