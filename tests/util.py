"""Shared helpers of the test-suite: golden-vector loading, shape sampling, and the
predicate that says where the reference's own edge handling is self-consistent."""
from __future__ import annotations

import glob
import os
import re
import struct

import numpy as np

from oracle.bindings import same_pads, shape

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REFDATA = os.path.join(GOLDEN, "reference")


def read_bin(path):
    """Reference golden format (test/test_utils.hpp:187-215): big-endian uint32 count,
    then that many raw float32."""
    with open(path, "rb") as f:
        (n,) = struct.unpack(">I", f.read(4))
        a = np.frombuffer(f.read(4 * n), dtype="<f4")
    assert a.size == n
    return a.copy()


_PAT = re.compile(r"^(in|out|filter)__(\w+?)_Ci(\d+)_H(\d+)_W(\d+)_k(\d+)_s(\d+)_([fv])(?:_Co(\d+))?_(\d+)\.bin$")


def _index():
    idx = {}
    for p in glob.glob(os.path.join(REFDATA, "*.bin")):
        m = _PAT.match(os.path.basename(p))
        if not m:
            continue
        role, kind, ci, h, w, k, s, pad, co, _n = m.groups()
        key = (kind, int(ci), int(h), int(w), int(k), int(s), pad, int(co) if co else 0)
        idx.setdefault(key, {})[role] = p
    return idx


def golden_cases(kind):
    """Cases of one kind with all their files present.
    kind: conv2d | dw_conv | maxpool | averagepool | relu | softmax | partial_bias.
    Yields dicts with C,H,W,k,s,pad,K and arrays x (unpacked CHW), w, y."""
    idx = _index()
    src_kind = {"maxpool": "pool", "averagepool": "pool", "softmax": "pool",
                "partial_bias": "pool"}.get(kind, kind)
    out_kind = {"maxpool": "pool"}.get(kind, kind)
    cases = []
    for key, files in sorted(idx.items()):
        if key[0] != out_kind or "out" not in files:
            continue
        _, ci, h, w, k, s, pad, co = key
        src = idx.get((src_kind, ci, h, w, k, s, pad, co), {})
        if "in" not in src:
            continue
        if kind in ("conv2d", "dw_conv") and "filter" not in files:
            continue
        cases.append(dict(kind=kind, C=ci, H=h, W=w, k=k, s=s, pad=pad, K=co,
                          x=src["in"], w=files.get("filter"), y=files["out"]))
    return cases


def case_id(c):
    return f"{c['kind']}_Ci{c['C']}_H{c['H']}_W{c['W']}_k{c['k']}_s{c['s']}_{c['pad']}_Co{c['K']}"


def case_pads(c):
    return same_pads(c["H"], c["W"], c["k"], c["k"], c["s"]) if c["pad"] == "f" else (0, 0, 0, 0)


def reference_close(a, b, rtol=5e-3, atol=1e-5):
    """almost_equal of the reference's tests, test/test_utils.hpp:41-46."""
    return np.all(np.abs(a - b) <= atol + rtol * np.abs(b))


def axis_defined_in_reference(i, f, s, pf, pb):
    """True where the reference's edge kernels compute what their own interior kernels
    define.  Found by sweeping the compiled reference: it holds when at most ONE output
    element per side touches padding and the trailing one overhangs the image by exactly
    one tap.  (With two padded rows, kernel_top writes both rows' steady-state outputs to
    the same row and moves its valid-row bound the wrong way,
    include/small/abstract_layer.hpp:1291-1292,1351.)"""
    if i < f or pf >= f or pb >= f:  # a window entirely inside padding is degenerate
        return False
    if -(-pf // s) > 1:
        return False
    o = (i + pf + pb - f) // s + 1
    over = [(j * s - pf + f) - i for j in range(o) if j * s - pf + f > i]
    return len(over) == 0 or over == [1]


def defined_in_reference(H, W, Fh, Fw, s, pads):
    t, b, l, r = pads
    return axis_defined_in_reference(H, Fh, s, t, b) and axis_defined_in_reference(W, Fw, s, l, r)


def sample_window_cases(rng, n, channels=(16, 32), first_layer=True, max_hw=14):
    """Random windowed-layer configurations inside the reference's defined domain."""
    out = []
    while len(out) < n:
        C = int(rng.choice(list(channels) + ([1, 2, 3] if first_layer else [])))
        H = int(rng.integers(1, max_hw)); W = int(rng.integers(1, max_hw))
        Fh = int(rng.choice([1, 2, 3, 5])); Fw = int(rng.choice([1, 2, 3, 4]))
        s = int(rng.choice([1, 2]))
        mode = rng.integers(0, 3)
        if mode == 0:
            pads = (0, 0, 0, 0)
        elif mode == 1:
            pads = same_pads(H, W, Fh, Fw, s)
        else:
            pads = tuple(int(v) for v in rng.integers(0, 2, 4))
        if not defined_in_reference(H, W, Fh, Fw, s, pads):
            continue
        out.append((C, H, W, Fh, Fw, s, pads))
    return out
