"""Helpers shared by the GPU parity tests: run one layer through the C ABI (via the Python
mirror of the reference interface) and through the oracle, image by image."""
from __future__ import annotations

import numpy as np
import torch

from oracle.bindings import Quant, shape
from smallframework_b200 import interface as S
from smallframework_b200 import packing as P

CB = P.CB


def rel_max_err(got, want):
    """max |got - want| / max |want|: the error measure of the fp32 gate (1e-5)."""
    denom = float(np.abs(want).max())
    return float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max()) / (denom if denom > 0 else 1.0)


def fbuf(a):
    return S.FloatBuffer(data=np.ascontiguousarray(a, np.float32))


def qbuf(a, zero=128, like=None):
    b = S.QUInt8Buffer(data=np.ascontiguousarray(a, np.uint8))
    b.m_zero = zero
    return b


def oracle_conv_batch(oracle, sh, xs, wp, bias=None, act=0, slope=0.0, seed=None, depthwise=False):
    outs = []
    for n in range(xs.shape[0]):
        outs.append(oracle.conv2d_f32(sh, xs[n], wp, bias=bias, act=act, slope=slope,
                                      out=None if seed is None else seed[n], depthwise=depthwise))
    return np.stack(outs)


def oracle_layer(oracle, L, first, cur, dtype="f32", seed=None):
    """One layer of a layer list (smallframework_b200.networks format) on the oracle for ONE
    packed image `cur`, blocking 16, output channels padded like the executor pads them.
    `seed`: the destination's previous content for a layer with `accumulate` (PartialConv2D)."""
    from smallframework_b200.networks import padded, padded_params
    cin = L["C"] if first else padded(L["C"])
    kp = padded(L["K"])
    sh = shape(cin, kp, L["H"], L["W"], L["Fh"], L["Fw"], L["stride"], L["pads"], CB)
    if L["op"] in ("conv", "dwconv"):
        dw = L["op"] == "dwconv"
        w, b = padded_params(L, first, dtype)
        if dtype == "f32":
            return oracle.conv2d_f32(sh, cur, w, bias=b, act=L.get("act", 0), slope=L.get("slope", 0.0),
                                     out=seed, depthwise=dw)
        q = L["q"]
        return oracle.conv2d_u8(sh, Quant(q["zero_in"], q["zero_filt"], q["lshift"], q["rshift"],
                                          q["multiplier"], 0), cur, w, bias=b, depthwise=dw)
    if L["op"] == "softmax":
        return oracle.softmax_f32(cin, L["H"], L["W"], CB, cur)
    if L["op"] == "alias":
        return cur
    avg = L["op"] == "avgpool"
    if dtype == "f32":
        return oracle.pool2d_f32(sh, cur, average=avg)
    q = L["q"] if "q" in L else dict(zero_in=0, zero_filt=0, lshift=0, rshift=0, multiplier=1 << 30)
    return oracle.pool2d_u8(sh, Quant(q["zero_in"], 0, q["lshift"], q["rshift"], q["multiplier"], 0),
                            cur, average=avg)


def oracle_chain(oracle, layers, x_packed, dtype="f32"):
    """One image through a layer list on the oracle.  Layers that name their buffers (src / dst,
    residual stages) read and write a dictionary of tensors; `accumulate` seeds the convolution
    with the destination's content (PartialConv2D)."""
    cur = x_packed
    named = {"in": x_packed}
    for i, L in enumerate(layers):
        if "src" in L:
            cur = named[L["src"]]
        seed = named[L["dst"]].copy() if (L.get("accumulate") and dtype == "f32") else None
        cur = oracle_layer(oracle, L, i == 0, cur, dtype, seed)
        if "dst" in L:
            named[L["dst"]] = cur
    return cur


def run_layers_checked(oracle, chain, layers, images, dtype="f32", tol=1e-5):
    """Runs `chain` eagerly, one layer call at a time, and after each call compares the images
    in `images` with the oracle applied to THE SAME INPUT the device kernel read (so a layer's
    error is its own, not the chain's).  Layers that their producer absorbs (a max pool, a depthwise
    convolution, the pool + dense tail) are checked together with that producer.  Returns per-layer (name, worst error) -- errors are max|x-ref|/max|ref| for
    fp32 and the count of differing bytes for uint8."""
    from smallframework_b200 import _lib
    from smallframework_b200.networks import _out_hw, padded
    st = chain.stream.cuda_stream
    plan = chain.io_plan()
    report = []
    N = chain.batch
    for i, io in enumerate(plan):
        if io is None:
            continue
        L = layers[i]
        if L["op"] == "alias":
            continue
        src, dst = io
        chain.stream.synchronize()
        cin = L["C"] if i == 0 else padded(L["C"])
        n_in = cin * L["H"] * L["W"]
        follow = chain.absorbed(i)
        last = layers[follow[-1]] if follow else L
        ho, wo = _out_hw(last)
        n_out = padded(last["K"]) * ho * wo
        xin = {n: src[n * n_in:(n + 1) * n_in].cpu().numpy() for n in images}
        before = {n: dst[n * n_out:(n + 1) * n_out].cpu().numpy() for n in images} if L.get("accumulate") else {}
        chain.enqueue_layer(i, src, dst, st)
        chain.stream.synchronize()
        assert _lib.device_status() == 0, L["name"]
        worst = 0.0
        for n in images:
            want = oracle_layer(oracle, L, i == 0, xin[n], dtype, before.get(n))
            for k in follow:
                want = oracle_layer(oracle, layers[k], False, want, dtype)
            got = dst[n * n_out:(n + 1) * n_out].cpu().numpy()
            if dtype == "f32":
                err = rel_max_err(got, want)
                assert err <= tol, (L["name"], n, err)
            else:
                err = float(np.count_nonzero(got != want))
                assert err == 0, (L["name"], n, err)
            worst = max(worst, err)
        report.append(("+".join([L["name"]] + [layers[k]["name"] for k in follow]), worst))
    return report
