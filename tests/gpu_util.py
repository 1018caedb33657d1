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


def oracle_chain(oracle, layers, x_packed, dtype="f32"):
    """One image through a layer list (smallframework_b200.networks format) on the oracle,
    blocking 16, padded output channels like the executor.  Layers that name their buffers
    (src / dst, residual stages) read and write a dictionary of tensors; `accumulate` seeds the
    convolution with the destination's content (PartialConv2D)."""
    from smallframework_b200.networks import padded, padded_params
    cur = x_packed
    named = {"in": x_packed}
    for i, L in enumerate(layers):
        if "src" in L:
            cur = named[L["src"]]
        cin = L["C"] if i == 0 else padded(L["C"])
        kp = padded(L["K"])
        sh = shape(cin, kp, L["H"], L["W"], L["Fh"], L["Fw"], L["stride"], L["pads"], CB)
        if L["op"] in ("conv", "dwconv"):
            dw = L["op"] == "dwconv"
            w, b = padded_params(L, i == 0, dtype)
            if dtype == "f32":
                seed = named[L["dst"]].copy() if L.get("accumulate") else None
                cur = oracle.conv2d_f32(sh, cur, w, bias=b, act=L.get("act", 0), slope=L.get("slope", 0.0),
                                        out=seed, depthwise=dw)
            else:
                q = L["q"]
                cur = oracle.conv2d_u8(sh, Quant(q["zero_in"], q["zero_filt"], q["lshift"], q["rshift"],
                                                 q["multiplier"], 0), cur, w, bias=b, depthwise=dw)
        elif L["op"] == "softmax":
            cur = oracle.softmax_f32(cin, L["H"], L["W"], CB, cur)
        elif L["op"] == "alias":
            pass
        else:
            avg = L["op"] == "avgpool"
            if dtype == "f32":
                cur = oracle.pool2d_f32(sh, cur, average=avg)
            else:
                q = L["q"] if "q" in L else dict(zero_in=0, zero_filt=0, lshift=0, rshift=0, multiplier=1 << 30)
                cur = oracle.pool2d_u8(sh, Quant(q["zero_in"], 0, q["lshift"], q["rshift"], q["multiplier"], 0),
                                       cur, average=avg)
        if "dst" in L:
            named[L["dst"]] = cur
    return cur
