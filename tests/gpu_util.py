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
