"""ctypes bindings for the checker libraries (TEST INFRASTRUCTURE).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import this module; the product package never does.

  Oracle  -> oracle/libsmall_oracle.so   (plain-C restatement, small_oracle.c)
  Ref     -> oracle/_ref/libsmall_{ref,zen2}.so  (the unmodified reference compiled
             from its own headers by oracle/Makefile; ref_shim.cpp)

All arrays are numpy arrays in SMaLL's packed layout for ONE image.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("C", "K", "H", "W", "Fh", "Fw", "stride",
                 "pad_t", "pad_b", "pad_l", "pad_r", "cib", "cob")]

    def out_hw(self):
        ho = max((self.H + self.pad_t + self.pad_b - self.Fh) // self.stride + 1, 0)
        wo = max((self.W + self.pad_l + self.pad_r - self.Fw) // self.stride + 1, 0)
        return ho, wo


class Quant(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("zero_in", "zero_filt", "lshift", "rshift", "multiplier", "k_zero")]


class RefLayer(C.Structure):
    _fields_ = [("op", C.c_int32), ("s", Shape), ("act", C.c_int32), ("slope", C.c_float),
                ("filt", C.c_void_p), ("bias", C.c_void_p), ("q", Quant)]


def shape(C_, K, H, W, Fh, Fw, stride, pads, cib, cob=None):
    t, b, l, r = pads
    return Shape(C_, K, H, W, Fh, Fw, stride, t, b, l, r, cib, cob if cob is not None else cib)


def same_pads(H, W, Fh, Fw, stride):
    """TF-style 'same' padding, include/small/utils.hpp:43-64; returns (t, b, l, r)."""
    def one(i, k):
        p = max(k - stride, 0) if i % stride == 0 else max(k - (i % stride), 0)
        return p // 2, p - p // 2
    t, b = one(H, Fh)
    l, r = one(W, Fw)
    return t, b, l, r


def build(reference_dir: str | None = None) -> None:
    """Compile the checker libraries (the C restatement always; the reference shims
    only where the reference tree is present)."""
    cmd = ["make", "-s", "-C", HERE]
    if reference_dir:
        cmd.append(f"REFERENCE_DIR={reference_dir}")
    subprocess.run(cmd, check=True)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        path = os.path.join(HERE, "libsmall_oracle.so")
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        self.lib.so_requant.restype = C.c_int32
        self.lib.so_requant.argtypes = [C.c_int32] * 4

    # -- float
    def conv2d_f32(self, s, x, f, bias=None, act=0, slope=0.0, out=None, depthwise=False):
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        accumulate = out is not None
        o = _f32(out).copy() if accumulate else np.zeros(k * ho * wo, np.float32)
        b = _f32(bias) if bias is not None else None
        fn = self.lib.so_dwconv2d_f32 if depthwise else self.lib.so_conv2d_f32
        x, f = _f32(x), _f32(f)
        fn(C.byref(s), _p(x), _p(f), _p(b), C.c_int(act), C.c_float(slope),
           C.c_int(int(accumulate)), _p(o))
        return o

    def groupconv2d_f32(self, s, groups, x, f, bias=None, act=0, slope=0.0, out=None):
        """`groups` convolutions s.C -> s.K; s.cob is the group block."""
        ho, wo = s.out_hw()
        accumulate = out is not None
        o = _f32(out).copy() if accumulate else np.zeros(groups * s.K * ho * wo, np.float32)
        b = _f32(bias) if bias is not None else None
        x, f = _f32(x), _f32(f)
        self.lib.so_groupconv2d_f32(C.byref(s), C.c_int32(groups), _p(x), _p(f), _p(b), C.c_int(act),
                                    C.c_float(slope), C.c_int(int(accumulate)), _p(o))
        return o

    def pool2d_f32(self, s, x, average=False):
        ho, wo = s.out_hw()
        o = np.zeros(s.C * ho * wo, np.float32)
        x = _f32(x)
        (self.lib.so_avgpool2d_f32 if average else self.lib.so_maxpool2d_f32)(C.byref(s), _p(x), _p(o))
        return o

    def relu_f32(self, x):
        x = _f32(x); o = np.empty_like(x)
        self.lib.so_relu_f32(C.c_int64(x.size), _p(x), _p(o)); return o

    def leaky_relu_f32(self, x, slope):
        x = _f32(x); o = np.empty_like(x)
        self.lib.so_leaky_relu_f32(C.c_int64(x.size), _p(x), C.c_float(slope), _p(o)); return o

    def accum_f32(self, x, out):
        x = _f32(x); o = _f32(out).copy()
        self.lib.so_accum_f32(C.c_int64(x.size), _p(x), _p(o)); return o

    def bias_f32(self, Cn, H, W, cb, bias, out=None):
        o = _f32(out).copy() if out is not None else np.zeros(Cn * H * W, np.float32)
        b = _f32(bias)
        self.lib.so_bias_f32(Cn, H, W, cb, _p(b), C.c_int(int(out is not None)), _p(o)); return o

    def upsample2d_f32(self, Cn, H, W, cb, scale, x):
        x = _f32(x); o = np.zeros(Cn * H * W * scale * scale, np.float32)
        self.lib.so_upsample2d_f32(Cn, H, W, cb, scale, _p(x), _p(o)); return o

    def softmax_f32(self, Cn, H, W, cb, x):
        x = _f32(x); o = np.empty_like(x)
        self.lib.so_softmax_f32(Cn, H, W, cb, _p(x), _p(o)); return o

    # -- uint8
    def requant(self, acc, lshift, rshift, mult):
        return self.lib.so_requant(int(acc), lshift, rshift, mult)

    def conv2d_u8(self, s, q, x, f, bias=None, depthwise=False):
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        o = np.zeros(k * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        b = np.ascontiguousarray(bias, dtype=np.int32) if bias is not None else None
        fn = self.lib.so_dwconv2d_u8 if depthwise else self.lib.so_conv2d_u8
        fn(C.byref(s), C.byref(q), _p(x), _p(f), _p(b), _p(o))
        return o

    def partial_conv2d_u8(self, s, q, x, f, partial, depthwise=False):
        """One block of output channels; `partial` = int32 [Ho*Wo*block] (see small_oracle.h)."""
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        assert k == s.cob
        o = np.zeros(k * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        part = np.ascontiguousarray(partial, dtype=np.int32)
        assert part.size == o.size
        fn = self.lib.so_partial_dwconv2d_u8 if depthwise else self.lib.so_partial_conv2d_u8
        fn(C.byref(s), C.byref(q), _p(x), _p(f), _p(part), _p(o))
        return o

    def groupconv2d_u8(self, s, q, groups, x, f, bias=None):
        ho, wo = s.out_hw()
        o = np.zeros(groups * s.K * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        b = np.ascontiguousarray(bias, dtype=np.int32) if bias is not None else None
        self.lib.so_groupconv2d_u8(C.byref(s), C.byref(q), C.c_int32(groups), _p(x), _p(f), _p(b), _p(o))
        return o

    def pool2d_u8(self, s, q, x, average=False):
        ho, wo = s.out_hw()
        o = np.zeros(s.C * ho * wo, np.uint8)
        x = _u8(x)
        (self.lib.so_avgpool2d_u8 if average else self.lib.so_maxpool2d_u8)(
            C.byref(s), C.byref(q), _p(x), _p(o))
        return o

    def relu_u8(self, q, x):
        x = _u8(x); o = np.empty_like(x)
        self.lib.so_relu_u8(C.c_int64(x.size), C.byref(q), _p(x), _p(o)); return o

    def conv_weights_prepare_f32(self, K, w, bias=None, bn=None, eps=1e-5, cb=16):
        """w: [Keff, C, Fh, Fw]; bn: (gamma, beta, mean, var) or None.  Returns (packed filters, packed bias or None)."""
        Keff, Cn, Fh, Fw = w.shape
        w = _f32(w)
        packed = np.zeros(K * Cn * Fh * Fw, np.float32)
        pb = np.zeros(K, np.float32) if (bias is not None or bn is not None) else None
        b = _f32(bias) if bias is not None else None
        g = [_f32(v) for v in bn] if bn is not None else [None] * 4
        self.lib.so_conv_weights_prepare_f32(K, Keff, Cn, Fh, Fw, cb, _p(w), _p(b), _p(g[0]), _p(g[1]), _p(g[2]), _p(g[3]),
                                             C.c_float(eps), _p(packed), _p(pb))
        return packed, pb

    # -- detection head
    def yolo_decode_f32(self, Cp, H, W, cb, anchors, num_classes, stride, x):
        """anchors: list of (w, h); returns [len(anchors)*H*W, 5 + num_classes]."""
        x = _f32(x)
        a = _f32(np.asarray(anchors, np.float32).ravel())
        o = np.zeros((len(anchors) * H * W, num_classes + 5), np.float32)
        self.lib.so_yolo_decode_f32(Cp, H, W, cb, len(anchors), num_classes, C.c_float(stride), _p(a), _p(x), _p(o))
        return o

    def nms_f32(self, pred, num_classes, conf_thr, iou_thr, max_det=4096):
        """pred: [P, 5 + num_classes]; returns (kept rows [n, 7], candidates above the threshold)."""
        pred = _f32(pred)
        o = np.zeros((max_det, 7), np.float32)
        cand = C.c_int32(0)
        self.lib.so_nms_f32.restype = C.c_int32
        n = self.lib.so_nms_f32(_p(pred), pred.shape[0], num_classes, C.c_float(conf_thr), C.c_float(iou_thr),
                                max_det, _p(o), C.byref(cand))
        return o[:min(n, max_det)], cand.value


class Ref:
    """The unmodified reference behind ref_shim.cpp.  platform: 'ref' or 'zen2'."""

    def __init__(self, platform="ref"):
        path = os.path.join(HERE, "_ref", f"libsmall_{platform}.so")
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: run `make -C oracle` on a machine that has the reference tree")
        self.lib = C.CDLL(path)
        self.lib.ref_last_error.restype = C.c_char_p
        self.float_cb = self.lib.ref_float_cb()
        self.quint8_cb = self.lib.ref_quint8_cb()
        self.has_quint8 = bool(self.lib.ref_has_quint8())
        self.platform = platform

    def _check(self, rc):
        if rc == 1:
            raise ValueError(self.lib.ref_last_error().decode())
        if rc != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def set_threads(self, n):
        self.lib.ref_set_threads(int(n))

    def conv2d_f32(self, s, x, f, out=None, depthwise=False):
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        o = _f32(out).copy() if out is not None else np.zeros(k * ho * wo, np.float32)
        x, f = _f32(x), _f32(f)
        fn = self.lib.ref_dwconv2d_f32 if depthwise else self.lib.ref_conv2d_f32
        self._check(fn(C.byref(s), _p(x), _p(f), C.c_int(int(out is not None)), _p(o)))
        return o

    def pool2d_f32(self, s, x, average=False):
        ho, wo = s.out_hw()
        o = np.zeros(s.C * ho * wo, np.float32)
        x = _f32(x)
        self._check(self.lib.ref_pool2d_f32(C.byref(s), C.c_int(int(average)), _p(x), _p(o)))
        return o

    def eltwise_f32(self, op, Cn, H, W, x, slope=0.0, out=None):
        code = {"relu": 0, "leaky": 1, "accum": 2, "softmax": 3, "upsample": 4}[op]
        x = _f32(x)
        n = Cn * H * W * (4 if op == "upsample" else 1)
        o = _f32(out).copy() if out is not None else np.zeros(n, np.float32)
        self._check(self.lib.ref_eltwise_f32(code, Cn, H, W, C.c_float(slope), _p(x), _p(o)))
        return o

    def bias_f32(self, Cn, H, W, bias, out=None):
        o = _f32(out).copy() if out is not None else np.zeros(Cn * H * W, np.float32)
        b = _f32(bias)
        self._check(self.lib.ref_bias_f32(Cn, H, W, _p(b), C.c_int(int(out is not None)), _p(o)))
        return o

    def conv2d_u8(self, s, q, x, f, depthwise=False):
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        o = np.zeros(k * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        self._check(self.lib.ref_conv2d_u8(C.byref(s), C.byref(q), C.c_int(int(depthwise)),
                                           _p(x), _p(f), _p(o)))
        return o

    def partial_conv2d_u8(self, s, q, x, f, partial, depthwise=False):
        """small::PartialConv2D / PartialDepthwiseConv2D<QUInt8Buffer> on one block of output channels
        (this build's block is 1 channel): the int32 partial sums are placed at the start of the
        four-times over-allocated output buffer, as the loop nest expects them."""
        ho, wo = s.out_hw()
        k = s.C if depthwise else s.K
        o = np.zeros(k * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        part = np.ascontiguousarray(partial, dtype=np.int32)
        assert part.size == o.size
        self._check(self.lib.ref_partial_conv2d_u8(C.byref(s), C.byref(q), C.c_int(int(depthwise)),
                                                   _p(x), _p(f), _p(part), _p(o)))
        return o

    def groupconv2d_f32(self, s, groups, x, f, out=None):
        """small::GroupConv2D / PartialGroupConv2D: `groups` groups of s.C channels each."""
        ho, wo = s.out_hw()
        o = _f32(out).copy() if out is not None else np.zeros(groups * s.C * ho * wo, np.float32)
        x, f = _f32(x), _f32(f)
        self._check(self.lib.ref_groupconv2d_f32(C.byref(s), C.c_int(groups), _p(x), _p(f),
                                                 C.c_int(int(out is not None)), _p(o)))
        return o

    def groupconv2d_u8(self, s, q, groups, x, f):
        ho, wo = s.out_hw()
        o = np.zeros(groups * s.C * ho * wo, np.uint8)
        x, f = _u8(x), _u8(f)
        self._check(self.lib.ref_groupconv2d_u8(C.byref(s), C.byref(q), C.c_int(groups), _p(x), _p(f), _p(o)))
        return o

    def maxpool2d_u8(self, s, q, x):
        ho, wo = s.out_hw()
        o = np.zeros(s.C * ho * wo, np.uint8)
        x = _u8(x)
        self._check(self.lib.ref_maxpool2d_u8(C.byref(s), C.byref(q), _p(x), _p(o)))
        return o

    def relu_u8(self, Cn, H, W, q, x):
        x = _u8(x); o = np.empty_like(x)
        self._check(self.lib.ref_relu_u8(Cn, H, W, C.byref(q), _p(x), _p(o)))
        return o

    def run_chain(self, layers, x, images, threads, out_elems, dtype="f32"):
        """layers: list of dicts(op, s, act, slope, filt, bias, q). Returns (seconds, out)."""
        arr = (RefLayer * len(layers))()
        keep = []
        for i, L in enumerate(layers):
            arr[i].op = {"conv": 0, "dwconv": 1, "maxpool": 2, "avgpool": 3}[L["op"]]
            arr[i].s = L["s"]
            arr[i].act = L.get("act", 0)
            arr[i].slope = L.get("slope", 0.0)
            for key in ("filt", "bias"):
                a = L.get(key)
                if a is not None:
                    a = np.ascontiguousarray(a)
                    keep.append(a)
                    setattr(arr[i], key, a.ctypes.data)
            if "q" in L:
                arr[i].q = L["q"]
        sec = C.c_double(0)
        if dtype == "f32":
            x = _f32(x); o = np.zeros(out_elems, np.float32)
            fn = self.lib.ref_run_chain_f32
        else:
            x = _u8(x); o = np.zeros(out_elems, np.uint8)
            fn = self.lib.ref_run_chain_u8
        self._check(fn(arr, len(layers), _p(x), C.c_size_t(x.size), int(images), int(threads),
                       _p(o), C.c_size_t(out_elems), C.byref(sec)))
        return sec.value, o
