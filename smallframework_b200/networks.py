"""Layer chains of the benchmark configurations and their executor.

The reference drives the functional interface from fixed layer lists with two ping-pong
buffers (include/small/models/TinyYoloV2.hpp:92-135, demo/tinyyolov2.cpp:263-386,
include/small/models/DSCNNTiny.hpp).  `Chain` does the same against the C ABI: packed
weights are uploaded once, every layer call is enqueued on one stream, and the whole
sequence is captured in a CUDA graph so that a step is a single graph launch.

Weights are random (seeded); there are no checkpoints.  A layer list is a list of dicts:
  op      conv | dwconv | maxpool | avgpool
  C, K    input / output channels (K = effective count; filters are zero-padded to a
          multiple of 16 like include/small/Conv2DLayer.hpp:393-404 does)
  H, W, Fh, Fw, stride, pads(t, b, l, r)
  act     0 none, 1 ReLU, 2 LeakyReLU (slope)
  w, b    unpacked [K, C, Fh, Fw] (dw: [C, Fh, Fw]) weights and per-channel bias
  q       uint8 only: dict(zero_in, zero_filt, lshift, rshift, multiplier)
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from ._lib import Layer, check, lib
from .packing import CB, calc_padding, output_dim, pack_conv_filter, pack_dw_filter


def _same(H, W, Fh, Fw, s):
    t, b = calc_padding(H, Fh, s)
    l, r = calc_padding(W, Fw, s)
    return (t, b, l, r)


def _out_hw(L):
    t, b, l, r = L["pads"]
    return (output_dim(L["H"], t, b, L["Fh"], L["stride"]),
            output_dim(L["W"], l, r, L["Fw"], L["stride"]))


def _he(rng, shape_, fan_in):
    return rng.normal(0.0, math.sqrt(2.0 / fan_in), shape_).astype(np.float32)


# --------------------------------------------------------------------------- Tiny-YOLOv2 fp32
def tiny_yolov2(seed=4, size=416):
    """Eight 3x3 same-pad convolutions (16..1024, 1024) each with bias + LeakyReLU(0.1);
    2x2 max pool after the first six (stride 2 five times, then stride 1 with pads
    (0,1,0,1), demo/tinyyolov2.cpp:504-507); a final 1x1 convolution to 125 channels.
    He-normal weights, biases uniform in [-0.1, 0.1]."""
    rng = np.random.default_rng(seed)
    chans = [16, 32, 64, 128, 256, 512, 1024, 1024]
    layers, c, h = [], 3, size
    for i, k in enumerate(chans):
        layers.append(dict(op="conv", name=f"conv{i + 1}", C=c, K=k, H=h, W=h, Fh=3, Fw=3, stride=1,
                           pads=_same(h, h, 3, 3, 1), act=2, slope=0.1,
                           w=_he(rng, (k, c, 3, 3), c * 9),
                           b=rng.uniform(-0.1, 0.1, k).astype(np.float32)))
        c = k
        if i < 5:
            layers.append(dict(op="maxpool", name=f"maxpool{i + 1}", C=c, K=c, H=h, W=h, Fh=2, Fw=2,
                               stride=2, pads=(0, 0, 0, 0)))
            h //= 2
        elif i == 5:
            layers.append(dict(op="maxpool", name="maxpool6", C=c, K=c, H=h, W=h, Fh=2, Fw=2,
                               stride=1, pads=(0, 1, 0, 1)))
    layers.append(dict(op="conv", name="conv9", C=c, K=125, H=h, W=h, Fh=1, Fw=1, stride=1,
                       pads=(0, 0, 0, 0), act=0, slope=0.0, w=_he(rng, (125, c, 1, 1), c),
                       b=rng.uniform(-0.1, 0.1, 125).astype(np.float32)))
    return layers


# --------------------------------------------------------------------------- DS-CNN uint8
def _requant_params(scale):
    """scale = multiplier * 2^-31 * 2^-rshift with the multiplier in [2^30, 2^31)."""
    rshift = int(np.clip(math.floor(-math.log2(scale)), 0, 30))
    mult = int(np.clip(round(scale * 2.0 ** (31 + rshift)), 1, (1 << 31) - 1))
    return 0, rshift, mult


def _calibrate(x, w, bias, zi, zf, stride, pads, depthwise):
    """int64 accumulators of a few images, computed with torch on the CPU (set-up only):
    zero padding of the SHIFTED input equals skipping padded taps."""
    xs = torch.from_numpy(x.astype(np.float64) + zi)
    ws = torch.from_numpy(w.astype(np.float64) + zf)
    t, b, l, r = pads
    xs = torch.nn.functional.pad(xs, (l, r, t, b))
    groups = xs.shape[1] if depthwise else 1
    if depthwise:
        ws = ws[:, None]
    acc = torch.nn.functional.conv2d(xs, ws, stride=stride, groups=groups)
    return acc.numpy() + bias.astype(np.float64)[None, :, None, None]


def ds_cnn(seed=1, calib_images=8):
    """DS-CNN keyword spotting, uint8: stem 10x4 stride 2 same-pad to 64 channels; four blocks
    of depthwise 3x3 + pointwise 1x1 (64 channels); average pool 25x5; dense 64 -> 12.
    Every convolution ends in the requantisation whose clamp to [0, 255] is the ReLU.
    Weights are uniform bytes with zero point 128, which in the reference's convention of
    ADDED offsets (intrinsics_quint8.h:201) is zero_filt = -128; the network input has zero
    point 128 (zero_in = -128), later activations 0.  Biases are int32 in [-1024, 1024].
    Multipliers are calibrated on a few seeded images so activations span 0..255."""
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, (calib_images, 1, 49, 10)).astype(np.uint8)
    layers = []

    def add(op, name, C_, K, H, W, Fh, Fw, s, pads, zi, cur):
        depthwise = op == "dwconv"
        wshape = (C_, Fh, Fw) if depthwise else (K, C_, Fh, Fw)
        w = rng.integers(0, 256, wshape).astype(np.uint8)
        b = rng.integers(-1024, 1025, K).astype(np.int32)
        acc = _calibrate(cur, w, b, zi, -128, s, pads, depthwise)
        top = max(float(np.percentile(acc, 99.9)), 1.0)
        lshift, rshift, mult = _requant_params(255.0 / top)
        layers.append(dict(op=op, name=name, C=C_, K=K, H=H, W=W, Fh=Fh, Fw=Fw, stride=s, pads=pads,
                           act=0, slope=0.0, w=w, b=b,
                           q=dict(zero_in=zi, zero_filt=-128, lshift=lshift, rshift=rshift,
                                  multiplier=mult)))
        nxt = np.clip(np.rint(acc * (mult * 2.0 ** (-31 - rshift))), 0, 255).astype(np.uint8)
        return nxt

    cur = add("conv", "stem", 1, 64, 49, 10, 10, 4, 2, _same(49, 10, 10, 4, 2), -128, x)
    for i in range(4):
        cur = add("dwconv", f"dw{i + 1}", 64, 64, 25, 5, 3, 3, 1, _same(25, 5, 3, 3, 1), 0, cur)
        cur = add("conv", f"pw{i + 1}", 64, 64, 25, 5, 1, 1, 1, (0, 0, 0, 0), 0, cur)
    # average pool: sum of 125 taps requantised by 1/125
    lshift, rshift, mult = _requant_params(1.0 / 125.0)
    layers.append(dict(op="avgpool", name="avgpool", C=64, K=64, H=25, W=5, Fh=25, Fw=5, stride=1,
                       pads=(0, 0, 0, 0),
                       q=dict(zero_in=0, zero_filt=0, lshift=lshift, rshift=rshift, multiplier=mult)))
    pooled = np.clip(np.rint(cur.astype(np.float64).sum(axis=(2, 3), keepdims=True) / 125.0), 0, 255
                     ).astype(np.uint8)
    add("conv", "dense", 64, 12, 1, 1, 1, 1, 1, (0, 0, 0, 0), 0, pooled)
    return layers


# --------------------------------------------------------------------------- ResNet-8 fp32
def resnet8(seed=0, size=32):
    """ResNet-8 of the MLCommons-Tiny image-classification model the reference's
    include/small/models/Resnet8Tiny.hpp builds: stem conv 3x3 16ch + ReLU; three residual stages
    (16 ch stride 1 identity shortcut; 32 ch stride 2 and 64 ch stride 2 with 1x1 stride-2
    convolution shortcuts), each conv3x3 + ReLU, conv3x3, add, ReLU; global average pool;
    dense 64 -> 10 (a 1x1 convolution on the 1x1 image); softmax.  The add is done the way the
    reference does it (Resnet8Tiny.hpp:284-288): the second convolution is a PartialConv2D that
    accumulates onto the shortcut's buffer, with the ReLU in the same kernel here.
    Layers name their buffers (src/dst): this list is a small DAG.  He-normal weights, biases 0."""
    rng = np.random.default_rng(seed)
    L, h = [], size
    conv = lambda name, c, k, hh, f, s, act, src, dst, acc=0: dict(
        op="conv", name=name, C=c, K=k, H=hh, W=hh, Fh=f, Fw=f, stride=s, pads=_same(hh, hh, f, f, s),
        act=act, slope=0.0, w=_he(rng, (k, c, f, f), c * f * f), b=None, src=src, dst=dst, accumulate=acc)
    L.append(conv("stem", 3, 16, h, 3, 1, 1, "in", "x"))
    # stage 1: identity shortcut -> accumulate onto the stage input itself
    L.append(conv("s1a", 16, 16, h, 3, 1, 1, "x", "a"))
    L.append(conv("s1b", 16, 16, h, 3, 1, 1, "a", "x", acc=1))
    c = 16
    for st, k in ((2, 32), (3, 64)):
        L.append(conv(f"s{st}a", c, k, h, 3, 2, 1, "x", "a"))
        L.append(conv(f"s{st}sc", c, k, h, 1, 2, 0, "x", "y"))
        h //= 2
        L.append(conv(f"s{st}b", k, k, h, 3, 1, 1, "a", "y", acc=1))
        L.append(dict(op="alias", name=f"s{st}out", src="y", dst="x", C=k, K=k, H=h, W=h, Fh=1, Fw=1, stride=1,
                      pads=(0, 0, 0, 0)))
        c = k
    L.append(dict(op="avgpool", name="avgpool", C=c, K=c, H=h, W=h, Fh=h, Fw=h, stride=1, pads=(0, 0, 0, 0),
                  src="x", dst="p"))
    L.append(dict(op="conv", name="dense", C=c, K=10, H=1, W=1, Fh=1, Fw=1, stride=1, pads=(0, 0, 0, 0), act=0,
                  slope=0.0, w=_he(rng, (10, c, 1, 1), c), b=None, src="p", dst="d"))
    L.append(dict(op="softmax", name="softmax", C=10, K=10, H=1, W=1, Fh=1, Fw=1, stride=1, pads=(0, 0, 0, 0),
                  src="d", dst="o"))
    return L


# --------------------------------------------------------------------------- MobileNet-v1 x0.25
def mobilenet_v1_025(seed=2, size=96, dtype="f32"):
    """MobileNet-v1 width 0.25 (include/small/models/MobileNetTiny.hpp): stem conv 3x3 8ch stride 2;
    13 depthwise-separable blocks (channels 16,32,32,64,64,128,128x5,256,256; stride 2 at blocks
    2,4,6,12), every convolution followed by ReLU; average pool 3x3; dense 256 -> 2; softmax (fp32).
    uint8: zero points as in ds_cnn(), multipliers calibrated on a few seeded images."""
    rng = np.random.default_rng(seed)
    chans = [16, 32, 32, 64, 64, 128, 128, 128, 128, 128, 128, 256, 256]
    strides = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]
    u8 = dtype == "u8"
    cur = rng.integers(0, 256, (2, 3, size, size)).astype(np.uint8) if u8 else None
    L = []

    def add(op, name, C_, K, H, Fh, s, zi):
        nonlocal cur
        pads = _same(H, H, Fh, Fh, s)
        dw = op == "dwconv"
        wshape = (C_, Fh, Fh) if dw else (K, C_, Fh, Fh)
        d = dict(op=op, name=name, C=C_, K=K, H=H, W=H, Fh=Fh, Fw=Fh, stride=s, pads=pads, act=0 if u8 else 1,
                 slope=0.0)
        if u8:
            w = rng.integers(0, 256, wshape).astype(np.uint8)
            b = rng.integers(-1024, 1025, K).astype(np.int32)
            acc = _calibrate(cur, w, b, zi, -128, s, pads, dw)
            top = max(float(np.percentile(acc, 99.9)), 1.0)
            lshift, rshift, mult = _requant_params(255.0 / top)
            d.update(w=w, b=b, q=dict(zero_in=zi, zero_filt=-128, lshift=lshift, rshift=rshift, multiplier=mult))
            cur = np.clip(np.rint(acc * (mult * 2.0 ** (-31 - rshift))), 0, 255).astype(np.uint8)
        else:
            d.update(w=_he(rng, wshape, (1 if dw else C_) * Fh * Fh), b=None)
        L.append(d)

    h = size
    add("conv", "stem", 3, 8, h, 3, 2, -128)
    h //= 2
    c = 8
    for i, (k, s) in enumerate(zip(chans, strides)):
        add("dwconv", f"dw{i + 1}", c, c, h, 3, s, 0)
        h //= s
        add("conv", f"pw{i + 1}", c, k, h, 1, 1, 0)
        c = k
    if u8:
        lshift, rshift, mult = _requant_params(1.0 / (h * h))
        L.append(dict(op="avgpool", name="avgpool", C=c, K=c, H=h, W=h, Fh=h, Fw=h, stride=1, pads=(0, 0, 0, 0),
                      q=dict(zero_in=0, zero_filt=0, lshift=lshift, rshift=rshift, multiplier=mult)))
        cur = np.clip(np.rint(cur.astype(np.float64).sum(axis=(2, 3), keepdims=True) / (h * h)), 0, 255).astype(np.uint8)
        add("conv", "dense", c, 2, 1, 1, 1, 0)
    else:
        L.append(dict(op="avgpool", name="avgpool", C=c, K=c, H=h, W=h, Fh=h, Fw=h, stride=1, pads=(0, 0, 0, 0)))
        L.append(dict(op="conv", name="dense", C=c, K=2, H=1, W=1, Fh=1, Fw=1, stride=1, pads=(0, 0, 0, 0), act=0,
                      slope=0.0, w=_he(rng, (2, c, 1, 1), c), b=None))
        L.append(dict(op="softmax", name="softmax", C=2, K=2, H=1, W=1, Fh=1, Fw=1, stride=1, pads=(0, 0, 0, 0)))
    return L


# --------------------------------------------------------------------------- YOLOv3-tiny layer sweep
def yolov3_tiny_convs(seed=3, size=416):
    """The 13 convolution layers of YOLOv3-tiny at 416x416 (test/cfg_data/yolov3-tiny.cfg:26-173 of
    the reference), each a one-layer list to be timed alone: inputs U[-1,1), weights N(0, 0.05),
    bias + LeakyReLU(0.1) except the two linear 1x1 heads.  255 output channels pad to 256."""
    rng = np.random.default_rng(seed)
    s = size
    spec = [(3, 16, s, 3, 2), (16, 32, s // 2, 3, 2), (32, 64, s // 4, 3, 2), (64, 128, s // 8, 3, 2),
            (128, 256, s // 16, 3, 2), (256, 512, s // 32, 3, 2), (512, 1024, s // 32, 3, 2),
            (1024, 256, s // 32, 1, 2), (256, 512, s // 32, 3, 2), (512, 255, s // 32, 1, 0),
            (256, 128, s // 32, 1, 2), (384, 256, s // 16, 3, 2), (256, 255, s // 16, 1, 0)]
    out = []
    for i, (c, k, h, f, act) in enumerate(spec):
        out.append([dict(op="conv", name=f"y3t{i}", C=c, K=k, H=h, W=h, Fh=f, Fw=f, stride=1,
                         pads=_same(h, h, f, f, 1), act=act, slope=0.1,
                         w=rng.normal(0.0, 0.05, (k, c, f, f)).astype(np.float32),
                         b=rng.uniform(-0.1, 0.1, k).astype(np.float32))])
    return out


def input_shape(layers):
    L = layers[0]
    return (L["C"], L["H"], L["W"])


def output_shape(layers):
    L = layers[-1]
    ho, wo = _out_hw(L)
    return (L["K"], ho, wo)


def padded(k):
    return -(-k // CB) * CB


def padded_params(L, first, dtype):
    """(packed filter, bias) of a conv / dwconv layer with channel counts rounded up to the block
    of 16 the way include/small/Conv2DLayer.hpp:393-404 pads odd channel counts: filters of padded
    OUTPUT channels and weights of padded INPUT channels contribute nothing (zero for fp32; for
    uint8 the byte whose shifted value w + zero_filt is 0), padded biases are 0."""
    kp = padded(L["K"])
    zero_w = 0
    if dtype == "u8":
        zf = L["q"]["zero_filt"]
        zero_w = np.uint8(-zf) if -zf in range(256) else 0
    if L["op"] == "conv":
        cp = L["C"] if first else padded(L["C"])
        w = np.full((kp, cp) + L["w"].shape[2:], zero_w, L["w"].dtype)
        w[:L["K"], :L["C"]] = L["w"]
        wt = pack_conv_filter(w)
    else:
        w = np.full((kp,) + L["w"].shape[1:], zero_w, L["w"].dtype)
        w[:L["K"]] = L["w"]
        wt = pack_dw_filter(w)
    b = None
    if L.get("b") is not None:
        b = np.zeros(kp, L["b"].dtype)
        b[:L["K"]] = L["b"]
    return wt, b


def algorithmic_work(L, elt):
    """(flops, bytes) of one image: 2*Ho*Wo*K*C*Fh*Fw for a dense convolution, all taps
    counted; bytes = input + output activations plus weights and bias once per launch
    (returned separately as the third value)."""
    ho, wo = _out_hw(L)
    taps = L["Fh"] * L["Fw"]
    if L["op"] == "conv":
        flops = 2 * ho * wo * L["K"] * L["C"] * taps
        wbytes = L["K"] * L["C"] * taps * elt + L["K"] * 4
    elif L["op"] == "dwconv":
        flops = 2 * ho * wo * L["C"] * taps
        wbytes = L["C"] * taps * elt + L["C"] * 4
    elif L["op"] in ("softmax", "alias"):
        flops, wbytes = ho * wo * L["C"], 0
    else:
        flops = ho * wo * L["C"] * taps
        wbytes = 0
    abytes = (L["C"] * L["H"] * L["W"] + L["K"] * ho * wo) * elt
    return flops, abytes, wbytes


# --------------------------------------------------------------------------- executor
class Chain:
    """A layer list bound to device memory for a fixed batch.

    enqueue(stream) issues every layer through the C ABI; capture() records that sequence
    into a CUDA graph; launch() replays it.  `x` (input) and `y` (output) are the device
    tensors at the two ends."""

    def __init__(self, layers, batch, dtype="f32", device="cuda", tensor_core="auto", fuse_pool=True,
                 fuse_u8=True):
        """tensor_core: "auto" = fp32 convolutions run on the tensor cores where the library
        prefers them there (small_b200_conv2d_f32_tf32x3_preferred); True = every covered
        layer; False = CUDA cores only.  fuse_pool: a CUDA-core convolution followed by a 2x2
        stride-2 max pool runs as one kernel where the library covers the pair (the reference's
        Conv2D_Bias_ReLU_Maxpool2D path); the pool's entry in `fused_into` then names its
        producer and enqueue_layer() does nothing for it.  fuse_u8: a uint8 convolution followed by a
        3x3 depthwise convolution (the reference's Conv2D_ReLU_DepthwiseConv2D_ReLU pairing), or by the
        global average pool and the dense layer that end the keyword-spotting network, runs as one kernel
        where the library covers the shapes; the absorbed layers are entered in `fused_into` likewise."""
        self.layers, self.batch, self.dtype = layers, batch, dtype
        self.fuse_pool = fuse_pool
        self.tensor_core = tensor_core
        self.tdtype = torch.float32 if dtype == "f32" else torch.uint8
        self.elt = 4 if dtype == "f32" else 1
        self.dev = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.dev)
        c, h, w = input_shape(layers)
        self.x = torch.zeros(batch * c * h * w, dtype=self.tdtype, device=self.dev)
        max_act = 0
        self.params = []
        for L in layers:
            ho, wo = _out_hw(L)
            kp = padded(L["K"])
            max_act = max(max_act, batch * kp * ho * wo)
            if L["op"] == "alias":
                self.params.append((None, None))
                continue
            wt = bs = None
            if L["op"] in ("conv", "dwconv"):
                w_np, b_np = padded_params(L, len(self.params) == 0, dtype)
                wt = torch.from_numpy(w_np).to(self.dev)
                if b_np is not None:
                    bs = torch.from_numpy(b_np).to(self.dev)
            self.params.append((wt, bs))
        self.bufs = [torch.zeros(max_act, dtype=self.tdtype, device=self.dev) for _ in range(2)]
        # layers that name their buffers (a small DAG, e.g. residual stages) get one tensor per name
        self.named = {"in": self.x}
        for L in layers:
            for key in ("src", "dst"):
                if key in L and L[key] not in self.named:
                    self.named[L[key]] = torch.zeros(max_act, dtype=self.tdtype, device=self.dev)
        # tensor-core fp32 path: filters re-laid once (hi + lo copies)
        self.prepared = [None] * len(layers)
        if dtype == "f32" and tensor_core:
            for i, L in enumerate(layers):
                if L["op"] != "conv" or (i == 0 and L["C"] % CB != 0):
                    continue
                d = self._desc(L, padded(L["C"]))
                # "auto": the library's own choice (the C++ platform headers ask the same function)
                if tensor_core == "auto" and not lib().small_b200_conv2d_f32_tf32x3_preferred(C.byref(d)):
                    continue
                if not lib().small_b200_conv2d_f32_tf32x3_supported(C.byref(d)):
                    continue
                wt = self.params[i][0]
                prep = torch.empty(2 * wt.numel(), dtype=torch.float32, device=self.dev)
                check(lib().small_b200_filter_prepare_tf32x3(C.byref(d), wt.data_ptr(), prep.data_ptr(),
                                                             torch.cuda.current_stream().cuda_stream))
                self.prepared[i] = prep
            torch.cuda.synchronize()
        self.fused_into = {}  # index of a max pool -> index of the convolution that absorbs it
        if dtype == "f32" and fuse_pool:
            for i in range(len(layers) - 1):
                L, Pn = layers[i], layers[i + 1]
                if L["op"] != "conv" or Pn["op"] != "maxpool" or "src" in L:
                    continue
                dc = self._desc(L, L["C"] if i == 0 else padded(L["C"]))
                dp = self._desc(Pn, padded(Pn["C"]))
                if self.prepared[i] is not None:
                    # tensor-core convolution: the pool runs in its epilogue where the library covers the pair
                    if lib().small_b200_conv2d_maxpool_f32_tf32x3_supported(C.byref(dc), C.byref(dp)):
                        self.fused_into[i + 1] = i
                    continue
                if lib().small_b200_conv2d_maxpool_f32_supported(C.byref(dc), C.byref(dp)):
                    self.fused_into[i + 1] = i
        if dtype == "u8" and fuse_u8:
            i = 0
            while i < len(layers) - 1:
                L = layers[i]
                if L["op"] == "conv" and "src" not in L:
                    dc = self._desc(L, L["C"] if i == 0 else padded(L["C"]))
                    nxt = layers[i + 1]
                    if nxt["op"] == "dwconv" and lib().small_b200_conv2d_dwconv2d_u8_supported(
                            C.byref(dc), C.byref(self._desc(nxt, padded(nxt["C"])))):
                        self.fused_into[i + 1] = i
                        i += 2
                        continue
                    if (nxt["op"] == "avgpool" and i + 2 < len(layers) and layers[i + 2]["op"] == "conv" and
                            lib().small_b200_conv2d_avgpool_dense_u8_supported(
                                C.byref(dc), C.byref(self._desc(nxt, padded(nxt["C"]))),
                                C.byref(self._desc(layers[i + 2], padded(layers[i + 2]["C"]))))):
                        self.fused_into[i + 1] = i
                        self.fused_into[i + 2] = i
                        i += 3
                        continue
                i += 1
        self.graph = None
        self.graphs = []
        self.y = None
        self.kernels_per_step = 0
        self._descs = []

    def absorbed(self, i):
        """Indices of the layers that run inside layer i's kernel, in order."""
        return sorted(k for k, v in self.fused_into.items() if v == i)

    def _desc(self, L, cin):
        t, b, l, r = L["pads"]
        q = L.get("q", {})
        return Layer(self.batch, cin, padded(L["K"]), L["H"], L["W"], L["Fh"], L["Fw"], L["stride"],
                     t, b, l, r, L.get("accumulate", 0), L.get("act", 0), L.get("slope", 0.0),
                     q.get("zero_in", 0), q.get("zero_filt", 0), q.get("lshift", 0),
                     q.get("rshift", 0), q.get("multiplier", 0), 0)

    def enqueue_layer(self, i, src, dst, stream):
        L = self.layers[i]
        wt, bs = self.params[i]
        cin = L["C"] if i == 0 else padded(L["C"])
        d = self._desc(L, cin)
        sfx = "f32" if self.dtype == "f32" else "u8"
        l = lib()
        p = lambda t: t.data_ptr() if t is not None else None
        if i in self.fused_into:
            return  # computed by its producer
        follow = self.absorbed(i)
        if L["op"] == "conv" and follow and self.dtype == "u8":
            ds = [self._desc(self.layers[k], padded(self.layers[k]["C"])) for k in follow]
            w2, b2 = self.params[follow[-1]]
            if len(follow) == 1:
                check(l.small_b200_conv2d_dwconv2d_u8(C.byref(d), C.byref(ds[0]), p(src), p(wt), p(bs), p(w2), p(b2),
                                                      p(dst), stream))
            else:
                check(l.small_b200_conv2d_avgpool_dense_u8(C.byref(d), C.byref(ds[0]), C.byref(ds[1]), p(src), p(wt),
                                                           p(bs), p(w2), p(b2), p(dst), stream))
        elif L["op"] == "conv" and follow and self.prepared[i] is not None:
            dp = self._desc(self.layers[i + 1], padded(self.layers[i + 1]["C"]))
            check(l.small_b200_conv2d_maxpool_f32_tf32x3(C.byref(d), C.byref(dp), p(src), p(self.prepared[i]), p(bs),
                                                         p(dst), stream))
        elif L["op"] == "conv" and follow:
            dp = self._desc(self.layers[i + 1], padded(self.layers[i + 1]["C"]))
            check(l.small_b200_conv2d_maxpool_f32(C.byref(d), C.byref(dp), p(src), p(wt), p(bs), p(dst), stream))
        elif L["op"] == "conv" and self.prepared[i] is not None:
            check(l.small_b200_conv2d_f32_tf32x3(C.byref(d), p(src), p(self.prepared[i]),
                                                 p(bs), p(dst), stream))
        elif L["op"] == "conv":
            check(getattr(l, f"small_b200_conv2d_{sfx}")(C.byref(d), p(src), p(wt), p(bs), p(dst), stream))
        elif L["op"] == "dwconv":
            check(getattr(l, f"small_b200_dwconv2d_{sfx}")(C.byref(d), p(src), p(wt), p(bs), p(dst), stream))
        elif L["op"] == "maxpool":
            check(getattr(l, f"small_b200_maxpool2d_{sfx}")(C.byref(d), p(src), p(dst), stream))
        elif L["op"] == "avgpool":
            check(getattr(l, f"small_b200_avgpool2d_{sfx}")(C.byref(d), p(src), p(dst), stream))
        elif L["op"] == "softmax":
            check(l.small_b200_softmax_f32(self.batch, cin * L["H"] * L["W"], p(src), p(dst), stream))
        elif L["op"] == "alias":
            pass  # the next layers read `src` under the name `dst`
        else:
            raise ValueError(L["op"])

    def io_plan(self):
        """(source, destination) tensors of every layer in the order enqueue() runs them;
        None for a layer that its producer absorbs."""
        plan, src = [], self.x
        names = dict(self.named)
        for i, L in enumerate(self.layers):
            if i in self.fused_into:
                plan.append(None)  # its producer wrote the pooled tensor
                continue
            if "src" in L:
                if L["op"] == "alias":
                    names[L["dst"]] = names[L["src"]]
                plan.append((names[L["src"]], names[L["dst"]]))
                src = names[L["dst"]]
                continue
            dst = self.bufs[1] if src is self.bufs[0] else self.bufs[0]
            plan.append((src, dst))
            src = dst
        return plan

    def enqueue(self, stream=None):
        stream = self.stream.cuda_stream if stream is None else stream
        src = self.x
        n0 = _lib.launch_count()
        for i, io in enumerate(self.io_plan()):
            if io is None:
                continue
            src, dst = io
            self.enqueue_layer(i, src, dst, stream)
            src = dst
        self.kernels_per_step = _lib.launch_count() - n0
        k, ho, wo = output_shape(self.layers)
        self.y = src[: self.batch * padded(k) * ho * wo]
        return self.y

    def capture(self, inputs=None):
        """Records the layer sequence into a CUDA graph.  `inputs`: a list of device tensors shaped
        like `x`; one graph is recorded per tensor, reading its input from there (launch(k) replays
        graph k), so that a benchmark can rotate over more input data than the L2 cache holds."""
        l = lib()
        self.graphs = []
        for xin in (inputs if inputs is not None else [self.x]):
            saved, self.x = self.x, xin
            self.named["in"] = xin
            self.stream.synchronize()
            gp = C.c_void_p()
            check(l.small_b200_graph_begin(self.stream.cuda_stream))
            try:
                self.enqueue()
            finally:
                check(l.small_b200_graph_end(self.stream.cuda_stream, C.byref(gp)))
                self.x = saved
                self.named["in"] = saved
            self.graphs.append(gp)
        self.graph = self.graphs[0]
        return self

    def launch(self, k=0):
        if self.graph is None:
            self.capture()
        check(lib().small_b200_graph_launch(self.graphs[k % len(self.graphs)], self.stream.cuda_stream))

    def __del__(self):
        try:
            for g in getattr(self, "graphs", []):
                lib().small_b200_graph_destroy(g)
        except Exception:
            pass
