"""Darknet `.cfg` / `.weights` loader for the device path.

The reference builds a DAG of Layer objects from a Darknet configuration and a weight file
(include/small/models/Darknet.hpp:786-1040: [net], [convolutional], [maxpool], [route], [upsample],
[shortcut], [yolo]) and prepares every convolution's weights on the host (Conv2DLayer.hpp:135-341).
Here the host only parses: `build_plan` turns the configuration into a list of layer records with
shapes, parents and offsets into the weight file; `DarknetModel` uploads the weight file once, lets
the device pad / pack / fold batch normalisation per layer (small_b200_conv_weights_prepare_f32),
and runs the layers through the C ABI: convolutions with bias and LeakyReLU(0.1) in the kernel
(the slope the reference passes, Darknet.hpp:326-329), pools, routes as concatenations, nearest
upsampling, shortcuts, and box decoding; `detect` adds collection + non-maximum suppression.

Weight file layout (Darknet.hpp:817-834, :283-311, :339-349): a 20-byte header, then per
convolution either [beta, gamma, running mean, running variance] or [bias], each `filters` floats,
followed by the filter [filters][channels][size][size].
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .packing import CB, calc_padding, output_dim

HEADER_BYTES = 20
LEAKY_SLOPE = 0.1
BN_EPS = 1e-5


def parse_cfg(text):
    """[(section name, {key: value})] in file order; comments and blank lines dropped."""
    blocks = []
    for raw in text.splitlines():
        line = raw.strip()
        if not line or line[0] in "#;":
            continue
        if line[0] == "[":
            blocks.append((line.strip("[]").strip(), {}))
        elif blocks and "=" in line:
            k, v = line.split("=", 1)
            blocks[-1][1][k.strip()] = v.strip()
    return blocks


def _padded(c):
    return -(-c // CB) * CB


def build_plan(cfg_text):
    """The network as a list of records (no device needed).  Every record has
    op, parents (indices of earlier records, -1 = the network input), C / K (effective channels in and
    out), Cp / Kp (as stored: padded to the block, 3-channel input excepted), H, W, Ho, Wo, and for
    convolutions size / stride / pads / bn / act / w_off (float offset into the weight file behind the
    header), for yolo layers anchors / classes."""
    blocks = parse_cfg(cfg_text)
    if not blocks or blocks[0][0] != "net":
        raise ValueError("Darknet cfg ERROR: the first section must be [net]")
    net = blocks[0][1]
    shape = (int(net.get("channels", 3)), int(net["height"]), int(net["width"]))
    plan, w_off = [], 0
    out_shape = lambda i: shape if i < 0 else (plan[i]["K"], plan[i]["Ho"], plan[i]["Wo"])
    for name, kv in blocks[1:]:
        i = len(plan)
        prev = i - 1
        c, h, w = out_shape(prev)
        rec = dict(op=name, parents=[prev], C=c, Cp=c if prev < 0 and c < CB else _padded(c), H=h, W=w)
        if name == "convolutional":
            k, size, stride = int(kv["filters"]), int(kv["size"]), int(kv.get("stride", 1))
            if prev >= 0 and plan[prev]["Kp"] != plan[prev]["K"]:
                raise ValueError("Darknet cfg ERROR: a convolution after a layer with padded output channels is "
                                 "not supported (nor is it by the reference's Conv2DLayer)")
            pads = (calc_padding(h, size, stride) + calc_padding(w, size, stride)) if kv.get("pad", "1") == "1" \
                else (0, 0, 0, 0)
            act = {"leaky": 2, "relu": 1, "linear": 0}[kv.get("activation", "linear")]
            bn = kv.get("batch_normalize", "0") == "1"
            rec.update(op="conv", K=k, Kp=_padded(k), size=size, stride=stride, pads=pads, bn=bn, act=act, w_off=w_off,
                       Ho=output_dim(h, pads[0], pads[1], size, stride), Wo=output_dim(w, pads[2], pads[3], size, stride))
            w_off += (4 if bn else 1) * k + k * c * size * size
        elif name == "maxpool":
            size, stride = int(kv["size"]), int(kv.get("stride", 1))
            pads = calc_padding(h, size, stride) + calc_padding(w, size, stride)  # PADDING_F, Darknet.hpp:381
            rec.update(op="maxpool", K=c, Kp=rec["Cp"], size=size, stride=stride, pads=pads,
                       Ho=output_dim(h, pads[0], pads[1], size, stride), Wo=output_dim(w, pads[2], pads[3], size, stride))
        elif name == "upsample":
            s = int(kv.get("stride", 2))
            rec.update(op="upsample", K=c, Kp=rec["Cp"], scale=s, Ho=h * s, Wo=w * s)
        elif name == "route":
            ids = [int(v) for v in kv["layers"].split(",")]
            parents = [i + v if v < 0 else v for v in ids]
            if len(parents) not in (1, 2):
                raise ValueError("Darknet cfg ERROR: route layer must have only 1 or 2 layers")
            shapes = [out_shape(p) for p in parents]
            if any(s[1:] != shapes[0][1:] for s in shapes) or any(plan[p]["Kp"] != plan[p]["K"] for p in parents):
                raise ValueError("Darknet cfg ERROR: route inputs must share their image size and be unpadded")
            k = sum(s[0] for s in shapes)
            rec.update(op="route", parents=parents, C=k, Cp=k, K=k, Kp=k, H=shapes[0][1], W=shapes[0][2],
                       Ho=shapes[0][1], Wo=shapes[0][2])
        elif name == "shortcut":
            if kv.get("activation", "linear") != "linear":
                raise ValueError("Darknet cfg ERROR: unsupported activation in shortcut layer")
            other = i + int(kv["from"])
            if out_shape(other) != (c, h, w):
                raise ValueError("Darknet cfg ERROR: shortcut inputs differ in shape")
            rec.update(op="shortcut", parents=[prev, other], K=c, Kp=rec["Cp"], Ho=h, Wo=w)
        elif name == "yolo":
            mask = [int(v) for v in kv["mask"].split(",")]
            flat = [int(v) for v in kv["anchors"].split(",")]
            pairs = list(zip(flat[0::2], flat[1::2]))
            classes = int(kv["classes"])
            anchors = [pairs[m] for m in mask]
            if len(anchors) * (classes + 5) != c:
                raise ValueError("YOLOLayer ERROR: incorrect input buffer shape.")
            rec.update(op="yolo", K=c, Kp=rec["Cp"], anchors=anchors, classes=classes, Ho=h, Wo=w,
                       img=int(net["height"]), preds=len(anchors) * h * w)
        else:
            raise ValueError(f"Darknet cfg ERROR: unsupported section [{name}]")
        plan.append(rec)
    return shape, plan, w_off


def random_weights(cfg_text, seed=0):
    """A weight file (bytes) for `cfg_text` with seeded random parameters -- what stands in for a real
    `.weights` file where none can be had: He-normal filters, BN statistics near identity."""
    _, plan, total = build_plan(cfg_text)
    rng = np.random.default_rng(seed)
    w = np.zeros(total, np.float32)
    for r in plan:
        if r["op"] != "conv":
            continue
        k, o = r["K"], r["w_off"]
        if r["bn"]:
            w[o:o + k] = rng.normal(0, 0.1, k)                 # beta
            w[o + k:o + 2 * k] = rng.uniform(0.8, 1.2, k)      # gamma
            w[o + 2 * k:o + 3 * k] = rng.normal(0, 0.1, k)     # running mean
            w[o + 3 * k:o + 4 * k] = rng.uniform(0.5, 1.5, k)  # running variance
            o += 4 * k
        else:
            w[o:o + k] = rng.normal(0, 0.1, k)
            o += k
        n = k * r["C"] * r["size"] ** 2
        w[o:o + n] = rng.normal(0, np.sqrt(2.0 / (r["C"] * r["size"] ** 2)), n)
    return np.zeros(HEADER_BYTES, np.uint8).tobytes() + w.tobytes()


class DarknetModel:
    """A Darknet network on one GPU.  x: packed input [batch][H][W][C] (C <= 3) or [batch][C/16][H][W][16]."""

    def __init__(self, cfg_text, weights, batch=1, device="cuda", tensor_core="auto"):
        import torch

        from ._lib import Layer, check, lib
        self.torch, self.check, self.lib, self.Layer = torch, check, lib(), Layer
        self.batch, self.dev = batch, torch.device(device)
        self.shape, self.plan, n_floats = build_plan(cfg_text)
        raw = weights if isinstance(weights, (bytes, bytearray)) else open(weights, "rb").read()
        if len(raw) < HEADER_BYTES + 4 * n_floats:
            raise ValueError("Darknet weights ERROR: the file is shorter than the configuration needs")
        host = np.frombuffer(raw, dtype=np.float32, offset=HEADER_BYTES, count=n_floats)
        self.raw = torch.from_numpy(host.copy()).to(self.dev)   # the whole file, uploaded once
        self.stream = torch.cuda.current_stream(self.dev)
        st = self.stream.cuda_stream
        c, h, w = self.shape
        self.x = torch.zeros(batch * c * h * w, device=self.dev)
        self.out, self.params = [], []
        for r in self.plan:
            n_out = batch * (r["preds"] * (r["classes"] + 5) if r["op"] == "yolo" else r["Kp"] * r["Ho"] * r["Wo"])
            alias = r["op"] == "route" and len(r["parents"]) == 1
            self.out.append(None if alias else torch.zeros(n_out, device=self.dev))
            if r["op"] != "conv":
                self.params.append(None)
                continue
            k, kp, cin, f = r["K"], r["Kp"], r["C"], r["size"]
            base = self.raw.data_ptr() + 4 * r["w_off"]
            ptr = lambda j: base + 4 * j * k
            packed = torch.empty(kp * cin * f * f, device=self.dev)
            bias = torch.empty(kp, device=self.dev)
            if r["bn"]:
                check(self.lib.small_b200_conv_weights_prepare_f32(kp, k, cin, f, f, ptr(4), None, ptr(1), ptr(0), ptr(2),
                                                                   ptr(3), BN_EPS, packed.data_ptr(), bias.data_ptr(), st))
            else:
                check(self.lib.small_b200_conv_weights_prepare_f32(kp, k, cin, f, f, ptr(1), ptr(0), None, None, None,
                                                                   None, 0.0, packed.data_ptr(), bias.data_ptr(), st))
            d = self._desc(r)
            prepared = None
            use_tc = tensor_core and self.lib.small_b200_conv2d_f32_tf32x3_supported(C.byref(d)) and (
                tensor_core is True or self.lib.small_b200_conv2d_f32_tf32x3_preferred(C.byref(d)))
            if use_tc:
                prepared = torch.empty(2 * packed.numel(), device=self.dev)
                check(self.lib.small_b200_filter_prepare_tf32x3(C.byref(d), packed.data_ptr(), prepared.data_ptr(), st))
            self.params.append((packed, bias, prepared))
        self.stream.synchronize()

    def _desc(self, r):
        return self.Layer(self.batch, r["Cp"], r["Kp"], r["H"], r["W"], r["size"], r["size"], r["stride"], *r["pads"],
                          0, r.get("act", 0), LEAKY_SLOPE, 0, 0, 0, 0, 0, 0)

    def _src(self, i):
        if i < 0:
            return self.x
        return self.out[i] if self.out[i] is not None else self._src(self.plan[i]["parents"][0])

    def inference(self, x=None):
        """Enqueues the network; returns the device tensors of the yolo layers, each
        [batch][predictions][5 + classes]."""
        l, check, st = self.lib, self.check, self.stream.cuda_stream
        if x is not None:
            self.x.copy_(self.torch.as_tensor(x, device=self.dev).reshape(-1))
        heads = []
        for i, r in enumerate(self.plan):
            src = [self._src(p) for p in r["parents"]]
            dst = self.out[i]
            if r["op"] == "conv":
                packed, bias, prepared = self.params[i]
                d = self._desc(r)
                if prepared is not None:
                    check(l.small_b200_conv2d_f32_tf32x3(C.byref(d), src[0].data_ptr(), prepared.data_ptr(), bias.data_ptr(),
                                                         dst.data_ptr(), st))
                else:
                    check(l.small_b200_conv2d_f32(C.byref(d), src[0].data_ptr(), packed.data_ptr(), bias.data_ptr(),
                                                  dst.data_ptr(), st))
            elif r["op"] == "maxpool":
                check(l.small_b200_maxpool2d_f32(C.byref(self._desc(r)), src[0].data_ptr(), dst.data_ptr(), st))
            elif r["op"] == "upsample":
                if r["scale"] != 2:
                    raise ValueError("Upsample<float> ERROR: scale factor unsupported (only 1 or 2).")
                check(l.small_b200_upsample2d_f32(self.batch, r["Cp"], r["H"], r["W"], src[0].data_ptr(), dst.data_ptr(), st))
            elif r["op"] == "route":
                if len(src) == 2:
                    b0 = self.plan[r["parents"][0]]["K"] * r["H"] * r["W"] * 4
                    b1 = self.plan[r["parents"][1]]["K"] * r["H"] * r["W"] * 4
                    check(l.small_b200_concat(self.batch, b0, src[0].data_ptr(), b1, src[1].data_ptr(), dst.data_ptr(), st))
            elif r["op"] == "shortcut":
                n = dst.numel()
                check(l.small_b200_memcpy_d2d(dst.data_ptr(), src[0].data_ptr(), 4 * n, st))
                check(l.small_b200_accum_f32(n, src[1].data_ptr(), dst.data_ptr(), st))
            elif r["op"] == "yolo":
                a = np.ascontiguousarray(np.asarray(r["anchors"], np.float32).ravel())
                check(l.small_b200_yolo_decode_f32(self.batch, r["Cp"], r["H"], r["W"], len(r["anchors"]), r["classes"],
                                                   float(r["img"] // r["H"]), a.ctypes.data, src[0].data_ptr(),
                                                   dst.data_ptr(), st))
                heads.append(dst.view(self.batch, r["preds"], r["classes"] + 5))
        return heads

    def detect(self, x=None, confidence_threshold=0.25, iou_threshold=0.45, max_candidates=16384, max_detections=1024):
        """Darknet::process_outputs per image: numpy arrays [n, 7] of x, y, w, h, objectness, class score, class id."""
        from . import interface as S
        heads = self.inference(x)
        classes = self.plan[-1]["classes"] if self.plan[-1]["op"] == "yolo" else [r for r in self.plan if r["op"] == "yolo"][-1]["classes"]
        out = []
        for n in range(self.batch):
            rec = self.torch.cat([hd[n] for hd in heads], dim=0).contiguous()
            buf = S.FloatBuffer(data=rec.reshape(-1))
            out.append(S.NonMaxSuppression(buf, rec.shape[0], classes, confidence_threshold, iou_threshold,
                                           max_candidates=max_candidates, max_detections=max_detections))
        return out
