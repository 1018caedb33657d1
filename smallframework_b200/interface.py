"""Python mirror of the reference's functional layer interface for device-resident buffers.

Function names, argument order and error behaviour follow
include/small/interface.hpp:49-497 as defined in include/small/interface_abstract.hpp;
the only addition is the keyword `batch` (the reference's 2-D functions have no batch
dimension; here a batch is image-major, every image laid out exactly as the reference
would lay it out) and `stream`.  Every function only enqueues work on the stream.

Buffers are `FloatBuffer` / `QUInt8Buffer` objects owning a flat torch CUDA tensor; torch
is used for device memory and streams only.  There is no CPU path: a missing library or a
non-CUDA buffer raises.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from ._lib import ACT_LEAKY, ACT_NONE, ACT_RELU, Layer, check, lib
from .packing import CB


# --------------------------------------------------------------------------- buffers
class FloatBuffer:
    """include/small/platforms/b200/Buffer.hpp FloatBuffer: a flat array of float."""
    W_ob, C_ob, C_ib, SIMD, UNROLL = 6, CB, CB, 4, 1
    dtype = torch.float32

    def __init__(self, num_elts=0, device="cuda", data=None):
        if data is not None:
            self.t = _to_device(data, self.dtype, device)
        else:
            self.t = torch.empty(int(num_elts), dtype=self.dtype, device=device)

    def size(self):
        return self.t.numel()

    def data(self):
        return self.t

    def ptr(self):
        return self.t.data_ptr()

    def numpy(self):
        return self.t.cpu().numpy()

    def swap(self, other):
        self.__dict__, other.__dict__ = other.__dict__, self.__dict__

    @classmethod
    def zero(cls):
        return 0


class QUInt8Buffer(FloatBuffer):
    """QUInt8Buffer with the reference's public quantisation fields, initialised the way
    quantized_init() does for the range [-1, 1]
    (include/small/platforms/reference/QUInt8Buffer.hpp:222-272)."""
    W_ob = 2
    dtype = torch.uint8

    def __init__(self, num_elts=0, device="cuda", data=None):
        super().__init__(num_elts, device, data)
        b = 8
        max_q = (1 << b) - 1
        dscale = 2.0 / max_q + 1e-17
        q, shift = math.frexp(dscale)
        q_fixed = int(round(q * (1 << 31)))
        if q_fixed == (1 << 31):
            q_fixed //= 2
            shift += 1
        if shift < -31:
            shift, q_fixed = 0, 0
        if shift > 30:
            shift, q_fixed = 30, (1 << 31) - 1
        self.b = b
        self.multiplier = q_fixed
        self.m_zero = int(np.rint((1.0 * 0 - (-1.0) * max_q) / 2.0))
        self.scale = float(np.float32(dscale))
        self.lshift = shift if shift > 0 else 0
        self.rshift = 0 if shift > 0 else -shift
        self.min_val, self.max_val, self.offset = 0, 255, 0

    def zero(self):  # instance method here: the zero point is a field
        return self.m_zero


def _to_device(data, dtype, device):
    if isinstance(data, torch.Tensor):
        return data.to(device=device, dtype=dtype).contiguous().reshape(-1)
    np_dtype = np.float32 if dtype == torch.float32 else np.uint8
    return torch.from_numpy(np.ascontiguousarray(data, dtype=np_dtype).reshape(-1)).to(device)


def _stream(stream):
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


def _ptr(buf):
    if buf is None:
        return None
    t = buf.t if isinstance(buf, FloatBuffer) else buf
    if not t.is_cuda:
        raise _lib.SmallB200Error("buffers must live on a CUDA device (no CPU path)")
    return t.data_ptr()


def _is_q(buf):
    return isinstance(buf, QUInt8Buffer)


def _layer(batch, C_, K, H, W, Fh, Fw, stride, t, b, l, r, accumulate=0, act=ACT_NONE, slope=0.0,
           inp=None, filt=None, out=None):
    L = Layer(batch, C_, K, H, W, Fh, Fw, stride, t, b, l, r, accumulate, act, slope,
              0, 0, 0, 0, 0, 0)
    if _is_q(out):
        L.zero_in = inp.zero() if _is_q(inp) else 0
        L.zero_filt = filt.zero() if _is_q(filt) else 0
        L.lshift, L.rshift, L.multiplier = out.lshift, out.rshift, out.multiplier
        L.k_zero = 0
    return L


def _need(buf, elems, what):
    if buf.size() < elems:
        raise ValueError(f"{what}: buffer holds {buf.size()} elements, {elems} needed")


# --------------------------------------------------------------------------- dense conv
def _conv(name, partial, kh, kw, stride, t, b, l, r, K, C_, H, W, inp, filt, out, bias, act,
          slope, batch, stream, path=None):
    L = _layer(batch, C_, K, H, W, kh, kw, stride, t, b, l, r, int(partial), act, slope, inp, filt, out)
    ho, wo = L.out_hw()
    if C_ % CB == 0 or C_ in (1, 2, 3):
        _need(inp, batch * C_ * H * W, name + " input")
        _need(filt, K * C_ * kh * kw, name + " filter")
    if K % CB == 0:
        # the quint8 partial form finds its int32 partial sums in the output buffer
        _need(out, (4 if partial and _is_q(out) else 1) * batch * K * ho * wo, name + " output")
    if _is_q(out):
        fn = {None: lib().small_b200_conv2d_u8, "cuda_cores": lib().small_b200_conv2d_u8_cuda_cores,
              "tensor_core": lib().small_b200_conv2d_u8_tensor_core}[path]
    else:
        fn = lib().small_b200_conv2d_f32
    check(fn(C.byref(L), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(out), _stream(stream)))


def Conv2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
           output_channels, input_channels, input_height, input_width,
           input_buf, filter_buf, output_buf, *, batch=1, stream=None, path=None):
    """small::Conv2D (interface_abstract.hpp:46-221 float, :229-404 quint8).  For quint8 buffers path =
    "cuda_cores" / "tensor_core" forces one of the two implementations of the same arithmetic."""
    _conv("Conv2D", False, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
          output_channels, input_channels, input_height, input_width, input_buf, filter_buf,
          output_buf, None, ACT_NONE, 0.0, batch, stream, path)


def PartialConv2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                  output_channels, input_channels, input_height, input_width,
                  input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """small::PartialConv2D (:416-587 float, :595-767 quint8): accumulates onto the existing output.  The
    quint8 form finds int32 partial sums [Ho*Wo][16] at the start of output_buf (four bytes per element)
    and is defined for 16 output channels and one image only (further blocks' sums would overlap)."""
    _conv("PartialConv2D", True, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
          output_channels, input_channels, input_height, input_width, input_buf, filter_buf,
          output_buf, None, ACT_NONE, 0.0, batch, stream)


def Conv2D_ReLU(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                output_channels, input_channels, input_height, input_width,
                input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """small::Conv2D_ReLU (fused_interface_abstract.hpp:55)."""
    _conv("Conv2D_ReLU", False, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
          output_channels, input_channels, input_height, input_width, input_buf, filter_buf,
          output_buf, None, ACT_RELU, 0.0, batch, stream)


def Conv2D_Bias_ReLU(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                     output_channels, input_channels, input_height, input_width,
                     input_buf, filter_buf, bias_buf, output_buf, *, batch=1, stream=None):
    """small::Conv2D_Bias_ReLU (fused_interface_abstract.hpp:217)."""
    _conv("Conv2D_Bias_ReLU", False, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad,
          r_pad, output_channels, input_channels, input_height, input_width, input_buf,
          filter_buf, output_buf, bias_buf, ACT_RELU, 0.0, batch, stream)


def Conv2D_Bias_Activation(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                           output_channels, input_channels, input_height, input_width,
                           input_buf, filter_buf, bias_buf, output_buf, *, activation=ACT_NONE,
                           negative_slope=0.0, batch=1, stream=None, path=None):
    """The single-element-before / -after slots of the reference's fused loop nest
    (abstract_layer.hpp:131-177) with bias before and none / ReLU / LeakyReLU after; equals
    the unfused chain Bias -> PartialConv2D -> activation of Conv2DLayer.hpp:827-878.
    For quint8 buffers bias_buf is an int32 torch tensor added to the accumulator seed."""
    _conv("Conv2D_Bias_Activation", False, kernel_height, kernel_width, stride, t_pad, b_pad,
          l_pad, r_pad, output_channels, input_channels, input_height, input_width, input_buf,
          filter_buf, output_buf, bias_buf, activation, negative_slope, batch, stream, path)


def conv2d_maxpool_supported(conv_kernel_height, conv_kernel_width, conv_stride, conv_pads,
                             pool_kernel_height, pool_kernel_width, pool_stride, pool_pads,
                             output_channels, input_channels, input_height, input_width):
    """Whether Conv2D_Bias_Activation_Maxpool2D runs as one kernel for this pair of shapes."""
    Lc = _layer(1, input_channels, output_channels, input_height, input_width, conv_kernel_height,
                conv_kernel_width, conv_stride, *conv_pads)
    ho, wo = Lc.out_hw()
    Lp = _layer(1, output_channels, output_channels, ho, wo, pool_kernel_height, pool_kernel_width,
                pool_stride, *pool_pads)
    return bool(lib().small_b200_conv2d_maxpool_f32_supported(C.byref(Lc), C.byref(Lp)))


def Conv2D_Bias_Activation_Maxpool2D(conv_kernel_height, conv_kernel_width, conv_stride, conv_pads,
                                     pool_kernel_height, pool_kernel_width, pool_stride, pool_pads,
                                     output_channels, input_channels, input_height, input_width,
                                     input_buf, filter_buf, bias_buf, output_buf, *,
                                     activation=ACT_NONE, negative_slope=0.0, batch=1, stream=None):
    """small::Conv2D_Maxpool2D / Conv2D_ReLU_Maxpool2D / Conv2D_Bias_ReLU_Maxpool2D
    (fused_interface_abstract.hpp:463-1418 of the reference) as ONE kernel, float buffers, for
    the shapes conv2d_maxpool_supported() accepts; bias_buf may be None."""
    Lc = _layer(batch, input_channels, output_channels, input_height, input_width, conv_kernel_height,
                conv_kernel_width, conv_stride, *conv_pads, 0, activation, negative_slope)
    ho, wo = Lc.out_hw()
    Lp = _layer(batch, output_channels, output_channels, ho, wo, pool_kernel_height, pool_kernel_width,
                pool_stride, *pool_pads)
    po, pw = Lp.out_hw()
    _need(output_buf, batch * output_channels * po * pw, "Conv2D_Maxpool2D output")
    check(lib().small_b200_conv2d_maxpool_f32(C.byref(Lc), C.byref(Lp), _ptr(input_buf), _ptr(filter_buf),
                                              _ptr(bias_buf), _ptr(output_buf), _stream(stream)))


# --------------------------------------------------------------------------- per-channel windows
def _window(fn_f32, fn_u8, name, has_filter, kh, kw, stride, t, b, l, r, C_, H, W, inp, filt, out,
            bias, partial, act, slope, batch, stream):
    L = _layer(batch, C_, C_, H, W, kh, kw, stride, t, b, l, r, int(partial), act, slope, inp, filt, out)
    ho, wo = L.out_hw()
    if C_ % CB == 0:
        _need(inp, batch * C_ * H * W, name + " input")
        _need(out, (4 if partial and _is_q(out) else 1) * batch * C_ * ho * wo, name + " output")
    fn = getattr(lib(), fn_u8 if _is_q(out) else fn_f32)
    if has_filter:
        check(fn(C.byref(L), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(out), _stream(stream)))
    else:
        check(fn(C.byref(L), _ptr(inp), _ptr(out), _stream(stream)))


def DepthwiseConv2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                    input_channels, input_height, input_width,
                    input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """small::DepthwiseConv2D (:994 float, :1059 quint8)."""
    _window("small_b200_dwconv2d_f32", "small_b200_dwconv2d_u8", "DepthwiseConv2D", True,
            kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad, input_channels,
            input_height, input_width, input_buf, filter_buf, output_buf, None, False, ACT_NONE,
            0.0, batch, stream)


def PartialDepthwiseConv2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                           input_channels, input_height, input_width,
                           input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """small::PartialDepthwiseConv2D (:1127 float, :1194 quint8).  The quint8 form finds int32 partial
    sums [Ho*Wo][16] at the start of output_buf (four bytes per element) and is defined for 16 channels and
    one image only: the partial sums of further channel blocks would overlap there."""
    _window("small_b200_dwconv2d_f32", "small_b200_dwconv2d_u8", "PartialDepthwiseConv2D", True,
            kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad, input_channels,
            input_height, input_width, input_buf, filter_buf, output_buf, None, True, ACT_NONE,
            0.0, batch, stream)


def DepthwiseConv2D_Bias_Activation(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad,
                                    r_pad, input_channels, input_height, input_width,
                                    input_buf, filter_buf, bias_buf, output_buf, *,
                                    activation=ACT_NONE, negative_slope=0.0, batch=1, stream=None):
    """small::DepthwiseConv2D_ReLU / _Bias_ReLU (fused_interface_abstract.hpp:1332, :1419)."""
    _window("small_b200_dwconv2d_f32", "small_b200_dwconv2d_u8", "DepthwiseConv2D", True,
            kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad, input_channels,
            input_height, input_width, input_buf, filter_buf, output_buf, bias_buf, False,
            activation, negative_slope, batch, stream)


def _group(name, partial, kh, kw, stride, groups, t, b, l, r, C_, H, W, inp, filt, out, bias, act,
           slope, batch, stream):
    if C_ % CB != 0:
        raise ValueError(f"{name} ERROR: in_channels unsupported.")
    L = _layer(batch, C_, C_, H, W, kh, kw, stride, t, b, l, r, int(partial), act, slope, inp, filt, out)
    ho, wo = L.out_hw()
    if groups > 0 and groups % CB == 0:
        _need(inp, batch * groups * C_ * H * W, name + " input")
        _need(filt, groups * C_ * C_ * kh * kw, name + " filter")
        _need(out, batch * groups * C_ * ho * wo, name + " output")
    fn = lib().small_b200_groupconv2d_u8 if _is_q(out) else lib().small_b200_groupconv2d_f32
    check(fn(C.byref(L), C.c_int32(groups), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(out), _stream(stream)))


def GroupConv2D(kernel_height, kernel_width, stride, output_groups, t_pad, b_pad, l_pad, r_pad,
                input_channels, input_height, input_width, input_buf, filter_buf, output_buf, *,
                bias_buf=None, activation=ACT_NONE, negative_slope=0.0, batch=1, stream=None):
    """small::GroupConv2D (:1265 float, :1332 quint8): `output_groups` convolutions, each from
    `input_channels` to `input_channels` channels; the 16 lanes of a block are 16 groups
    (in [G/16][C][H][W][16], filter [G/16][K][C][Fh][Fw][16], out [G/16][K][Ho][Wo][16])."""
    _group("GroupConv2D", False, kernel_height, kernel_width, stride, output_groups, t_pad, b_pad,
           l_pad, r_pad, input_channels, input_height, input_width, input_buf, filter_buf,
           output_buf, bias_buf, activation, negative_slope, batch, stream)


def PartialGroupConv2D(kernel_height, kernel_width, stride, output_groups, t_pad, b_pad, l_pad, r_pad,
                       input_channels, input_height, input_width, input_buf, filter_buf, output_buf,
                       *, batch=1, stream=None):
    """small::PartialGroupConv2D (:1402 float).  The quint8 form (:1470) keeps the int32 partial sums of
    output channel k at byte k * Ho*Wo*16 of the uint8 output, four times the channel's length: for the
    16-or-more channels per group the interface accepts they always overlap, so the library refuses it."""
    _group("PartialGroupConv2D", True, kernel_height, kernel_width, stride, output_groups, t_pad,
           b_pad, l_pad, r_pad, input_channels, input_height, input_width, input_buf, filter_buf,
           output_buf, None, ACT_NONE, 0.0, batch, stream)


def MaxPool2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
              input_channels, input_height, input_width, input_buf, output_buf, *,
              batch=1, stream=None):
    """small::MaxPool2D (:778 float, :843 quint8)."""
    _window("small_b200_maxpool2d_f32", "small_b200_maxpool2d_u8", "MaxPool2D", False,
            kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad, input_channels,
            input_height, input_width, input_buf, None, output_buf, None, False, ACT_NONE, 0.0,
            batch, stream)


def AveragePool2D(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                  input_channels, input_height, input_width, input_buf, output_buf, *,
                  batch=1, stream=None):
    """small::AveragePool2D (:910, float); the quint8 form has no counterpart in the reference."""
    _window("small_b200_avgpool2d_f32", "small_b200_avgpool2d_u8", "AveragePool2D", False,
            kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad, input_channels,
            input_height, input_width, input_buf, None, output_buf, None, False, ACT_NONE, 0.0,
            batch, stream)


# --------------------------------------------------------------------------- elementwise
def _chan_check(name, channels):
    if channels % CB != 0:
        raise ValueError(f"{name} ERROR: in_channels unsupported.")


def ReLUActivation(input_channels, input_height, input_width, input_buf, output_buf, *,
                   batch=1, stream=None):
    """small::ReLUActivation (:1541 float; :1577 quint8 = requantised max(a + zero, 0))."""
    n = batch * input_channels * input_height * input_width
    if _is_q(output_buf):
        _chan_check("ReLUActivation<quint8>", input_channels)
        L = _layer(batch, input_channels, input_channels, input_height, input_width, 1, 1, 1,
                   0, 0, 0, 0, inp=input_buf, out=output_buf)
        check(lib().small_b200_relu_u8(n, C.byref(L), _ptr(input_buf), _ptr(output_buf), _stream(stream)))
    else:
        _chan_check("ReLUActivation<float>", input_channels)
        check(lib().small_b200_relu_f32(n, _ptr(input_buf), _ptr(output_buf), _stream(stream)))


def LeakyReLUActivation(input_channels, input_height, input_width, input_buf, filter_buf,
                        output_buf, *, batch=1, stream=None):
    """small::LeakyReLUActivation (:1616): the slope arrives as a one-element buffer (or a float)."""
    _chan_check("LeakyReLUActivation<float>", input_channels)
    slope = float(filter_buf.t[0].item()) if isinstance(filter_buf, FloatBuffer) else float(filter_buf)
    n = batch * input_channels * input_height * input_width
    check(lib().small_b200_leaky_relu_f32(n, _ptr(input_buf), slope, _ptr(output_buf), _stream(stream)))


def Dropout(input_channels, input_height, input_width, input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """small::Dropout (:1697): output = input * rate, the rate arriving as a one-element buffer (or a float)."""
    _chan_check("Dropout<float>", input_channels)
    rate = float(filter_buf.t[0].item()) if isinstance(filter_buf, FloatBuffer) else float(filter_buf)
    n = batch * input_channels * input_height * input_width
    check(lib().small_b200_scale_f32(n, _ptr(input_buf), rate, _ptr(output_buf), _stream(stream)))


def Accum(input_channels, input_height, input_width, input_buf, output_buf, *, batch=1, stream=None):
    """small::Accum (:1950): output += input."""
    _chan_check("Accum<float>", input_channels)
    n = batch * input_channels * input_height * input_width
    check(lib().small_b200_accum_f32(n, _ptr(input_buf), _ptr(output_buf), _stream(stream)))


def Bias(num_channels, output_height, output_width, input_buf, output_buf, *, batch=1, stream=None):
    """small::Bias (:1992): output[c, h, w] = bias[c]."""
    check(lib().small_b200_bias_f32(batch, num_channels, output_height, output_width,
                                    _ptr(input_buf), 0, _ptr(output_buf), _stream(stream)))


def PartialBias(num_channels, output_height, output_width, input_buf, output_buf, *, batch=1,
                stream=None):
    """small::PartialBias (:2035): output[c, h, w] += bias[c]."""
    check(lib().small_b200_bias_f32(batch, num_channels, output_height, output_width,
                                    _ptr(input_buf), 1, _ptr(output_buf), _stream(stream)))


def UpSample2D(scale_factor, input_channels, input_height, input_width, input_buf, output_buf, *,
               batch=1, stream=None):
    """small::UpSample2D (:1845): scale 1 copies, scale 2 is nearest-neighbour, others throw."""
    if scale_factor == 1:
        n = batch * input_channels * input_height * input_width
        check(lib().small_b200_memcpy_d2d(_ptr(output_buf), _ptr(input_buf), n * 4, _stream(stream)))
    elif scale_factor == 2:
        check(lib().small_b200_upsample2d_f32(batch, input_channels, input_height, input_width,
                                              _ptr(input_buf), _ptr(output_buf), _stream(stream)))
    else:
        raise ValueError("Upsample<float> ERROR: scale factor unsupported (only 1 or 2).")


def SoftMax(input_channels, input_height, input_width, input_buf, output_buf, *, batch=1, stream=None):
    """small::SoftMax (:1778): normalised over ALL input_channels*height*width elements of an
    image.  Channels padded up to the block size by a layer class would add exp(0) terms, so
    callers pass the effective element count by keeping padded logits out of the tensor."""
    _chan_check("SoftMax<float>", input_channels)
    check(lib().small_b200_softmax_f32(batch, input_channels * input_height * input_width,
                                       _ptr(input_buf), _ptr(output_buf), _stream(stream)))


def Concat(input0_channels, input1_channels, input_height, input_width, input0_buf, input1_buf,
           output_buf, *, batch=1, stream=None):
    """small::Concat (:2072): channel concatenation of two packed buffers."""
    esz = input0_buf.t.element_size()
    b0 = input0_channels * input_height * input_width * esz
    b1 = input1_channels * input_height * input_width * esz
    check(lib().small_b200_concat(batch, b0, _ptr(input0_buf), b1, _ptr(input1_buf),
                                  _ptr(output_buf), _stream(stream)))


def Dense(output_elements, input_elements, input_buf, filter_buf, output_buf, *, batch=1, stream=None):
    """A fully connected layer the way the reference's models build it: Conv2D 1x1 on a 1x1
    image with FILTER_FC packing (include/small/models/DSCNNTiny.hpp:255-263).  The
    reference's own small::Dense (:2113) is an uncalled placeholder that instantiates a
    depthwise scaling, not a matrix-vector product."""
    Conv2D(1, 1, 1, 0, 0, 0, 0, output_elements, input_elements, 1, 1, input_buf, filter_buf,
           output_buf, batch=batch, stream=stream)


# --------------------------------------------------------------------------- tensor-core fp32 conv
def tf32x3_supported(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                     output_channels, input_channels, input_height, input_width):
    L = _layer(1, input_channels, output_channels, input_height, input_width, kernel_height,
               kernel_width, stride, t_pad, b_pad, l_pad, r_pad)
    return bool(lib().small_b200_conv2d_f32_tf32x3_supported(C.byref(L)))


def prepare_filter_3xTF32(kernel_height, kernel_width, output_channels, input_channels,
                          filter_buf, prepared_buf, *, stream=None):
    """Re-lay a packed filter for the tensor-core path (hi copy + lo copy, 2x the elements)."""
    L = _layer(1, input_channels, output_channels, 16, 16, kernel_height, kernel_width, 1, 0, 0, 0, 0)
    check(lib().small_b200_filter_prepare_tf32x3(C.byref(L), _ptr(filter_buf), _ptr(prepared_buf),
                                                 _stream(stream)))


def Conv2D_3xTF32(kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
                  output_channels, input_channels, input_height, input_width,
                  input_buf, prepared_filter_buf, bias_buf, output_buf, *,
                  partial=False, activation=ACT_NONE, negative_slope=0.0, batch=1, stream=None):
    """small::Conv2D / PartialConv2D<FloatBuffer> (+ bias / activation) on the tensor cores;
    prepared_filter_buf = prepare_filter_3xTF32(filter)."""
    L = _layer(batch, input_channels, output_channels, input_height, input_width, kernel_height,
               kernel_width, stride, t_pad, b_pad, l_pad, r_pad, int(partial), activation, negative_slope)
    check(lib().small_b200_conv2d_f32_tf32x3(C.byref(L), _ptr(input_buf),
                                             _ptr(prepared_filter_buf), _ptr(bias_buf),
                                             _ptr(output_buf), _stream(stream)))


def conv2d_maxpool_3xTF32_supported(conv_kernel_height, conv_kernel_width, conv_pads, output_channels,
                                    input_channels, input_height, input_width):
    """Whether Conv2D_Maxpool2D_3xTF32 covers this convolution followed by a 2x2 stride-2 max pool."""
    Lc = _layer(1, input_channels, output_channels, input_height, input_width, conv_kernel_height,
                conv_kernel_width, 1, *conv_pads)
    ho, wo = Lc.out_hw()
    Lp = _layer(1, output_channels, output_channels, ho, wo, 2, 2, 2, 0, 0, 0, 0)
    return bool(lib().small_b200_conv2d_maxpool_f32_tf32x3_supported(C.byref(Lc), C.byref(Lp)))


def Conv2D_Maxpool2D_3xTF32(conv_kernel_height, conv_kernel_width, conv_pads, output_channels, input_channels,
                            input_height, input_width, input_buf, prepared_filter_buf, bias_buf, output_buf, *,
                            activation=ACT_NONE, negative_slope=0.0, batch=1, stream=None):
    """small::Conv2D_Maxpool2D / Conv2D_ReLU_Maxpool2D / Conv2D_Bias_ReLU_Maxpool2D<FloatBuffer>
    (fused_interface_abstract.hpp:463-1418 of the reference) on the tensor cores: stride-1 convolution
    (+ bias, + activation) with the 2x2 stride-2 max pool in its epilogue;
    prepared_filter_buf = prepare_filter_3xTF32(filter)."""
    Lc = _layer(batch, input_channels, output_channels, input_height, input_width, conv_kernel_height,
                conv_kernel_width, 1, *conv_pads, 0, activation, negative_slope)
    ho, wo = Lc.out_hw()
    Lp = _layer(batch, output_channels, output_channels, ho, wo, 2, 2, 2, 0, 0, 0, 0)
    _need(output_buf, batch * output_channels * (ho // 2) * (wo // 2), "Conv2D_Maxpool2D output")
    check(lib().small_b200_conv2d_maxpool_f32_tf32x3(C.byref(Lc), C.byref(Lp), _ptr(input_buf),
                                                     _ptr(prepared_filter_buf), _ptr(bias_buf),
                                                     _ptr(output_buf), _stream(stream)))


# --------------------------------------------------------------------------- fused uint8 blocks
def _qlayer(batch, C_, K, H, W, Fh, Fw, stride, pads, inp_zero, filt_zero, out_q):
    """A uint8 layer descriptor from explicit quantisation parameters: out_q = (lshift, rshift, multiplier)."""
    L = Layer(batch, C_, K, H, W, Fh, Fw, stride, *pads, 0, ACT_NONE, 0.0, 0, 0, 0, 0, 0, 0)
    L.zero_in, L.zero_filt = inp_zero, filt_zero
    L.lshift, L.rshift, L.multiplier = out_q
    return L


def Conv2D_ReLU_DepthwiseConv2D_ReLU(conv_kernel_height, conv_kernel_width, conv_stride,
                                     conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad,
                                     dw_kernel_height, dw_kernel_width, dw_stride,
                                     dw_t_pad, dw_b_pad, dw_l_pad, dw_r_pad,
                                     output_channels, input_channels, input_height, input_width,
                                     input_buf, filter_buf, inter_output_buf, dwise_filter_buf, output_buf, *,
                                     conv_bias=None, dw_bias=None, batch=1, stream=None):
    """small::Conv2D_ReLU_DepthwiseConv2D_ReLU (fused_interface_abstract.hpp:1840; the argument list is
    the reference's) for QUInt8Buffer operands, where the clamp of each requantisation is the ReLU.
    inter_output_buf carries the quantisation of the intermediate (its zero point and the
    multiplier / shifts the convolution requantises with); no data is written to it when the pair
    runs as one kernel.  Pairs the one-kernel form does not cover run as two calls through it."""
    if not (_is_q(input_buf) and _is_q(output_buf) and _is_q(inter_output_buf)):
        raise ValueError("Conv2D_ReLU_DepthwiseConv2D_ReLU: this form takes QUInt8Buffer operands")
    Lc = _qlayer(batch, input_channels, output_channels, input_height, input_width, conv_kernel_height,
                 conv_kernel_width, conv_stride, (conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad),
                 input_buf.zero(), filter_buf.zero(),
                 (inter_output_buf.lshift, inter_output_buf.rshift, inter_output_buf.multiplier))
    ho, wo = Lc.out_hw()
    Ld = _qlayer(batch, output_channels, output_channels, ho, wo, dw_kernel_height, dw_kernel_width, dw_stride,
                 (dw_t_pad, dw_b_pad, dw_l_pad, dw_r_pad), inter_output_buf.zero(), dwise_filter_buf.zero(),
                 (output_buf.lshift, output_buf.rshift, output_buf.multiplier))
    po, pw = Ld.out_hw()
    _need(output_buf, batch * output_channels * po * pw, "Conv2D_ReLU_DepthwiseConv2D_ReLU output")
    if lib().small_b200_conv2d_dwconv2d_u8_supported(C.byref(Lc), C.byref(Ld)):
        check(lib().small_b200_conv2d_dwconv2d_u8(C.byref(Lc), C.byref(Ld), _ptr(input_buf), _ptr(filter_buf),
                                                  _ptr(conv_bias), _ptr(dwise_filter_buf), _ptr(dw_bias),
                                                  _ptr(output_buf), _stream(stream)))
        return True
    _need(inter_output_buf, batch * output_channels * ho * wo, "Conv2D_ReLU_DepthwiseConv2D_ReLU intermediate")
    check(lib().small_b200_conv2d_u8(C.byref(Lc), _ptr(input_buf), _ptr(filter_buf), _ptr(conv_bias),
                                     _ptr(inter_output_buf), _stream(stream)))
    check(lib().small_b200_dwconv2d_u8(C.byref(Ld), _ptr(inter_output_buf), _ptr(dwise_filter_buf), _ptr(dw_bias),
                                       _ptr(output_buf), _stream(stream)))
    return False


# --------------------------------------------------------------------------- detection head
def YOLODecode(anchors, num_classes, input_img_size, padded_channels, input_height, input_width, input_buf,
               output_buf, *, batch=1, stream=None):
    """small::YOLOLayer::compute_output (include/small/YOLOLayer.hpp:96-222) on the device: the packed
    activation becomes [batch][len(anchors) * H * W][5 + num_classes] records.  anchors: (w, h) pairs of
    this layer's mask; the stride is input_img_size / input_height as in the layer's constructor."""
    a = np.ascontiguousarray(np.asarray(anchors, np.float32).ravel())
    _need(input_buf, batch * padded_channels * input_height * input_width, "YOLOLayer input")
    _need(output_buf, batch * len(anchors) * input_height * input_width * (num_classes + 5), "YOLOLayer output")
    check(lib().small_b200_yolo_decode_f32(batch, padded_channels, input_height, input_width, len(anchors),
                                           num_classes, float(input_img_size // input_height),
                                           a.ctypes.data, _ptr(input_buf), _ptr(output_buf), _stream(stream)))


def NonMaxSuppression(pred_buf, num_pred, num_classes, confidence_threshold=0.25, iou_threshold=0.45, *,
                      max_candidates=16384, max_detections=1024, stream=None):
    """Darknet::process_outputs + small::basic_nms (include/small/models/Darknet.hpp:78-122,
    include/small/non_max_suppression.hpp:98-155) on the device.  Returns a numpy array [n, 7] of
    x, y, w, h, objectness, class score, class id in keep order (this call waits for the device)."""
    l = lib()
    scratch = torch.empty(l.small_b200_nms_scratch_bytes(max_candidates), dtype=torch.uint8, device=pred_buf.t.device)
    dets = torch.zeros(max_detections * 7, dtype=torch.float32, device=pred_buf.t.device)
    counts = torch.zeros(2, dtype=torch.int32, device=pred_buf.t.device)
    check(l.small_b200_nms_f32(_ptr(pred_buf), num_pred, num_classes, confidence_threshold, iou_threshold,
                               max_candidates, scratch.data_ptr(), max_detections, dets.data_ptr(),
                               counts.data_ptr(), _stream(stream)))
    kept, cand = (int(v) for v in counts.cpu())
    if cand > max_candidates:
        raise _lib.SmallB200Error(f"NMS: {cand} candidates above the confidence threshold, room for {max_candidates}")
    return dets.cpu().numpy().reshape(max_detections, 7)[:min(kept, max_detections)]
