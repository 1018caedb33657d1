"""Host-side packing between plain NCHW / KCRS tensors and SMaLL's blocked layout.

Mirrors include/small/buffers.hpp of the reference:
  activations  [C/cb][H][W][cb]                       packed_buffer_index :83-120
  conv filter  [K/cob][C/cib][Fh][Fw][cib][cob]       packed_weight_index :33-79
  dw filter    [C/cb][Fh][Fw][cb]                     pack_buffer (FILTER_DW) :266-395
with the first-layer exception cib := C when C is 1, 2 or 3 and smaller than the
platform block (:52-57).  A batch is image-major: [N] x the single-image layout, so
every image is byte-identical to what the reference would hold for it.
"""
from __future__ import annotations

import numpy as np

#: channel block of the B200 platform, for both element types (FLOAT_C_ob == FLOAT_C_ib
#: == QUINT8_C_ob == QUINT8_C_ib in include/small/platforms/b200/params.h)
CB = 16


def effective_block(channels: int, block: int) -> int:
    if channels < block:
        if channels in (1, 2, 3):
            return channels
        raise RuntimeError("num_channels < channel_blocking && num_channels not in {1, 2, 3}")
    if channels % block:
        raise RuntimeError("num_channels % channel_blocking != 0")
    return block


def pack_activation(x: np.ndarray, cb: int = CB) -> np.ndarray:
    """[..., C, H, W] -> flat [..., C/cb, H, W, cb] (leading dims = batch)."""
    *lead, c, h, w = x.shape
    b = effective_block(c, cb)
    y = x.reshape(*lead, c // b, b, h, w)
    y = np.moveaxis(y, -3, -1)  # [..., C/b, H, W, b]
    return np.ascontiguousarray(y).reshape(*lead, -1)


def unpack_activation(flat: np.ndarray, c: int, h: int, w: int, cb: int = CB) -> np.ndarray:
    """flat [..., C*H*W] packed -> [..., C, H, W]."""
    lead = flat.shape[:-1]
    b = effective_block(c, cb)
    y = flat.reshape(*lead, c // b, h, w, b)
    y = np.moveaxis(y, -1, -3)  # [..., C/b, b, H, W]
    return np.ascontiguousarray(y).reshape(*lead, c, h, w)


def pack_conv_filter(wt: np.ndarray, cib: int = CB, cob: int = CB) -> np.ndarray:
    """[K, C, Fh, Fw] -> flat [K/cob][C/cib][Fh][Fw][cib][cob]."""
    k, c, fh, fw = wt.shape
    bi = effective_block(c, cib)
    if k % cob:
        raise RuntimeError("num_filters % filter_blocking != 0")
    y = wt.reshape(k // cob, cob, c // bi, bi, fh, fw)
    y = y.transpose(0, 2, 4, 5, 3, 1)
    return np.ascontiguousarray(y).reshape(-1)


def unpack_conv_filter(flat: np.ndarray, k: int, c: int, fh: int, fw: int,
                       cib: int = CB, cob: int = CB) -> np.ndarray:
    bi = effective_block(c, cib)
    y = flat.reshape(k // cob, c // bi, fh, fw, bi, cob).transpose(0, 5, 1, 4, 2, 3)
    return np.ascontiguousarray(y).reshape(k, c, fh, fw)


def pack_dw_filter(wt: np.ndarray, cb: int = CB) -> np.ndarray:
    """[C, Fh, Fw] (or [C, 1, Fh, Fw]) -> flat [C/cb][Fh][Fw][cb]."""
    if wt.ndim == 4:
        wt = wt[:, 0]
    c, fh, fw = wt.shape
    if c % cb:
        raise RuntimeError("num_channels % channel_blocking != 0")
    y = wt.reshape(c // cb, cb, fh, fw).transpose(0, 2, 3, 1)
    return np.ascontiguousarray(y).reshape(-1)


def pad_output_channels(wt: np.ndarray, bias: np.ndarray | None, cob: int = CB):
    """Zero-pad a [K, C, Fh, Fw] filter (and its bias) up to the next multiple of the
    output block, as the reference's layer class does (include/small/Conv2DLayer.hpp
    :393-404).  Returns (filter, bias, effective_K)."""
    k = wt.shape[0]
    kp = -(-k // cob) * cob
    if kp == k:
        return wt, bias, k
    w2 = np.zeros((kp,) + wt.shape[1:], wt.dtype)
    w2[:k] = wt
    b2 = None
    if bias is not None:
        b2 = np.zeros(kp, bias.dtype)
        b2[:k] = bias
    return w2, b2, k


def calc_padding(i: int, k: int, stride: int):
    """'same' padding of one dimension, include/small/utils.hpp:43-64 -> (front, back)."""
    p = max(k - stride, 0) if i % stride == 0 else max(k - (i % stride), 0)
    return p // 2, p - p // 2


def output_dim(i: int, pad_front: int, pad_back: int, k: int, stride: int) -> int:
    """include/small/utils.hpp:159-165 on the padded extent."""
    return max((i + pad_front + pad_back - k) // stride + 1, 0)
