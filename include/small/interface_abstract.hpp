// interface_abstract.hpp (B200 platform) -- definitions of the functional layer interface
// declared in the reference's include/small/interface.hpp:49-497.
//
// The reference defines each function as a set of instantiations of its CPU loop nest.
// Here each function fills a small_b200_layer descriptor and calls the matching entry
// point of libsmall_b200.so (include/small_b200.h).  Signatures, accepted arguments and
// the exceptions thrown for unsupported strides / channel counts are the reference's.
// Calls are asynchronous; results become visible to the host through Buffer::data() /
// operator[], which wait for the device.
#pragma once

#include <stdint.h>

#include <cstdlib>
#include <stdexcept>
#include <string>
#include <type_traits>

#include <small/op_type.hpp>
#include <small/utils.hpp>

namespace small
{
namespace b200
{
template <class BufferT>
inline constexpr bool is_quint8 = std::is_same_v<BufferT, QUInt8Buffer>;

inline small_b200_layer describe(int C, int K, int H, int W, int Fh, int Fw, int stride,
                                 int t, int b, int l, int r, int accumulate = 0,
                                 int act = SMALL_B200_ACT_NONE, float slope = 0.f)
{
    small_b200_layer L{};
    L.N = batch();
    L.C = C; L.K = K; L.H = H; L.W = W; L.Fh = Fh; L.Fw = Fw; L.stride = stride;
    L.pad_t = t; L.pad_b = b; L.pad_l = l; L.pad_r = r;
    L.accumulate = accumulate; L.act = act; L.slope = slope;
    L.stride_h = row_stride();
    return L;
}

// Quantisation parameters travel inside the buffers (QUInt8Buffer.hpp:222-230): zero points
// of input and filter, multiplier and shifts of the OUTPUT (q_abstract_layer.hpp:922-938).
template <class BufferT>
inline void quantise(small_b200_layer &L, BufferT const &in, BufferT const *filt, BufferT const &out)
{
    if constexpr (is_quint8<BufferT>)
    {
        L.zero_in = in.zero();
        L.zero_filt = filt ? filt->zero() : 0;
        L.lshift = out.lshift; L.rshift = out.rshift; L.multiplier = out.multiplier;
        L.k_zero = 0;
    }
}

// On by default: fp32 convolutions the library prefers on the tensor cores
// (small_b200_conv2d_f32_tf32x3_preferred) run there.  Against an fp64 recomputation the 3xTF32
// kernel is closer to the exact result than the reference's sequential fp32 sum, and the
// reference's own tests (|x - golden| <= 1e-5 + 5e-3 |golden| element by element,
// test/include/test_utils.hpp) pass on it.  SMALL_B200_TENSOR_CORE=0 in the environment, or
// small::b200::tensor_core() = false, keeps every convolution on the CUDA cores.
inline bool &tensor_core()
{
    static bool on = [] {
        const char *e = std::getenv("SMALL_B200_TENSOR_CORE");
        return !(e && e[0] == '0');
    }();
    return on;
}
inline bool tensor_core_enabled() { return tensor_core(); }

template <class BufferT>
inline void conv(bool partial, int act, int kh, int kw, int stride, int t, int b, int l, int r,
                 int K, int C, int H, int W, BufferT const &in, BufferT const &filt,
                 BufferT const *bias, BufferT &out)
{
    flush_deferred();
    small_b200_layer L = describe(C, K, H, W, kh, kw, stride, t, b, l, r, partial, act);
    quantise(L, in, &filt, out);
    if constexpr (is_quint8<BufferT>)
    {
        if (bias)
            throw std::invalid_argument("Conv2D<quint8> ERROR: a uint8 bias buffer is not meaningful; "
                                        "pass an int32 bias through the C ABI.");
        throw_on(small_b200_conv2d_u8(&L, in.device_ptr(), filt.device_ptr(), nullptr, out.device_ptr(), b200::stream()));
    }
    else
    {
        // A call without an activation whose arguments the library accepts waits for the next call:
        // an in-place ReLU / LeakyReLU of its output becomes its epilogue (DeferredConv, Buffer.hpp).
        const bool acceptable = (stride == 1 || stride == 2) && (C % SMALL_B200_CB == 0 || C == 1 || C == 2 || C == 3) &&
                                K > 0 && K % SMALL_B200_CB == 0 && H > 0 && W > 0 && kh > 0 && kw > 0;
        const bool defer = act == SMALL_B200_ACT_NONE && acceptable;
        const long long out_elems = (long long)L.N * K *
                                    (long long)small::output_dim(H + t + b, row_stride() > 0 ? row_stride() : stride, kh) *
                                    (long long)small::output_dim(W + l + r, stride, kw);
        // Wide stride-1 layers run on the tensor cores (tcgen05 kind::tf32, 3xTF32 split).  The
        // kernel wants the filter re-laid; that copy is made once and kept with the filter buffer
        // until the host touches the buffer again.
        if (tensor_core_enabled() && small_b200_conv2d_f32_tf32x3_preferred(&L))
        {
            const uint64_t key = ((uint64_t)K << 40) ^ ((uint64_t)C << 20) ^ ((uint64_t)kh << 8) ^ (uint64_t)kw;
            float *prepared = filt.companion(key);
            if (!prepared)
            {
                prepared = filt.make_companion(key, 2 * (size_t)K * C * kh * kw);
                throw_on(small_b200_filter_prepare_tf32x3(&L, filt.device_ptr(), prepared, b200::stream()));
            }
            const float *ip = in.device_ptr(), *bp = bias ? bias->device_ptr() : nullptr;
            float *op = out.device_ptr();
            if (defer)
            {
                DeferredConv &d = deferred();
                d.L = L; d.in = ip; d.filt = prepared; d.bias = bp; d.out = op; d.on_stream = b200::stream();
                d.tensor_core = true; d.depthwise = false; d.out_elems = out_elems; d.valid = true;
            }
            else
                throw_on(small_b200_conv2d_f32_tf32x3(&L, ip, prepared, bp, op, b200::stream()));
        }
        else
        {
            const float *ip = in.device_ptr(), *fp = filt.device_ptr(), *bp = bias ? bias->device_ptr() : nullptr;
            float *op = out.device_ptr();
            if (defer)
            {
                DeferredConv &d = deferred();
                d.L = L; d.in = ip; d.filt = fp; d.bias = bp; d.out = op; d.on_stream = b200::stream();
                d.tensor_core = false; d.depthwise = false; d.out_elems = out_elems; d.valid = true;
            }
            else
                throw_on(small_b200_conv2d_f32(&L, ip, fp, bp, op, b200::stream()));
        }
    }
}

// An in-place activation of the output of the convolution that is waiting: taken into its epilogue.
template <class BufferT>
inline bool fuse_activation(BufferT const &in, BufferT &out, int64_t n, int act, float slope)
{
    if constexpr (is_quint8<BufferT>)
        return false;
    else
    {
        DeferredConv &d = deferred();
        if (!d.valid || d.L.act != SMALL_B200_ACT_NONE || in.raw_ptr() != out.raw_ptr() || out.raw_ptr() != d.out ||
            n != d.out_elems || d.on_stream != b200::stream())
            return false;
        d.L.act = act;
        d.L.slope = slope;
        return true;
    }
}

template <class BufferT>
inline void dwconv(bool partial, int act, int kh, int kw, int stride, int t, int b, int l, int r,
                   int C, int H, int W, BufferT const &in, BufferT const &filt, BufferT const *bias,
                   BufferT &out)
{
    small_b200_layer L = describe(C, C, H, W, kh, kw, stride, t, b, l, r, partial, act);
    quantise(L, in, &filt, out);
    if constexpr (is_quint8<BufferT>)
    {
        if (bias)
            throw std::invalid_argument("DepthwiseConv2D<quint8> ERROR: a uint8 bias buffer is not meaningful; "
                                        "pass an int32 bias through the C ABI.");
        throw_on(small_b200_dwconv2d_u8(&L, in.device_ptr(), filt.device_ptr(), nullptr, out.device_ptr(), b200::stream()));
    }
    else
    {
        // deferred like the dense convolution (DeferredConv, Buffer.hpp): an in-place activation joins it
        const float *ip = in.device_ptr(), *fp = filt.device_ptr(), *bp = bias ? bias->device_ptr() : nullptr;
        float *op = out.device_ptr();
        if (act == SMALL_B200_ACT_NONE && (stride == 1 || stride == 2) && C > 0 && C % SMALL_B200_CB == 0 && H > 0 &&
            W > 0 && kh > 0 && kw > 0)
        {
            DeferredConv &d = deferred();
            d.L = L; d.in = ip; d.filt = fp; d.bias = bp; d.out = op; d.on_stream = b200::stream();
            d.tensor_core = false; d.depthwise = true; d.valid = true;
            d.out_elems = (long long)L.N * C *
                          (long long)small::output_dim(H + t + b, row_stride() > 0 ? row_stride() : stride, kh) *
                          (long long)small::output_dim(W + l + r, stride, kw);
        }
        else
            throw_on(small_b200_dwconv2d_f32(&L, ip, fp, bp, op, b200::stream()));
    }
}

template <class BufferT>
inline void groupconv(bool partial, int kh, int kw, int stride, int groups, int t, int b, int l, int r,
                      int C, int H, int W, BufferT const &in, BufferT const &filt, BufferT &out)
{
    const char *type = is_quint8<BufferT> ? "quint8" : "float";
    if (C % SMALL_B200_CB != 0)
        throw std::invalid_argument(std::string("GroupConv2D<") + type + "> ERROR: in_channels unsupported.");
    small_b200_layer L = describe(C, C, H, W, kh, kw, stride, t, b, l, r, partial);
    quantise(L, in, &filt, out);
    if constexpr (is_quint8<BufferT>)
        throw_on(small_b200_groupconv2d_u8(&L, groups, in.device_ptr(), filt.device_ptr(), nullptr,
                                           out.device_ptr(), b200::stream()));
    else
        throw_on(small_b200_groupconv2d_f32(&L, groups, in.device_ptr(), filt.device_ptr(), nullptr,
                                            out.device_ptr(), b200::stream()));
}

template <class BufferT>
inline void pool(bool average, int kh, int kw, int stride, int t, int b, int l, int r, int C, int H,
                 int W, BufferT const &in, BufferT &out)
{
    small_b200_layer L = describe(C, C, H, W, kh, kw, stride, t, b, l, r);
    quantise(L, in, (BufferT const *)nullptr, out);
    if constexpr (is_quint8<BufferT>)
        throw_on((average ? small_b200_avgpool2d_u8 : small_b200_maxpool2d_u8)(
            &L, in.device_ptr(), out.device_ptr(), b200::stream()));
    else
        throw_on((average ? small_b200_avgpool2d_f32 : small_b200_maxpool2d_f32)(
            &L, in.device_ptr(), out.device_ptr(), b200::stream()));
}

inline void require_block(int channels, int block, char const *msg)
{
    if (channels % block != 0)
        throw std::invalid_argument(msg);
}
} // namespace b200

//============================================================================
template <class BufferT, bool = true>
void Conv2D(int kernel_height, int kernel_width, int stride,
            uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
            int output_channels, int input_channels, int input_height, int input_width,
            BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::conv(false, SMALL_B200_ACT_NONE, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad,
               r_pad, output_channels, input_channels, input_height, input_width, input_buf,
               filter_buf, (BufferT const *)nullptr, output_buf);
}

template <class BufferT, bool = true>
void PartialConv2D(int kernel_height, int kernel_width, int stride,
                   uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                   int output_channels, int input_channels, int input_height, int input_width,
                   BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::conv(true, SMALL_B200_ACT_NONE, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad,
               r_pad, output_channels, input_channels, input_height, input_width, input_buf,
               filter_buf, (BufferT const *)nullptr, output_buf);
}

template <class BufferT, bool = true>
void DepthwiseConv2D(int kernel_height, int kernel_width, int stride,
                     uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                     int input_channels, int input_height, int input_width,
                     BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::dwconv(false, SMALL_B200_ACT_NONE, kernel_height, kernel_width, stride, t_pad, b_pad,
                 l_pad, r_pad, input_channels, input_height, input_width, input_buf, filter_buf,
                 (BufferT const *)nullptr, output_buf);
}

template <class BufferT, bool = true>
void PartialDepthwiseConv2D(int kernel_height, int kernel_width, int stride,
                            uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                            int input_channels, int input_height, int input_width,
                            BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::dwconv(true, SMALL_B200_ACT_NONE, kernel_height, kernel_width, stride, t_pad, b_pad,
                 l_pad, r_pad, input_channels, input_height, input_width, input_buf, filter_buf,
                 (BufferT const *)nullptr, output_buf);
}

// Grouped convolution (reference: interface_abstract.hpp:1265, :1332, :1402, :1470).  The 16
// lanes of a block are 16 groups, each a convolution from input_channels to input_channels
// channels: I [G/16][C][H][W][16], F [G/16][C][C][Fh][Fw][16], O [G/16][C][Ho][Wo][16].  The
// same argument checks and messages as the reference, plus a check of output_groups (the
// reference's nest silently assumes a multiple of the block).
template <class BufferT, bool = true>
void GroupConv2D(int kernel_height, int kernel_width, int stride, int output_groups,
                 uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                 int input_channels, int input_height, int input_width,
                 BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::groupconv(false, kernel_height, kernel_width, stride, output_groups, t_pad, b_pad, l_pad,
                    r_pad, input_channels, input_height, input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void PartialGroupConv2D(int kernel_height, int kernel_width, int stride, int output_groups,
                        uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                        int input_channels, int input_height, int input_width,
                        BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::groupconv(true, kernel_height, kernel_width, stride, output_groups, t_pad, b_pad, l_pad,
                    r_pad, input_channels, input_height, input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void MaxPool2D(int kernel_height, int kernel_width, int stride,
               uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
               int input_channels, int input_height, int input_width,
               BufferT const &input_buf, BufferT &output_buf)
{
    b200::pool(false, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
               input_channels, input_height, input_width, input_buf, output_buf);
}

template <class BufferT, bool = true>
void AveragePool2D(int kernel_height, int kernel_width, int stride,
                   uint8_t t_pad, uint8_t b_pad, uint8_t l_pad, uint8_t r_pad,
                   int input_channels, int input_height, int input_width,
                   BufferT const &input_buf, BufferT &output_buf)
{
    b200::pool(true, kernel_height, kernel_width, stride, t_pad, b_pad, l_pad, r_pad,
               input_channels, input_height, input_width, input_buf, output_buf);
}

template <class BufferT, bool = true>
void ReLUActivation(int input_channels, int input_height, int input_width,
                    BufferT const &input_buf, BufferT &output_buf)
{
    const int64_t n = (int64_t)b200::batch() * input_channels * input_height * input_width;
    if constexpr (b200::is_quint8<BufferT>)
    {
        b200::require_block(input_channels, QUINT8_C_ib, "ReLUActivation<quint8> ERROR: in_channels unsupported.");
        small_b200_layer L = b200::describe(input_channels, input_channels, input_height, input_width,
                                            1, 1, 1, 0, 0, 0, 0);
        b200::quantise(L, input_buf, (BufferT const *)nullptr, output_buf);
        b200::throw_on(small_b200_relu_u8(n, &L, input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
    }
    else
    {
        b200::require_block(input_channels, FLOAT_C_ib, "ReLUActivation<float> ERROR: in_channels unsupported.");
        if (b200::fuse_activation(input_buf, output_buf, n, SMALL_B200_ACT_RELU, 0.f))
            return;
        b200::throw_on(small_b200_relu_f32(n, input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
    }
}

// The slope arrives as a one-element buffer (interface_abstract.hpp:1616-1647).
template <class BufferT, bool = true>
void LeakyReLUActivation(int input_channels, int input_height, int input_width,
                         BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "LeakyReLUActivation: no quint8 form in the reference either");
    b200::require_block(input_channels, FLOAT_C_ib, "LeakyReLUActivation<float> ERROR: in_channels unsupported.");
    const float slope = filter_buf.peek(0); // a parameter no kernel writes: no wait for the device
    const int64_t n = (int64_t)b200::batch() * input_channels * input_height * input_width;
    if (b200::fuse_activation(input_buf, output_buf, n, SMALL_B200_ACT_LEAKY, slope))
        return;
    b200::throw_on(small_b200_leaky_relu_f32(n, input_buf.device_ptr(), slope, output_buf.device_ptr(), b200::stream()));
}

// interface_abstract.hpp:1697 of the reference: output = input * filter_buf[0] (float only there too).
template <class BufferT, bool = true>
void Dropout(int input_channels, int input_height, int input_width,
             BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "Dropout: float only, as in the reference");
    b200::require_block(input_channels, FLOAT_C_ib, "Dropout<float> ERROR: in_channels unsupported.");
    const float rate = filter_buf.peek(0); // a parameter no kernel writes: no wait for the device
    const int64_t n = (int64_t)b200::batch() * input_channels * input_height * input_width;
    b200::throw_on(small_b200_scale_f32(n, input_buf.device_ptr(), rate, output_buf.device_ptr(), b200::stream()));
}

template <class BufferT, bool = true>
void SoftMax(int input_channels, int input_height, int input_width,
             BufferT const &input_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "SoftMax: float only, as in the reference");
    b200::require_block(input_channels, FLOAT_C_ib, "SoftMax<float> ERROR: in_channels unsupported.");
    b200::throw_on(small_b200_softmax_f32(b200::batch(), (int64_t)input_channels * input_height * input_width,
                                          input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
}

template <class BufferT, bool = true>
void UpSample2D(int scale_factor, int input_channels, int input_height, int input_width,
                BufferT const &input_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "UpSample2D: float only, as in the reference");
    if (scale_factor == 1)
        output_buf = input_buf; // the reference deep-copies too (:1859)
    else if (scale_factor == 2)
    {
        b200::require_block(input_channels, FLOAT_C_ib, "Upsample<float> ERROR: in_channels unsupported.");
        b200::throw_on(small_b200_upsample2d_f32(b200::batch(), input_channels, input_height, input_width,
                                                 input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
    }
    else
        throw std::invalid_argument("Upsample<float> ERROR: scale factor unsupported (only 1 or 2).");
}

template <class BufferT, bool = true>
void Accum(int input_channels, int input_height, int input_width,
           BufferT const &input_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "Accum: float only, as in the reference");
    b200::require_block(input_channels, FLOAT_C_ib, "Accum<float> ERROR: in_channels unsupported.");
    const int64_t n = (int64_t)b200::batch() * input_channels * input_height * input_width;
    b200::throw_on(small_b200_accum_f32(n, input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
}

template <class BufferT, bool = true>
void Bias(int num_channels, int output_height, int output_width,
          BufferT const &input_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "Bias: float only, as in the reference");
    b200::require_block(num_channels, FLOAT_C_ob, "Bias<float> ERROR: in_channels unsupported.");
    b200::throw_on(small_b200_bias_f32(b200::batch(), num_channels, output_height, output_width,
                                       input_buf.device_ptr(), 0, output_buf.device_ptr(), b200::stream()));
}

template <class BufferT, bool = true>
void PartialBias(int num_channels, int output_height, int output_width,
                 BufferT const &input_buf, BufferT &output_buf)
{
    static_assert(!b200::is_quint8<BufferT>, "PartialBias: float only, as in the reference");
    b200::require_block(num_channels, FLOAT_C_ob, "PartialBias<float> ERROR: in_channels unsupported.");
    b200::throw_on(small_b200_bias_f32(b200::batch(), num_channels, output_height, output_width,
                                       input_buf.device_ptr(), 1, output_buf.device_ptr(), b200::stream()));
}

// Channel concatenation of two packed buffers = two contiguous copies per image
// (interface_abstract.hpp:2072-2103).
template <class BufferT>
void Concat(uint32_t input0_channels, uint32_t input1_channels,
            uint32_t input_height, uint32_t input_width,
            BufferT const &input0_buf, BufferT const &input1_buf, BufferT &output_buf)
{
    const size_t esz = sizeof(typename BufferT::value_type);
    b200::throw_on(small_b200_concat(b200::batch(),
                                     (size_t)input0_channels * input_height * input_width * esz,
                                     input0_buf.device_ptr(),
                                     (size_t)input1_channels * input_height * input_width * esz,
                                     input1_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
}

// The reference's Dense is a placeholder that instantiates a 1x1 depthwise operation over a
// 1 x input_elements image with output_elements channels (interface_abstract.hpp:2113-2160);
// the same instantiation is issued here.  A real fully connected layer is Conv2D 1x1 on a
// 1x1 image, which is what the reference's models use (models/DSCNNTiny.hpp:255-263).
template <class BufferT, bool = true>
void Dense(int output_elements, int input_elements,
           BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::dwconv(false, SMALL_B200_ACT_NONE, 1, 1, 1, 0, 0, 0, 0, output_elements, 1, input_elements,
                 input_buf, filter_buf, (BufferT const *)nullptr, output_buf);
}

} // namespace small
