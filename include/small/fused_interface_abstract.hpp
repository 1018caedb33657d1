// fused_interface_abstract.hpp (B200 platform) -- the reference's fused layer functions
// (include/small/fused_interface_abstract.hpp:55-3667 of the reference, float only).
//
// One-op forms (conv / depthwise conv with bias before and ReLU after) run as ONE kernel:
// bias seeds the accumulators and the activation is applied in the output tile, which is
// what the reference's fused loop nest does (abstract_layer.hpp:2268-2969).
// conv -> 2x2 stride-2 max pool is one kernel too where the shapes allow (the pool is taken in
// registers before anything is stored).  The other two-op forms (other pools, conv -> depthwise
// conv, conv -> grouped conv) run the fused first op (bias and activation inside) into an
// intermediate buffer and the second op from there: two kernels, the full-size intermediate does
// reach memory.  The intermediate is the caller's `inter_output_buf` when that holds a whole
// intermediate tensor; the reference only needs per-thread tile scratch there
// (abstract_layer.hpp:3382,3409, no defined content on return), so a smaller one is common, and
// then a scratch buffer of the calling thread is used.
#pragma once

#include <memory>
#include <vector>

#include <small/utils.hpp>

namespace small
{
namespace b200
{
// Scratch of the calling thread for the intermediate of a two-op fused call.  Buffers are never
// freed or resized while the thread lives: a recorded InferenceGraph keeps the address it was
// recorded with, so a later, larger call gets a new buffer and the old one stays valid.  Calls of
// one thread on different streams share it (as they would share the reference's argument): give
// such calls an inter_output_buf of full size instead.
inline FloatBuffer &fused_scratch(size_t elems)
{
    static thread_local std::vector<std::unique_ptr<FloatBuffer>> pool;
    for (auto &b : pool)
        if (b->size() >= elems)
            return *b;
    pool.emplace_back(new FloatBuffer(elems));
    return *pool.back();
}

// The intermediate of a two-op call: the caller's buffer if it can hold it, else thread scratch.
template <class BufferT>
inline BufferT &fused_mid(BufferT &inter_output_buf, size_t elems)
{
    if constexpr (std::is_same_v<BufferT, FloatBuffer>)
        return inter_output_buf.size() >= elems ? inter_output_buf : fused_scratch(elems);
    else
    {
        if (inter_output_buf.size() < elems)
            throw std::invalid_argument("fused layer ERROR: inter_output_buf must hold the intermediate tensor.");
        return inter_output_buf;
    }
}

// Output extent along the height / width of a windowed layer under the current row stride.
inline int out_h(int H, int t, int b, int stride, int kh)
{
    return (int)small::output_dim(H + t + b, row_stride() > 0 ? row_stride() : stride, kh);
}
inline int out_w(int W, int l, int r, int stride, int kw) { return (int)small::output_dim(W + l + r, stride, kw); }

inline size_t conv_out_elems(int K, int H, int W, int kh, int kw, int s, int t, int b, int l, int r)
{
    return (size_t)batch() * K * out_h(H, t, b, s, kh) * out_w(W, l, r, s, kw);
}
} // namespace b200

#define SMALL_B200_CONV_ARGS                                                          \
    int conv_kernel_height, int conv_kernel_width, int conv_stride, uint8_t conv_t_pad, \
        uint8_t conv_b_pad, uint8_t conv_l_pad, uint8_t conv_r_pad
#define SMALL_B200_POOL_ARGS                                                          \
    int pool_kernel_height, int pool_kernel_width, int pool_stride, uint8_t pool_t_pad, \
        uint8_t pool_b_pad, uint8_t pool_l_pad, uint8_t pool_r_pad
#define SMALL_B200_CONV_PASS \
    conv_kernel_height, conv_kernel_width, conv_stride, conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad
#define SMALL_B200_POOL_PASS \
    pool_kernel_height, pool_kernel_width, pool_stride, pool_t_pad, pool_b_pad, pool_l_pad, pool_r_pad
#define SMALL_B200_POOL_PASS_G(groups) \
    pool_kernel_height, pool_kernel_width, pool_stride, groups, pool_t_pad, pool_b_pad, pool_l_pad, pool_r_pad
#define SMALL_B200_GPOOL_ARGS                                                          \
    int pool_kernel_height, int pool_kernel_width, int pool_stride, int output_groups,  \
        uint8_t pool_t_pad, uint8_t pool_b_pad, uint8_t pool_l_pad, uint8_t pool_r_pad

//============================================================================ one-op forms
template <class BufferT>
void Conv2D_ReLU(SMALL_B200_CONV_ARGS, int output_channels, int input_channels, int input_height,
                 int input_width, BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::conv(false, SMALL_B200_ACT_RELU, SMALL_B200_CONV_PASS, output_channels, input_channels,
               input_height, input_width, input_buf, filter_buf, (BufferT const *)nullptr, output_buf);
}

template <class BufferT>
void Conv2D_Bias_ReLU(SMALL_B200_CONV_ARGS, int output_channels, int input_channels, int input_height,
                      int input_width, BufferT const &input_buf, BufferT const &filter_buf,
                      BufferT const &bias_buf, BufferT &output_buf)
{
    b200::conv(false, SMALL_B200_ACT_RELU, SMALL_B200_CONV_PASS, output_channels, input_channels,
               input_height, input_width, input_buf, filter_buf, &bias_buf, output_buf);
}

template <class BufferT>
void DepthwiseConv2D_ReLU(SMALL_B200_CONV_ARGS, int input_channels, int input_height, int input_width,
                          BufferT const &input_buf, BufferT const &filter_buf, BufferT &output_buf)
{
    b200::dwconv(false, SMALL_B200_ACT_RELU, SMALL_B200_CONV_PASS, input_channels, input_height,
                 input_width, input_buf, filter_buf, (BufferT const *)nullptr, output_buf);
}

template <class BufferT>
void DepthwiseConv2D_Bias_ReLU(SMALL_B200_CONV_ARGS, int input_channels, int input_height, int input_width,
                               BufferT const &input_buf, BufferT const &filter_buf,
                               BufferT const &bias_buf, BufferT &output_buf)
{
    b200::dwconv(false, SMALL_B200_ACT_RELU, SMALL_B200_CONV_PASS, input_channels, input_height,
                 input_width, input_buf, filter_buf, &bias_buf, output_buf);
}

//============================================================================ conv -> max pool
namespace b200
{
template <class BufferT>
inline void conv_then_pool(int act, BufferT const *bias, SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS,
                           int K, int C, int H, int W, BufferT const &in, BufferT const &filt,
                           BufferT &inter, BufferT &out)
{
    const int Hm = out_h(H, conv_t_pad, conv_b_pad, conv_stride, conv_kernel_height);
    const int Wm = out_w(W, conv_l_pad, conv_r_pad, conv_stride, conv_kernel_width);
    if constexpr (!is_quint8<BufferT>)
    {
        // one kernel when the pair of shapes is covered: the pool is taken in registers
        small_b200_layer Lc = describe(C, K, H, W, conv_kernel_height, conv_kernel_width, conv_stride,
                                       conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad, 0, act);
        small_b200_layer Lp = describe(K, K, Hm, Wm, pool_kernel_height, pool_kernel_width, pool_stride,
                                       pool_t_pad, pool_b_pad, pool_l_pad, pool_r_pad);
        // on the tensor cores where the library prefers them for the convolution and its kernel has the
        // pooled epilogue for the pair (the re-laid filter is kept with the filter buffer, as in conv())
        if (tensor_core_enabled() && small_b200_conv2d_f32_tf32x3_preferred(&Lc) &&
            small_b200_conv2d_maxpool_f32_tf32x3_supported(&Lc, &Lp))
        {
            const uint64_t key = ((uint64_t)K << 40) ^ ((uint64_t)C << 20) ^ ((uint64_t)conv_kernel_height << 8) ^
                                 (uint64_t)conv_kernel_width;
            float *prepared = filt.companion(key);
            if (!prepared)
            {
                prepared = filt.make_companion(key, 2 * (size_t)K * C * conv_kernel_height * conv_kernel_width);
                throw_on(small_b200_filter_prepare_tf32x3(&Lc, filt.device_ptr(), prepared, b200::stream()));
            }
            throw_on(small_b200_conv2d_maxpool_f32_tf32x3(&Lc, &Lp, in.device_ptr(), prepared,
                                                          bias ? bias->device_ptr() : nullptr, out.device_ptr(), b200::stream()));
            return;
        }
        if (small_b200_conv2d_maxpool_f32_supported(&Lc, &Lp))
        {
            throw_on(small_b200_conv2d_maxpool_f32(&Lc, &Lp, in.device_ptr(), filt.device_ptr(),
                                                   bias ? bias->device_ptr() : nullptr, out.device_ptr(), b200::stream()));
            return;
        }
    }
    BufferT &mid = fused_mid(inter, conv_out_elems(K, H, W, SMALL_B200_CONV_PASS));
    conv(false, act, SMALL_B200_CONV_PASS, K, C, H, W, in, filt, bias, mid);
    pool(false, SMALL_B200_POOL_PASS, K, Hm, Wm, mid, out);
}

template <class BufferT>
inline void conv_then_dw(int act, BufferT const *bias, BufferT const *dw_bias, SMALL_B200_CONV_ARGS,
                         SMALL_B200_POOL_ARGS, int K, int C, int H, int W, BufferT const &in,
                         BufferT const &filt, BufferT const &dw_filt, BufferT &inter, BufferT &out)
{
    const int Hm = out_h(H, conv_t_pad, conv_b_pad, conv_stride, conv_kernel_height);
    const int Wm = out_w(W, conv_l_pad, conv_r_pad, conv_stride, conv_kernel_width);
    if constexpr (is_quint8<BufferT>)
    {
        // One kernel where the library covers the pair (a 1x1 or one-channel first convolution, a 3x3
        // 'same' depthwise convolution, images of at most 128 pixels): the intermediate stays in shared
        // memory and inter only lends its quantisation fields.  The clamp of the requantisation is the
        // ReLU of the quint8 forms.
        small_b200_layer Lc = describe(C, K, H, W, conv_kernel_height, conv_kernel_width, conv_stride,
                                       conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad);
        quantise(Lc, in, &filt, inter);
        small_b200_layer Ld = describe(K, K, Hm, Wm, pool_kernel_height, pool_kernel_width, pool_stride,
                                       pool_t_pad, pool_b_pad, pool_l_pad, pool_r_pad);
        quantise(Ld, inter, &dw_filt, out);
        if (!bias && !dw_bias && small_b200_conv2d_dwconv2d_u8_supported(&Lc, &Ld))
        {
            throw_on(small_b200_conv2d_dwconv2d_u8(&Lc, &Ld, in.device_ptr(), filt.device_ptr(), nullptr,
                                                   dw_filt.device_ptr(), nullptr, out.device_ptr(), b200::stream()));
            return;
        }
    }
    BufferT &mid = fused_mid(inter, conv_out_elems(K, H, W, SMALL_B200_CONV_PASS));
    conv(false, act, SMALL_B200_CONV_PASS, K, C, H, W, in, filt, bias, mid);
    dwconv(false, act, SMALL_B200_POOL_PASS, K, Hm, Wm, mid, dw_filt, dw_bias, out);
}

// The grouped convolution of the fused interface: `groups` dense 16 -> 16 convolutions, group g on
// channel block g (fused_interface_abstract.hpp:2740-2760 of the reference), with the bias-before /
// activation-after slots.
template <class BufferT>
inline void blockconv(int act, BufferT const *bias, int kh, int kw, int stride, int groups, int t, int b, int l,
                      int r, int C, int H, int W, BufferT const &in, BufferT const &filt, BufferT &out,
                      char const *name)
{
    if constexpr (is_quint8<BufferT>)
        throw std::invalid_argument(std::string(name) + "<quint8> ERROR: not provided (float only, as in the reference).");
    else
    {
        if (C % SMALL_B200_CB != 0)
            throw std::invalid_argument(std::string(name) + "<float> ERROR: in_channels unsupported.");
        if (stride != 1 && stride != 2)
            throw std::invalid_argument(std::string(name) + "<float> ERROR: conv_stride unsupported.");
        small_b200_layer L = describe(SMALL_B200_CB, SMALL_B200_CB, H, W, kh, kw, stride, t, b, l, r, 0, act);
        throw_on(small_b200_blockconv2d_f32(&L, groups, in.device_ptr(), filt.device_ptr(),
                                            bias ? bias->device_ptr() : nullptr, out.device_ptr(), b200::stream()));
    }
}

template <class BufferT>
inline void conv_then_blockconv(int act, BufferT const *bias, BufferT const *g_bias, SMALL_B200_CONV_ARGS,
                                SMALL_B200_POOL_ARGS, int groups, int K, int C, int H, int W, BufferT const &in,
                                BufferT const &filt, BufferT const &g_filt, BufferT &inter, BufferT &out,
                                char const *name)
{
    BufferT &mid = fused_mid(inter, conv_out_elems(K, H, W, SMALL_B200_CONV_PASS));
    conv(false, act, SMALL_B200_CONV_PASS, K, C, H, W, in, filt, bias, mid);
    const int Hm = out_h(H, conv_t_pad, conv_b_pad, conv_stride, conv_kernel_height);
    const int Wm = out_w(W, conv_l_pad, conv_r_pad, conv_stride, conv_kernel_width);
    blockconv(act, g_bias, SMALL_B200_POOL_PASS_G(groups), K, Hm, Wm, mid, g_filt, out, name);
}
} // namespace b200

template <class BufferT>
void Conv2D_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels, int input_channels,
                      int input_height, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT &inter_output_buf, BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_NONE, (BufferT const *)nullptr, SMALL_B200_CONV_PASS,
                         SMALL_B200_POOL_PASS, output_channels, input_channels, input_height,
                         input_width, input_buf, filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv2D_ReLU_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                           int input_channels, int input_height, int input_width,
                           BufferT const &input_buf, BufferT const &filter_buf,
                           BufferT &inter_output_buf, BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, SMALL_B200_CONV_PASS,
                         SMALL_B200_POOL_PASS, output_channels, input_channels, input_height,
                         input_width, input_buf, filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv2D_Bias_ReLU_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                                int input_channels, int input_height, int input_width,
                                BufferT const &input_buf, BufferT const &filter_buf,
                                BufferT const &bias_buf, BufferT &inter_output_buf,
                                BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_RELU, &bias_buf, SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS,
                         output_channels, input_channels, input_height, input_width, input_buf,
                         filter_buf, inter_output_buf, output_buf);
}

//============================================================================ conv -> depthwise conv
template <class BufferT>
void Conv2D_DepthwiseConv2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                            int input_channels, int input_height, int input_width,
                            BufferT const &input_buf, BufferT const &filter_buf,
                            BufferT &inter_output_buf, BufferT const &dwise_filter_buf,
                            BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_NONE, (BufferT const *)nullptr, (BufferT const *)nullptr,
                       SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_channels, input_channels,
                       input_height, input_width, input_buf, filter_buf, dwise_filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv2D_ReLU_DepthwiseConv2D_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                                      int input_channels, int input_height, int input_width,
                                      BufferT const &input_buf, BufferT const &filter_buf,
                                      BufferT &inter_output_buf, BufferT const &dwise_filter_buf,
                                      BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, (BufferT const *)nullptr,
                       SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_channels, input_channels,
                       input_height, input_width, input_buf, filter_buf, dwise_filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv2D_Bias_ReLU_DepthwiseConv2D_Bias_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS,
                                                int output_channels, int input_channels,
                                                int input_height, int input_width,
                                                BufferT const &input_buf, BufferT const &filter_buf,
                                                BufferT const &bias_buf, BufferT &inter_output_buf,
                                                BufferT const &dwise_filter_buf,
                                                BufferT const &dwise_bias_buf, BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_RELU, &bias_buf, &dwise_bias_buf, SMALL_B200_CONV_PASS,
                       SMALL_B200_POOL_PASS, output_channels, input_channels, input_height, input_width,
                       input_buf, filter_buf, dwise_filter_buf, inter_output_buf, output_buf);
}

//============================================================================ grouped forms
// fused_interface_abstract.hpp:2507-3667 of the reference.  The grouped convolution of this family is
// `output_groups` dense convolutions from 16 to 16 channels, one per channel block (see blockconv above).
template <class BufferT>
void GroupConv2D_ReLU(int conv_kernel_height, int conv_kernel_width, int conv_stride, int output_groups,
                      uint8_t conv_t_pad, uint8_t conv_b_pad, uint8_t conv_l_pad, uint8_t conv_r_pad,
                      int input_channels, int input_height, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT &output_buf)
{
    b200::blockconv(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, conv_kernel_height, conv_kernel_width,
                    conv_stride, output_groups, conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad, input_channels,
                    input_height, input_width, input_buf, filter_buf, output_buf, "GroupConv2D_ReLU");
}

template <class BufferT>
void GroupConv2D_Bias_ReLU(int conv_kernel_height, int conv_kernel_width, int conv_stride, int output_groups,
                           uint8_t conv_t_pad, uint8_t conv_b_pad, uint8_t conv_l_pad, uint8_t conv_r_pad,
                           int input_channels, int input_height, int input_width, BufferT const &input_buf,
                           BufferT const &filter_buf, BufferT const &bias_buf, BufferT &output_buf)
{
    b200::blockconv(SMALL_B200_ACT_RELU, &bias_buf, conv_kernel_height, conv_kernel_width, conv_stride,
                    output_groups, conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad, input_channels, input_height,
                    input_width, input_buf, filter_buf, output_buf, "GroupConv2D_Bias_ReLU");
}

template <class BufferT>
void Conv2D_GroupConv(SMALL_B200_CONV_ARGS, SMALL_B200_GPOOL_ARGS, int output_channels, int input_channels,
                      int input_height, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
                      BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::conv_then_blockconv(SMALL_B200_ACT_NONE, (BufferT const *)nullptr, (BufferT const *)nullptr,
                              SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_groups, output_channels,
                              input_channels, input_height, input_width, input_buf, filter_buf, dwise_filter_buf,
                              inter_output_buf, output_buf, "Conv2D_GroupConv");
}

template <class BufferT>
void Conv2D_ReLU_GroupConv2D_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_GPOOL_ARGS, int output_channels,
                                  int input_channels, int input_height, int input_width,
                                  BufferT const &input_buf, BufferT const &filter_buf, BufferT &inter_output_buf,
                                  BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::conv_then_blockconv(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, (BufferT const *)nullptr,
                              SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_groups, output_channels,
                              input_channels, input_height, input_width, input_buf, filter_buf, dwise_filter_buf,
                              inter_output_buf, output_buf, "Conv2D_ReLU_GroupConv2D_ReLU");
}

template <class BufferT>
void Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_GPOOL_ARGS, int output_channels,
                                            int input_channels, int input_height, int input_width,
                                            BufferT const &input_buf, BufferT const &filter_buf,
                                            BufferT const &bias_buf, BufferT &inter_output_buf,
                                            BufferT const &dwise_filter_buf, BufferT const &dwise_bias_buf,
                                            BufferT &output_buf)
{
    b200::conv_then_blockconv(SMALL_B200_ACT_RELU, &bias_buf, &dwise_bias_buf, SMALL_B200_CONV_PASS,
                              SMALL_B200_POOL_PASS, output_groups, output_channels, input_channels, input_height,
                              input_width, input_buf, filter_buf, dwise_filter_buf, inter_output_buf, output_buf,
                              "Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU");
}

} // namespace small
