// fused_interface_abstract.hpp (B200 platform) -- the reference's fused layer functions
// (include/small/fused_interface_abstract.hpp:55-3667 of the reference, float only).
//
// One-op forms (conv / depthwise conv with bias before and ReLU after) run as ONE kernel:
// bias seeds the accumulators and the activation is applied in the output tile, which is
// what the reference's fused loop nest does (abstract_layer.hpp:2268-2969).
// conv -> 2x2 stride-2 max pool is one kernel too where the shapes allow (the pool is taken in
// registers before anything is stored).  The other two-op forms (other pools, conv -> depthwise
// conv) run the fused first op into a device scratch buffer owned by this header and the second
// op from there.  The reference's
// `inter_output_buf` argument is per-thread scratch of its CPU loop nest
// (abstract_layer.hpp:3382,3409) with no defined content on return; it is left untouched.
#pragma once

#include <small/utils.hpp>

namespace small
{
namespace b200
{
// Grow-only device scratch for the intermediate of a two-op fused call.
inline FloatBuffer &fused_scratch(size_t elems)
{
    static FloatBuffer buf;
    if (buf.size() < elems)
        buf = FloatBuffer(elems);
    return buf;
}

inline size_t conv_out_elems(int K, int H, int W, int kh, int kw, int s, int t, int b, int l, int r)
{
    return (size_t)batch() * K * small::output_dim(H + t + b, s, kh) * small::output_dim(W + l + r, s, kw);
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
                           int K, int C, int H, int W, BufferT const &in, BufferT const &filt, BufferT &out)
{
    const int Hm = small::output_dim(H + conv_t_pad + conv_b_pad, conv_stride, conv_kernel_height);
    const int Wm = small::output_dim(W + conv_l_pad + conv_r_pad, conv_stride, conv_kernel_width);
    if constexpr (!is_quint8<BufferT>)
    {
        // one kernel when the pair of shapes is covered: the pool is taken in registers
        small_b200_layer Lc = describe(C, K, H, W, conv_kernel_height, conv_kernel_width, conv_stride,
                                       conv_t_pad, conv_b_pad, conv_l_pad, conv_r_pad, 0, act);
        small_b200_layer Lp = describe(K, K, Hm, Wm, pool_kernel_height, pool_kernel_width, pool_stride,
                                       pool_t_pad, pool_b_pad, pool_l_pad, pool_r_pad);
        if (small_b200_conv2d_maxpool_f32_supported(&Lc, &Lp))
        {
            throw_on(small_b200_conv2d_maxpool_f32(&Lc, &Lp, in.device_ptr(), filt.device_ptr(),
                                                   bias ? bias->device_ptr() : nullptr, out.device_ptr(), b200::stream()));
            return;
        }
    }
    FloatBuffer &mid = fused_scratch(conv_out_elems(K, H, W, SMALL_B200_CONV_PASS));
    conv(false, act, SMALL_B200_CONV_PASS, K, C, H, W, in, filt, bias, mid);
    pool(false, SMALL_B200_POOL_PASS, K, Hm, Wm, mid, out);
}

template <class BufferT>
inline void conv_then_dw(int act, BufferT const *bias, BufferT const *dw_bias, SMALL_B200_CONV_ARGS,
                         SMALL_B200_POOL_ARGS, int K, int C, int H, int W, BufferT const &in,
                         BufferT const &filt, BufferT const &dw_filt, BufferT &out)
{
    FloatBuffer &mid = fused_scratch(conv_out_elems(K, H, W, SMALL_B200_CONV_PASS));
    conv(false, act, SMALL_B200_CONV_PASS, K, C, H, W, in, filt, bias, mid);
    const int Hm = small::output_dim(H + conv_t_pad + conv_b_pad, conv_stride, conv_kernel_height);
    const int Wm = small::output_dim(W + conv_l_pad + conv_r_pad, conv_stride, conv_kernel_width);
    dwconv(false, act, SMALL_B200_POOL_PASS, K, Hm, Wm, mid, dw_filt, dw_bias, out);
}
} // namespace b200

template <class BufferT>
void Conv2D_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels, int input_channels,
                      int input_height, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT & /*inter_output_buf*/, BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_NONE, (BufferT const *)nullptr, SMALL_B200_CONV_PASS,
                         SMALL_B200_POOL_PASS, output_channels, input_channels, input_height,
                         input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT>
void Conv2D_ReLU_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                           int input_channels, int input_height, int input_width,
                           BufferT const &input_buf, BufferT const &filter_buf,
                           BufferT & /*inter_output_buf*/, BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, SMALL_B200_CONV_PASS,
                         SMALL_B200_POOL_PASS, output_channels, input_channels, input_height,
                         input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT>
void Conv2D_Bias_ReLU_Maxpool2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                                int input_channels, int input_height, int input_width,
                                BufferT const &input_buf, BufferT const &filter_buf,
                                BufferT const &bias_buf, BufferT & /*inter_output_buf*/,
                                BufferT &output_buf)
{
    b200::conv_then_pool(SMALL_B200_ACT_RELU, &bias_buf, SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS,
                         output_channels, input_channels, input_height, input_width, input_buf,
                         filter_buf, output_buf);
}

//============================================================================ conv -> depthwise conv
template <class BufferT>
void Conv2D_DepthwiseConv2D(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                            int input_channels, int input_height, int input_width,
                            BufferT const &input_buf, BufferT const &filter_buf,
                            BufferT & /*inter_output_buf*/, BufferT const &dwise_filter_buf,
                            BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_NONE, (BufferT const *)nullptr, (BufferT const *)nullptr,
                       SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_channels, input_channels,
                       input_height, input_width, input_buf, filter_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv2D_ReLU_DepthwiseConv2D_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS, int output_channels,
                                      int input_channels, int input_height, int input_width,
                                      BufferT const &input_buf, BufferT const &filter_buf,
                                      BufferT & /*inter_output_buf*/, BufferT const &dwise_filter_buf,
                                      BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_RELU, (BufferT const *)nullptr, (BufferT const *)nullptr,
                       SMALL_B200_CONV_PASS, SMALL_B200_POOL_PASS, output_channels, input_channels,
                       input_height, input_width, input_buf, filter_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv2D_Bias_ReLU_DepthwiseConv2D_Bias_ReLU(SMALL_B200_CONV_ARGS, SMALL_B200_POOL_ARGS,
                                                int output_channels, int input_channels,
                                                int input_height, int input_width,
                                                BufferT const &input_buf, BufferT const &filter_buf,
                                                BufferT const &bias_buf, BufferT & /*inter_output_buf*/,
                                                BufferT const &dwise_filter_buf,
                                                BufferT const &dwise_bias_buf, BufferT &output_buf)
{
    b200::conv_then_dw(SMALL_B200_ACT_RELU, &bias_buf, &dwise_bias_buf, SMALL_B200_CONV_PASS,
                       SMALL_B200_POOL_PASS, output_channels, input_channels, input_height, input_width,
                       input_buf, filter_buf, dwise_filter_buf, output_buf);
}

//============================================================================ grouped forms
// The grouped convolution is not provided on this platform (see GroupConv2D).
#define SMALL_B200_NO_GROUP(name)                                                         \
    template <class BufferT, class... Rest>                                               \
    void name(Rest &&...)                                                                 \
    {                                                                                     \
        throw std::invalid_argument(#name " ERROR: not provided on the B200 platform.");  \
    }
SMALL_B200_NO_GROUP(GroupConv2D_ReLU)
SMALL_B200_NO_GROUP(GroupConv2D_Bias_ReLU)
SMALL_B200_NO_GROUP(Conv2D_GroupConv)
SMALL_B200_NO_GROUP(Conv2D_ReLU_GroupConv2D_ReLU)
SMALL_B200_NO_GROUP(Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU)
#undef SMALL_B200_NO_GROUP

} // namespace small
