// fused_interface_abstract_1D.hpp (B200 platform) -- the fused 1-D forms of the reference
// (include/small/fused_interface_abstract_1D.hpp:55-3321): each is the fused 2-D form with a
// window height of 1 and every row (batch entry) kept, i.e. called under a RowStrideScope(1)
// (see interface_abstract_1D.hpp of this platform).
#pragma once

namespace small
{
#define SMALL_B200_C1_ARGS int conv_kernel_width, int conv_stride, uint8_t conv_l_pad, uint8_t conv_r_pad
#define SMALL_B200_P1_ARGS int pool_kernel_width, int pool_stride, uint8_t pool_l_pad, uint8_t pool_r_pad
#define SMALL_B200_G1_ARGS \
    int pool_kernel_width, int pool_stride, int output_groups, uint8_t pool_l_pad, uint8_t pool_r_pad
#define SMALL_B200_C1_PASS 1, conv_kernel_width, conv_stride, 0, 0, conv_l_pad, conv_r_pad
#define SMALL_B200_P1_PASS 1, pool_kernel_width, pool_stride, 0, 0, pool_l_pad, pool_r_pad
#define SMALL_B200_G1_PASS 1, pool_kernel_width, pool_stride, output_groups, 0, 0, pool_l_pad, pool_r_pad

template <class BufferT>
void Conv1D_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                 int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                 BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_ReLU(1, kernel_width, stride, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
                input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_Bias_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                      int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT const &bias_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_Bias_ReLU(1, kernel_width, stride, 0, 0, l_pad, r_pad, output_channels, input_channels,
                     batch_size, input_width, input_buf, filter_buf, bias_buf, output_buf);
}

template <class BufferT>
void DepthwiseConv1D_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                          int batch_size, int input_width, BufferT const &input_buf,
                          BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    DepthwiseConv2D_ReLU(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
                         input_buf, filter_buf, output_buf);
}

template <class BufferT>
void DepthwiseConv1D_Bias_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                               int batch_size, int input_width, BufferT const &input_buf,
                               BufferT const &filter_buf, BufferT const &bias_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    DepthwiseConv2D_Bias_ReLU(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size,
                              input_width, input_buf, filter_buf, bias_buf, output_buf);
}

template <class BufferT>
void GroupConv1D_ReLU(int kernel_width, int stride, int output_groups, uint8_t l_pad, uint8_t r_pad,
                      int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    GroupConv2D_ReLU(1, kernel_width, stride, output_groups, 0, 0, l_pad, r_pad, input_channels, batch_size,
                     input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT>
void GroupConv1D_Bias_ReLU(int kernel_width, int stride, int output_groups, uint8_t l_pad, uint8_t r_pad,
                           int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                           BufferT const &filter_buf, BufferT const &bias_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    GroupConv2D_Bias_ReLU(1, kernel_width, stride, output_groups, 0, 0, l_pad, r_pad, input_channels,
                          batch_size, input_width, input_buf, filter_buf, bias_buf, output_buf);
}

template <class BufferT>
void Conv1D_Maxpool1D(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_Maxpool2D(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv1D_ReLU_Maxpool1D(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_ReLU_Maxpool2D(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv1D_Bias_ReLU_Maxpool1D(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT const &bias_buf, BufferT &inter_output_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_Bias_ReLU_Maxpool2D(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, bias_buf, inter_output_buf, output_buf);
}

template <class BufferT>
void Conv1D_DepthwiseConv1D(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_DepthwiseConv2D(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_ReLU_DepthwiseConv1D_ReLU(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_ReLU_DepthwiseConv2D_ReLU(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_Bias_ReLU_DepthwiseConv1D_Bias_ReLU(SMALL_B200_C1_ARGS, SMALL_B200_P1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT const &bias_buf, BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT const &dwise_bias_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_Bias_ReLU_DepthwiseConv2D_Bias_ReLU(SMALL_B200_C1_PASS, SMALL_B200_P1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, bias_buf, inter_output_buf, dwise_filter_buf, dwise_bias_buf, output_buf);
}

template <class BufferT>
void Conv1D_GroupConv(SMALL_B200_C1_ARGS, SMALL_B200_G1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_GroupConv(SMALL_B200_C1_PASS, SMALL_B200_G1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_ReLU_GroupConv1D_ReLU(SMALL_B200_C1_ARGS, SMALL_B200_G1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_ReLU_GroupConv2D_ReLU(SMALL_B200_C1_PASS, SMALL_B200_G1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, inter_output_buf, dwise_filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_Bias_ReLU_GroupConv1D_Bias_ReLU(SMALL_B200_C1_ARGS, SMALL_B200_G1_ARGS, int output_channels, int input_channels,
        int batch_size, int input_width, BufferT const &input_buf, BufferT const &filter_buf,
        BufferT const &bias_buf, BufferT &inter_output_buf, BufferT const &dwise_filter_buf, BufferT const &dwise_bias_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU(SMALL_B200_C1_PASS, SMALL_B200_G1_PASS, output_channels, input_channels,
        batch_size, input_width, input_buf, filter_buf, bias_buf, inter_output_buf, dwise_filter_buf, dwise_bias_buf, output_buf);
}

#undef SMALL_B200_C1_ARGS
#undef SMALL_B200_P1_ARGS
#undef SMALL_B200_G1_ARGS
#undef SMALL_B200_C1_PASS
#undef SMALL_B200_P1_PASS
#undef SMALL_B200_G1_PASS
} // namespace small
