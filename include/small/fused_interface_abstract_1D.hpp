// fused_interface_abstract_1D.hpp (B200 platform) -- fused 1-D forms that map onto the
// fused 2-D kernels with a window height of 1 (stride 1 only, see
// interface_abstract_1D.hpp of this platform).
#pragma once

namespace small
{
template <class BufferT>
void Conv1D_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                 int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                 BufferT const &filter_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "Conv1D_ReLU");
    Conv2D_ReLU(1, kernel_width, 1, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
                input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT>
void Conv1D_Bias_ReLU(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                      int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                      BufferT const &filter_buf, BufferT const &bias_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "Conv1D_Bias_ReLU");
    Conv2D_Bias_ReLU(1, kernel_width, 1, 0, 0, l_pad, r_pad, output_channels, input_channels,
                     batch_size, input_width, input_buf, filter_buf, bias_buf, output_buf);
}
} // namespace small
