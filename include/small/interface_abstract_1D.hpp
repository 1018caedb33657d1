// interface_abstract_1D.hpp (B200 platform) -- the 1-D family of the reference
// (include/small/interface_abstract_1D.hpp).  Its layout [C/16][batch][W][16] is the 2-D
// layout with the batch in place of the height (abstract_layer.hpp:1838-1846), so a 1-D
// layer with stride 1 IS the 2-D layer with a window height of 1.  The 2-D kernels apply one
// stride to both axes, hence other strides of the 1-D family are rejected here.
#pragma once

namespace small
{
namespace b200
{
inline void require_unit_stride(int stride, char const *name)
{
    if (stride != 1)
        throw std::invalid_argument(std::string(name) + " ERROR: stride unsupported on the B200 platform.");
}
} // namespace b200

template <class BufferT, bool = true>
void Conv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
            int input_channels, int batch_size, int input_width, BufferT const &input_buf,
            BufferT const &filter_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "Conv1D");
    Conv2D(1, kernel_width, 1, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
           input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void PartialConv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                   int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                   BufferT const &filter_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "PartialConv1D");
    PartialConv2D(1, kernel_width, 1, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
                  input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void MaxPool1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
               int batch_size, int input_width, BufferT const &input_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "MaxPool1D");
    MaxPool2D(1, kernel_width, 1, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
              input_buf, output_buf);
}

template <class BufferT, bool = true>
void AveragePool1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                   int batch_size, int input_width, BufferT const &input_buf, BufferT &output_buf)
{
    b200::require_unit_stride(stride, "AveragePool1D");
    AveragePool2D(1, kernel_width, 1, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
                  input_buf, output_buf);
}

template <class BufferT, bool = true>
void ReLUActivation1D(int input_channels, int batch_size, int input_width,
                      BufferT const &input_buf, BufferT &output_buf)
{
    ReLUActivation(input_channels, batch_size, input_width, input_buf, output_buf);
}

template <class BufferT, bool = true>
void GroupConv1D(int, int, int, uint8_t, uint8_t, int, int, int, BufferT const &, BufferT const &, BufferT &)
{
    throw std::invalid_argument("GroupConv1D ERROR: not provided on the B200 platform.");
}

template <class BufferT, bool = true>
void PartialGroupConv1D(int, int, int, uint8_t, uint8_t, int, int, int, BufferT const &, BufferT const &,
                        BufferT &)
{
    throw std::invalid_argument("PartialGroupConv1D ERROR: not provided on the B200 platform.");
}

template <class BufferT, bool = true>
void UpSample1D(int, int, int, int, BufferT const &, BufferT &)
{
    throw std::invalid_argument("UpSample1D ERROR: not provided on the B200 platform.");
}

} // namespace small
