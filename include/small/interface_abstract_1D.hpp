// interface_abstract_1D.hpp (B200 platform) -- the 1-D family of the reference
// (include/small/interface_abstract_1D.hpp).  Its layout [C/16][batch][W][16] is the 2-D
// layout with the batch in place of the height (abstract_layer.hpp:1838-1846): a 1-D layer is the
// 2-D layer with a window height of 1 whose rows (the batch entries) are all kept, i.e. with a
// stride of 1 along the height whatever the stride along the width is.  The wrappers below open
// a RowStrideScope(1) and call the 2-D function.
#pragma once

namespace small
{
template <class BufferT, bool = true>
void Conv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
            int input_channels, int batch_size, int input_width, BufferT const &input_buf,
            BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    Conv2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
           input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void PartialConv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int output_channels,
                   int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                   BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    PartialConv2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, output_channels, input_channels, batch_size,
                  input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void MaxPool1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
               int batch_size, int input_width, BufferT const &input_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    MaxPool2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
              input_buf, output_buf);
}

template <class BufferT, bool = true>
void AveragePool1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                   int batch_size, int input_width, BufferT const &input_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    AveragePool2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
                  input_buf, output_buf);
}

template <class BufferT, bool = true>
void DepthwiseConv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                     int batch_size, int input_width, BufferT const &input_buf,
                     BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    DepthwiseConv2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size, input_width,
                    input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void PartialDepthwiseConv1D(int kernel_width, int stride, uint8_t l_pad, uint8_t r_pad, int input_channels,
                            int batch_size, int input_width, BufferT const &input_buf,
                            BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    PartialDepthwiseConv2D(1, kernel_width, stride, 0, 0, l_pad, r_pad, input_channels, batch_size,
                           input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void ReLUActivation1D(int input_channels, int batch_size, int input_width,
                      BufferT const &input_buf, BufferT &output_buf)
{
    ReLUActivation(input_channels, batch_size, input_width, input_buf, output_buf);
}

template <class BufferT, bool = true>
void GroupConv1D(int kernel_width, int stride, int output_groups, uint8_t l_pad, uint8_t r_pad,
                 int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                 BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    GroupConv2D(1, kernel_width, stride, output_groups, 0, 0, l_pad, r_pad, input_channels, batch_size,
                input_width, input_buf, filter_buf, output_buf);
}

template <class BufferT, bool = true>
void PartialGroupConv1D(int kernel_width, int stride, int output_groups, uint8_t l_pad, uint8_t r_pad,
                        int input_channels, int batch_size, int input_width, BufferT const &input_buf,
                        BufferT const &filter_buf, BufferT &output_buf)
{
    b200::RowStrideScope rows(1);
    PartialGroupConv2D(1, kernel_width, stride, output_groups, 0, 0, l_pad, r_pad, input_channels,
                       batch_size, input_width, input_buf, filter_buf, output_buf);
}

// interface_abstract_1D.hpp:1614 of the reference: scale 1 copies, scale 2 repeats every element of a
// row once, other factors throw.
template <class BufferT, bool = true>
void UpSample1D(int scale_factor, int input_channels, int batch_size, int input_width,
                BufferT const &input_buf, BufferT &output_buf)
{
    if (scale_factor == 1)
    {
        output_buf = input_buf;
        return;
    }
    if (scale_factor != 2)
        throw std::invalid_argument("Upsample<float> ERROR: scale factor unsupported (only 1 or 2).");
    if constexpr (b200::is_quint8<BufferT>)
        throw std::invalid_argument("Upsample<quint8> ERROR: not provided.");
    else
    {
        b200::require_block(input_channels, SMALL_B200_CB, "Upsample<float> ERROR: in_channels unsupported.");
        b200::throw_on(small_b200_upsample1d_f32(b200::batch(), input_channels, batch_size, input_width,
                                                 input_buf.device_ptr(), output_buf.device_ptr(), b200::stream()));
    }
}

} // namespace small
