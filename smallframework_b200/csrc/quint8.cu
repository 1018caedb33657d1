// quint8.cu -- the uint8 layers on the CUDA cores: dense convolution (general shapes),
// depthwise convolution, max / average pooling and ReLU, each followed by the
// reference's fixed-point requantisation.  Replaces
// small::quint8_detail::abstract_layer (include/small/q_abstract_layer.hpp:884-1571) and the
// QUINT8_{CONV,DW,MAX}_TILE_C / QUINT8_QUANTIZE_TILE_C microkernels
// (platforms/reference/intrinsics_quint8.h:191-289, :481-531).
//
// Arithmetic (bit-exact with the reference): zero points are ADDED, padded taps are
// SKIPPED (they contribute nothing, not even zero_in * w), accumulation is int32 and stays
// in registers for the whole reduction -- the reference parks partial sums in the output
// buffer between input-channel blocks (q_abstract_layer.hpp:1144), which is why its
// callers over-allocate outputs four times; nothing of that is needed here.
#include "common.cuh"

namespace
{
using namespace sb;

struct QArgs
{
    int N, C, K, H, W, Ho, Wo, Fh, Fw, stride, pad_t, pad_l;
    int cib, cbs;
    int zero_in, zero_filt, lshift, rshift, mult, k_zero;
};

__device__ __forceinline__ int byte_of(const uint4 &v, int i)
{
    const unsigned w = (i < 4) ? v.x : (i < 8) ? v.y : (i < 12) ? v.z : v.w;
    return (int)((w >> (8 * (i & 3))) & 0xffu);
}

__device__ __forceinline__ uint4 pack16(const int *v)
{
    uint4 o;
    o.x = (unsigned)v[0] | ((unsigned)v[1] << 8) | ((unsigned)v[2] << 16) | ((unsigned)v[3] << 24);
    o.y = (unsigned)v[4] | ((unsigned)v[5] << 8) | ((unsigned)v[6] << 16) | ((unsigned)v[7] << 24);
    o.z = (unsigned)v[8] | ((unsigned)v[9] << 8) | ((unsigned)v[10] << 16) | ((unsigned)v[11] << 24);
    o.w = (unsigned)v[12] | ((unsigned)v[13] << 8) | ((unsigned)v[14] << 16) | ((unsigned)v[15] << 24);
    return o;
}

// Dense convolution, one thread per output pixel and block of 16 output channels.
// All threads of a CTA share the output-channel block, so filter reads are warp-uniform
// 16-byte loads served by L1.
__global__ void __launch_bounds__(128)
conv2d_u8_direct_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                        const int32_t *__restrict__ bias, uint8_t *__restrict__ out)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    const int kb = blockIdx.y, n = blockIdx.z;
    if (p >= a.Ho * a.Wo)
        return;
    const int oh = p / a.Wo, ow = p - oh * a.Wo;
    int acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = a.k_zero + (bias ? bias[kb * CB + k] : 0);
    const int taps = a.Fh * a.Fw;
    const uint8_t *img = in + (size_t)n * a.C * a.H * a.W;
    const uint8_t *fk = filt + (size_t)kb * a.cbs * taps * a.cib * CB;
    for (int cb = 0; cb < a.cbs; ++cb)
    {
        const uint8_t *plane = img + (size_t)cb * a.H * a.W * a.cib;
        const uint8_t *fcb = fk + (size_t)cb * taps * a.cib * CB;
        for (int kh = 0; kh < a.Fh; ++kh)
        {
            const int ih = oh * a.stride - a.pad_t + kh;
            if (ih < 0 || ih >= a.H)
                continue;
            for (int kw = 0; kw < a.Fw; ++kw)
            {
                const int iw = ow * a.stride - a.pad_l + kw;
                if (iw < 0 || iw >= a.W)
                    continue;
                const uint8_t *px = plane + ((size_t)ih * a.W + iw) * a.cib;
                const uint4 *fw = reinterpret_cast<const uint4 *>(fcb + (size_t)(kh * a.Fw + kw) * a.cib * CB);
                if (a.cib == CB)
                {
                    const uint4 av = *reinterpret_cast<const uint4 *>(px);
#pragma unroll
                    for (int c = 0; c < CB; ++c)
                    {
                        const int x = byte_of(av, c) + a.zero_in;
                        const uint4 wv = __ldg(fw + c);
#pragma unroll
                        for (int k = 0; k < CB; ++k)
                            acc[k] += x * (byte_of(wv, k) + a.zero_filt);
                    }
                }
                else
                {
                    for (int c = 0; c < a.cib; ++c)
                    {
                        const int x = (int)px[c] + a.zero_in;
                        const uint4 wv = __ldg(fw + c);
#pragma unroll
                        for (int k = 0; k < CB; ++k)
                            acc[k] += x * (byte_of(wv, k) + a.zero_filt);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = requant(acc[k], a.lshift, a.rshift, a.mult);
    *reinterpret_cast<uint4 *>(out + (((size_t)n * (a.K / CB) + kb) * a.Ho * a.Wo + p) * CB) = pack16(acc);
}

// OP: 0 depthwise conv, 1 max pool, 2 average pool; one thread per output pixel and block
// of 16 channels (one 128-bit load per tap, one 128-bit store).
template <int OP>
__global__ void __launch_bounds__(256)
window_u8_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                 const int32_t *__restrict__ bias, uint8_t *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * (a.C / CB) * a.Ho * a.Wo;
    if (i >= total)
        return;
    const long long o = i;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n*(C/16)+cb
    const int cb = (int)(i % (a.C / CB));
    const uint8_t *plane = in + (size_t)i * a.H * a.W * CB;
    const int h0 = oh * a.stride - a.pad_t, w0 = ow * a.stride - a.pad_l;
    int acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = a.k_zero + ((OP == 0 && bias) ? bias[cb * CB + k] : 0);
    if (OP == 1)
    {
        // q_abstract_layer.hpp:277-288: interior tiles are seeded with the RAW first tap
        const bool interior = h0 >= 0 && w0 >= 0 && h0 + a.Fh <= a.H && w0 + a.Fw <= a.W;
        if (interior)
        {
            const uint4 v = *reinterpret_cast<const uint4 *>(plane + ((size_t)h0 * a.W + w0) * CB);
#pragma unroll
            for (int k = 0; k < CB; ++k)
                acc[k] = byte_of(v, k);
        }
    }
    for (int kh = 0; kh < a.Fh; ++kh)
    {
        const int ih = h0 + kh;
        if (ih < 0 || ih >= a.H)
            continue;
        for (int kw = 0; kw < a.Fw; ++kw)
        {
            const int iw = w0 + kw;
            if (iw < 0 || iw >= a.W)
                continue;
            const uint4 v = *reinterpret_cast<const uint4 *>(plane + ((size_t)ih * a.W + iw) * CB);
            if (OP == 0)
            {
                const uint4 f = __ldg(reinterpret_cast<const uint4 *>(
                    filt + (((size_t)cb * a.Fh + kh) * a.Fw + kw) * CB));
#pragma unroll
                for (int k = 0; k < CB; ++k)
                    acc[k] += (byte_of(v, k) + a.zero_in) * (byte_of(f, k) + a.zero_filt);
            }
            else if (OP == 1)
            {
#pragma unroll
                for (int k = 0; k < CB; ++k)
                {
                    const int x = byte_of(v, k) + a.zero_in;
                    acc[k] = x > acc[k] ? x : acc[k];
                }
            }
            else
            {
#pragma unroll
                for (int k = 0; k < CB; ++k)
                    acc[k] += byte_of(v, k) + a.zero_in;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = requant(acc[k], a.lshift, a.rshift, a.mult);
    *reinterpret_cast<uint4 *>(out + o * CB) = pack16(acc);
}

__global__ void __launch_bounds__(256)
relu_u8_kernel(long long n16, const QArgs a, const uint8_t *in, uint8_t *out) // in may alias out
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride)
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(in + i * 16);
        int r[CB];
#pragma unroll
        for (int k = 0; k < CB; ++k)
        {
            const int x = byte_of(v, k) + a.zero_in;
            r[k] = requant(x > a.k_zero ? x : a.k_zero, a.lshift, a.rshift, a.mult);
        }
        *reinterpret_cast<uint4 *>(out + i * 16) = pack16(r);
    }
}

void fill(const small_b200_layer *L, QArgs &a, bool dense)
{
    a.N = L->N; a.C = L->C; a.K = dense ? L->K : L->C; a.H = L->H; a.W = L->W;
    a.Fh = L->Fh; a.Fw = L->Fw; a.stride = L->stride; a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, L->stride);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    a.cib = dense ? eff_block(L->C) : CB;
    a.cbs = L->C / a.cib;
    a.zero_in = L->zero_in; a.zero_filt = L->zero_filt; a.lshift = L->lshift;
    a.rshift = L->rshift; a.mult = L->multiplier; a.k_zero = L->k_zero;
}

int check_quant(const small_b200_layer *L, const char *name)
{
    if (L->lshift < 0 || L->lshift > 31 || L->rshift < 0 || L->rshift > 31)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: shift out of range.");
    return SMALL_B200_OK;
}

template <int OP>
int launch_window(const small_b200_layer *L, const char *name, int max_stride, const uint8_t *in,
                  const uint8_t *filt, const int32_t *bias, uint8_t *out, void *stream)
{
    if (int rc = check_window_layer(L, name, false, max_stride))
        return rc;
    if (int rc = check_quant(L, name))
        return rc;
    QArgs a; fill(L, a, false);
    const long long items = (long long)a.N * (a.C / CB) * a.Ho * a.Wo;
    if (items == 0)
        return SMALL_B200_OK;
    window_u8_kernel<OP><<<(unsigned)((items + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched(name);
}
} // namespace

namespace sb
{
// Defined in conv_u8_tc.cu: the tensor-core path for shapes it supports.  Returns -1 when
// the shape is not covered, otherwise a SMALL_B200_* code.
int conv2d_u8_tensor_core(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                          const int32_t *bias, uint8_t *out, cudaStream_t st);
}

extern "C"
{
int small_b200_conv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                         const int32_t *bias, uint8_t *out, void *stream)
{
    if (int rc = check_window_layer(L, "Conv2D<quint8>", true, 2))
        return rc;
    if (int rc = check_quant(L, "Conv2D<quint8>"))
        return rc;
    if (L->accumulate)
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "PartialConv2D<quint8> ERROR: the int32 partial-sum form is not provided.");
    const int tc = conv2d_u8_tensor_core(L, in, filt, bias, out, as_stream(stream));
    if (tc >= 0)
        return tc;
    QArgs a; fill(L, a, true);
    if (a.N == 0 || a.Ho == 0 || a.Wo == 0)
        return SMALL_B200_OK;
    dim3 grid((a.Ho * a.Wo + 127) / 128, a.K / CB, a.N);
    conv2d_u8_direct_kernel<<<grid, 128, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("conv2d_u8_direct_kernel");
}

int small_b200_dwconv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                           const int32_t *bias, uint8_t *out, void *stream)
{
    return launch_window<0>(L, "DepthwiseConv2D<quint8>", 2, in, filt, bias, out, stream);
}

int small_b200_maxpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    return launch_window<1>(L, "MaxPool2D<quint8>", 2, in, nullptr, nullptr, out, stream);
}

int small_b200_avgpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    return launch_window<2>(L, "AveragePool2D<quint8>", 3, in, nullptr, nullptr, out, stream);
}

int small_b200_relu_u8(int64_t n, const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    if (n < 0 || n % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "ReLUActivation<quint8> ERROR: in_channels unsupported.");
    if (int rc = check_quant(L, "ReLUActivation<quint8>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    QArgs a{};
    a.zero_in = L->zero_in; a.lshift = L->lshift; a.rshift = L->rshift; a.mult = L->multiplier;
    a.k_zero = L->k_zero;
    const long long n16 = n / 16;
    long long blocks = (n16 + 255) / 256;
    const long long cap = (long long)num_sms() * 16;
    if (blocks > cap)
        blocks = cap;
    relu_u8_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(n16, a, in, out);
    return launched("relu_u8");
}
} // extern "C"
