// stream_f32.cu -- the bandwidth-bound fp32 layers: depthwise convolution, max / average
// pooling, ReLU, LeakyReLU, Accum, Bias, UpSample2D, SoftMax, Concat.
//
// In the reference these are further instantiations of the same loop nest
// (include/small/interface_abstract.hpp:778-2103 -> abstract_layer.hpp:1368) with the
// FLOAT_{DW,MAX,ACCUM,DIV,COND_SCALE,EXP}_TILE_C microkernels
// (platforms/reference/intrinsics_float.h:306-686).  Here every thread owns four adjacent
// channels of one output pixel, so each access is a 128-bit load or store and consecutive
// threads touch consecutive 16-byte pieces of the packed [C/16][H][W][16] layout.
#include "common.cuh"

namespace
{
using namespace sb;

struct WinArgs
{
    int N, C, H, W, Ho, Wo, Fh, Fw, stride, pad_t, pad_l;
    int sh; // stride along the height (`stride` is along the width)
    int accumulate, act;
    float slope;
    float norm;
};

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// decode a flat index over [N][C/16][Ho][Wo][4 quads]
__device__ __forceinline__ bool decode(const WinArgs &a, long long i, int &n, int &cb, int &oh, int &ow, int &q)
{
    const long long total = (long long)a.N * (a.C / CB) * a.Ho * a.Wo * 4;
    if (i >= total)
        return false;
    q = (int)(i & 3); i >>= 2;
    ow = (int)(i % a.Wo); i /= a.Wo;
    oh = (int)(i % a.Ho); i /= a.Ho;
    cb = (int)(i % (a.C / CB));
    n = (int)(i / (a.C / CB));
    return true;
}

// OP: 0 depthwise conv, 1 max pool, 2 average pool
template <int OP>
__global__ void __launch_bounds__(256)
window_f32_kernel(const WinArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                  const float *__restrict__ bias, float *__restrict__ out)
{
    int n, cb, oh, ow, q;
    if (!decode(a, (long long)blockIdx.x * blockDim.x + threadIdx.x, n, cb, oh, ow, q))
        return;
    const float *src = in + (((size_t)n * (a.C / CB) + cb) * a.H * a.W) * CB + q * 4;
    float *dst = out + ((((size_t)n * (a.C / CB) + cb) * a.Ho + oh) * a.Wo + ow) * CB + q * 4;
    const int h0 = oh * a.sh - a.pad_t, w0 = ow * a.stride - a.pad_l;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (OP == 0)
    {
        if (a.accumulate)
            acc = ld4(dst);
        if (bias)
        {
            const float4 b = ld4(bias + cb * CB + q * 4);
            acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
        }
    }
    if (OP == 1)
    {
        // interior windows start from their first tap, border windows from zero
        // (abstract_layer.hpp:515-523 versus :333, :720, :887)
        const bool interior = h0 >= 0 && w0 >= 0 && h0 + a.Fh <= a.H && w0 + a.Fw <= a.W;
        if (interior)
            acc = ld4(src + ((size_t)h0 * a.W + w0) * CB);
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
            const float4 x = ld4(src + ((size_t)ih * a.W + iw) * CB);
            if (OP == 0)
            {
                const float4 f = ld4(filt + (((size_t)cb * a.Fh + kh) * a.Fw + kw) * CB + q * 4);
                acc.x = fmaf(x.x, f.x, acc.x); acc.y = fmaf(x.y, f.y, acc.y);
                acc.z = fmaf(x.z, f.z, acc.z); acc.w = fmaf(x.w, f.w, acc.w);
            }
            else if (OP == 1)
            {
                acc.x = x.x > acc.x ? x.x : acc.x; acc.y = x.y > acc.y ? x.y : acc.y;
                acc.z = x.z > acc.z ? x.z : acc.z; acc.w = x.w > acc.w ? x.w : acc.w;
            }
            else
            {
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
            }
        }
    }
    if (OP == 2)
    {
        acc.x *= a.norm; acc.y *= a.norm; acc.z *= a.norm; acc.w *= a.norm;
    }
    if (OP == 0)
    {
        acc.x = apply_act(acc.x, a.act, a.slope); acc.y = apply_act(acc.y, a.act, a.slope);
        acc.z = apply_act(acc.z, a.act, a.slope); acc.w = apply_act(acc.w, a.act, a.slope);
    }
    st4(dst, acc);
}

// Depthwise 3x3, stride S: a thread owns four channels of FOUR neighbouring output pixels of a row.
// The 3 x (3S + 3) input values it needs are loaded once (18 or 27 loads for four outputs instead of
// 36) and the nine filter vectors once instead of four times; the one-pixel form above is bound by
// its load instructions, not by memory.  Same order of additions (kernel row, then column); a padded
// tap enters as zero.  Flat index over [N][C/16][Ho][strips][4 quads].
template <int S>
__global__ void __launch_bounds__(256)
dwconv3x3_f32_strip_kernel(const WinArgs a, int strips, const float *__restrict__ in, const float *__restrict__ filt,
                           const float *__restrict__ bias, float *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * (a.C / CB) * a.Ho * strips * 4;
    if (i >= total)
        return;
    const int q = (int)(i & 3); i >>= 2;
    const int st = (int)(i % strips); i /= strips;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n * (C/16) + cb
    const int cb = (int)(i % (a.C / CB));
    const float *src = in + (size_t)i * a.H * a.W * CB + q * 4;
    const int ow0 = st * 4;
    float *dst = out + (((size_t)i * a.Ho + oh) * a.Wo + ow0) * CB + q * 4;
    const int h0 = oh * S - a.pad_t, w0 = ow0 * S - a.pad_l;
    constexpr int NC = 3 * S + 3;
    float4 f[9];
#pragma unroll
    for (int t = 0; t < 9; ++t)
        f[t] = __ldg(reinterpret_cast<const float4 *>(filt + ((size_t)cb * 9 + t) * CB + q * 4));
    float4 acc[4];
#pragma unroll
    for (int o = 0; o < 4; ++o)
    {
        acc[o] = (a.accumulate && ow0 + o < a.Wo) ? ld4(dst + o * CB) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias)
        {
            const float4 b = ld4(bias + cb * CB + q * 4);
            acc[o].x += b.x; acc[o].y += b.y; acc[o].z += b.z; acc[o].w += b.w;
        }
    }
#pragma unroll
    for (int kh = 0; kh < 3; ++kh)
    {
        const int ih = h0 + kh;
        if (ih < 0 || ih >= a.H)
            continue;
        float4 x[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j)
        {
            const int iw = w0 + j;
            x[j] = (iw >= 0 && iw < a.W) ? ld4(src + ((size_t)ih * a.W + iw) * CB) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int o = 0; o < 4; ++o)
#pragma unroll
            for (int kw = 0; kw < 3; ++kw)
            {
                const float4 xv = x[o * S + kw], fv = f[kh * 3 + kw];
                acc[o].x = fmaf(xv.x, fv.x, acc[o].x); acc[o].y = fmaf(xv.y, fv.y, acc[o].y);
                acc[o].z = fmaf(xv.z, fv.z, acc[o].z); acc[o].w = fmaf(xv.w, fv.w, acc[o].w);
            }
    }
#pragma unroll
    for (int o = 0; o < 4; ++o)
        if (ow0 + o < a.Wo)
        {
            float4 v = acc[o];
            v.x = apply_act(v.x, a.act, a.slope); v.y = apply_act(v.y, a.act, a.slope);
            v.z = apply_act(v.z, a.act, a.slope); v.w = apply_act(v.w, a.act, a.slope);
            st4(dst + o * CB, v);
        }
}

// OP: 0 ReLU, 1 LeakyReLU, 2 Accum (out += in), 3 scale (out = in * slope).  n4 = number of float4.
template <int OP>
__global__ void __launch_bounds__(256)
eltwise_f32_kernel(long long n4, const float *in, float slope, float *out) // in may alias out
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
    {
        float4 x = ld4(in + i * 4);
        if (OP == 0)
        {
            x.x = x.x > 0.f ? x.x : 0.f; x.y = x.y > 0.f ? x.y : 0.f;
            x.z = x.z > 0.f ? x.z : 0.f; x.w = x.w > 0.f ? x.w : 0.f;
        }
        else if (OP == 1)
        {
            x.x = x.x > 0.f ? x.x : x.x * slope; x.y = x.y > 0.f ? x.y : x.y * slope;
            x.z = x.z > 0.f ? x.z : x.z * slope; x.w = x.w > 0.f ? x.w : x.w * slope;
        }
        else if (OP == 3)
        {
            x.x *= slope; x.y *= slope; x.z *= slope; x.w *= slope;
        }
        else
        {
            const float4 o = ld4(out + i * 4);
            x.x = o.x + x.x; x.y = o.y + x.y; x.z = o.z + x.z; x.w = o.w + x.w;
        }
        st4(out + i * 4, x);
    }
}

__global__ void __launch_bounds__(256)
bias_f32_kernel(int N, int C, long long hw, const float *__restrict__ bias, int accumulate, float *out)
{
    const long long total = (long long)N * (C / CB) * hw * 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    const int q = (int)(i & 3);
    const int cb = (int)((i >> 2) / hw % (C / CB));
    float4 b = ld4(bias + cb * CB + q * 4);
    if (accumulate)
    {
        const float4 o = ld4(out + i * 4);
        b.x = o.x + b.x; b.y = o.y + b.y; b.z = o.z + b.z; b.w = o.w + b.w;
    }
    st4(out + i * 4, b);
}

__global__ void __launch_bounds__(256)
upsample2_f32_kernel(int N, int C, int H, int W, int sh, const float *__restrict__ in, float *__restrict__ out)
{
    const int Ho = sh * H, Wo = 2 * W; // sh = 1: the 1-D form, rows are batch entries
    const long long total = (long long)N * (C / CB) * Ho * Wo * 4;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    const long long o = i;
    const int q = (int)(i & 3); i >>= 2;
    const int ow = (int)(i % Wo); i /= Wo;
    const int oh = (int)(i % Ho); i /= Ho; // i = n*(C/16)+cb
    st4(out + o * 4, ld4(in + ((i * H + oh / sh) * W + ow / 2) * CB + q * 4));
}

// One CTA per image: exp pass with the sum kept in registers, block reduction with warp
// shuffles, scale pass.  The reference makes the same three passes
// (interface_abstract.hpp:1790-1830) without subtracting the maximum.
__global__ void __launch_bounds__(1024)
softmax_f32_kernel(long long elems, const float *in, float *out) // in may alias out
{
    __shared__ float warp_sums[32];
    __shared__ float total;
    const float *x = in + (size_t)blockIdx.x * elems;
    float *y = out + (size_t)blockIdx.x * elems;
    float s = 0.f;
    for (long long i = threadIdx.x; i < elems; i += blockDim.x)
    {
        const float e = expf(x[i]);
        y[i] = e;
        s += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0)
        warp_sums[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32)
    {
        float t = (threadIdx.x < (blockDim.x + 31) / 32) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0)
            total = t;
    }
    __syncthreads();
    const float inv = (float)(1.0 / (double)total);
    for (long long i = threadIdx.x; i < elems; i += blockDim.x)
        y[i] = y[i] * inv;
}

__global__ void __launch_bounds__(256)
concat_kernel(int N, long long v0, const uint4 *__restrict__ in0, long long v1,
              const uint4 *__restrict__ in1, uint4 *__restrict__ out)
{
    const long long per = v0 + v1, total = per * N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        const long long n = i / per, r = i - n * per;
        out[i] = (r < v0) ? in0[n * v0 + r] : in1[n * v1 + (r - v0)];
    }
}

int fill(const small_b200_layer *L, WinArgs &a)
{
    a.N = L->N; a.C = L->C; a.H = L->H; a.W = L->W; a.Fh = L->Fh; a.Fw = L->Fw;
    a.stride = L->stride; a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.sh = row_stride(L);
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, a.sh);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    a.accumulate = L->accumulate; a.act = L->act; a.slope = L->slope;
    a.norm = (float)(1.0 / (1.0 * L->Fh * L->Fw)); // abstract_layer.hpp:565-569
    return 0;
}

inline unsigned blocks_for(long long items, int threads = 256)
{
    return (unsigned)((items + threads - 1) / threads);
}

inline unsigned grid_stride_blocks(long long items)
{
    const long long want = (items + 255) / 256;
    const long long cap = (long long)num_sms() * 16;
    return (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
}
} // namespace

extern "C"
{
int small_b200_dwconv2d_f32(const small_b200_layer *L, const float *in, const float *filt,
                            const float *bias, float *out, void *stream)
{
    if (int rc = check_window_layer(L, "DepthwiseConv2D<float>", false, 2))
        return rc;
    WinArgs a; fill(L, a);
    const long long items = (long long)a.N * (a.C / CB) * a.Ho * a.Wo * 4;
    if (items == 0)
        return SMALL_B200_OK;
    if (a.Fh == 3 && a.Fw == 3 && a.Wo >= 4 && a.sh == a.stride)
    {
        const int strips = (a.Wo + 3) / 4;
        const long long threads = (long long)a.N * (a.C / CB) * a.Ho * strips * 4;
        if (a.stride == 1)
            dwconv3x3_f32_strip_kernel<1><<<blocks_for(threads), 256, 0, as_stream(stream)>>>(a, strips, in, filt, bias, out);
        else
            dwconv3x3_f32_strip_kernel<2><<<blocks_for(threads), 256, 0, as_stream(stream)>>>(a, strips, in, filt, bias, out);
        return launched("dwconv3x3_f32_strip_kernel");
    }
    window_f32_kernel<0><<<blocks_for(items), 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("dwconv2d_f32");
}

int small_b200_maxpool2d_f32(const small_b200_layer *L, const float *in, float *out, void *stream)
{
    if (int rc = check_window_layer(L, "MaxPool2D<float>", false, 2))
        return rc;
    WinArgs a; fill(L, a);
    const long long items = (long long)a.N * (a.C / CB) * a.Ho * a.Wo * 4;
    if (items == 0)
        return SMALL_B200_OK;
    window_f32_kernel<1><<<blocks_for(items), 256, 0, as_stream(stream)>>>(a, in, nullptr, nullptr, out);
    return launched("maxpool2d_f32");
}

int small_b200_avgpool2d_f32(const small_b200_layer *L, const float *in, float *out, void *stream)
{
    if (int rc = check_window_layer(L, "AveragePool2D<float>", false, 3))
        return rc;
    WinArgs a; fill(L, a);
    const long long items = (long long)a.N * (a.C / CB) * a.Ho * a.Wo * 4;
    if (items == 0)
        return SMALL_B200_OK;
    window_f32_kernel<2><<<blocks_for(items), 256, 0, as_stream(stream)>>>(a, in, nullptr, nullptr, out);
    return launched("avgpool2d_f32");
}

static int check_n(int64_t n, const char *name)
{
    if (n < 0 || n % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: in_channels unsupported.");
    return SMALL_B200_OK;
}

int small_b200_relu_f32(int64_t n, const float *in, float *out, void *stream)
{
    if (int rc = check_n(n, "ReLUActivation<float>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    eltwise_f32_kernel<0><<<grid_stride_blocks(n / 4), 256, 0, as_stream(stream)>>>(n / 4, in, 0.f, out);
    return launched("relu_f32");
}

int small_b200_leaky_relu_f32(int64_t n, const float *in, float slope, float *out, void *stream)
{
    if (int rc = check_n(n, "LeakyReLUActivation<float>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    eltwise_f32_kernel<1><<<grid_stride_blocks(n / 4), 256, 0, as_stream(stream)>>>(n / 4, in, slope, out);
    return launched("leaky_relu_f32");
}

int small_b200_scale_f32(int64_t n, const float *in, float scale, float *out, void *stream)
{
    if (int rc = check_n(n, "Dropout<float>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    eltwise_f32_kernel<3><<<grid_stride_blocks(n / 4), 256, 0, as_stream(stream)>>>(n / 4, in, scale, out);
    return launched("scale_f32");
}

int small_b200_accum_f32(int64_t n, const float *in, float *out, void *stream)
{
    if (int rc = check_n(n, "Accum<float>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    eltwise_f32_kernel<2><<<grid_stride_blocks(n / 4), 256, 0, as_stream(stream)>>>(n / 4, in, 0.f, out);
    return launched("accum_f32");
}

int small_b200_bias_f32(int32_t N, int32_t C, int32_t H, int32_t W, const float *bias,
                        int32_t accumulate, float *out, void *stream)
{
    if (C <= 0 || C % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Bias<float> ERROR: in_channels unsupported.");
    const long long items = (long long)N * (C / CB) * H * W * 4;
    if (items <= 0)
        return SMALL_B200_OK;
    bias_f32_kernel<<<blocks_for(items), 256, 0, as_stream(stream)>>>(N, C, (long long)H * W, bias, accumulate, out);
    return launched("bias_f32");
}

int small_b200_upsample2d_f32(int32_t N, int32_t C, int32_t H, int32_t W, const float *in,
                              float *out, void *stream)
{
    if (C <= 0 || C % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Upsample<float> ERROR: in_channels unsupported.");
    const long long items = (long long)N * (C / CB) * H * W * 16;
    if (items <= 0)
        return SMALL_B200_OK;
    upsample2_f32_kernel<<<blocks_for(items), 256, 0, as_stream(stream)>>>(N, C, H, W, 2, in, out);
    return launched("upsample2d_f32");
}

int small_b200_upsample1d_f32(int32_t N, int32_t C, int32_t rows, int32_t W, const float *in, float *out, void *stream)
{
    if (C <= 0 || C % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Upsample<float> ERROR: in_channels unsupported.");
    const long long items = (long long)N * (C / CB) * rows * W * 8;
    if (items <= 0)
        return SMALL_B200_OK;
    upsample2_f32_kernel<<<blocks_for(items), 256, 0, as_stream(stream)>>>(N, C, rows, W, 1, in, out);
    return launched("upsample1d_f32");
}

int small_b200_softmax_f32(int32_t N, int64_t elems_per_image, const float *in, float *out, void *stream)
{
    if (N <= 0 || elems_per_image <= 0)
        return SMALL_B200_OK;
    const int threads = elems_per_image >= 1024 ? 1024 : (int)((elems_per_image + 31) / 32 * 32);
    softmax_f32_kernel<<<N, threads, 0, as_stream(stream)>>>(elems_per_image, in, out);
    return launched("softmax_f32");
}

int small_b200_concat(int32_t N, size_t bytes0, const void *in0, size_t bytes1, const void *in1,
                      void *out, void *stream)
{
    if (bytes0 % 16 || bytes1 % 16)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Concat ERROR: sizes must be multiples of 16 bytes.");
    const long long v0 = bytes0 / 16, v1 = bytes1 / 16;
    if (N <= 0 || v0 + v1 == 0)
        return SMALL_B200_OK;
    concat_kernel<<<grid_stride_blocks((v0 + v1) * N), 256, 0, as_stream(stream)>>>(
        N, v0, (const uint4 *)in0, v1, (const uint4 *)in1, (uint4 *)out);
    return launched("concat");
}
} // extern "C"
