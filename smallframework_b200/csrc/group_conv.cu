// group_conv.cu -- grouped convolution, fp32 and uint8.
//
// Replaces small::GroupConv2D / PartialGroupConv2D (include/small/interface_abstract.hpp:1265,
// :1332, :1402, :1470), i.e. the loop nest instantiated with G_b = C_ob, K_b = F_cb = 1
// (include/small/abstract_layer.hpp:1419-1432):
//     in   [N][G/16][C][H][W][16 g]
//     filt    [G/16][K][C][Fh][Fw][16 g]
//     out  [N][G/16][K][Ho][Wo][16 g]
// G groups, each an independent convolution from C input channels to K output channels (the
// reference's interface passes input_channels for both); the 16 lanes of a block are 16
// different groups, so a tap is a lane-wise multiply-add, exactly as in the depthwise layers.
// The reduction runs input channel by input channel, kernel row by kernel row, and padded taps
// are skipped -- the order of the reference's nest.
//
// These layers move little data per flop of reuse (every output channel of a group re-reads the
// group's input), so a thread keeps KT output channels of one pixel in registers and reads each
// input value once for all of them; consecutive threads touch consecutive 16-byte pieces.
#include "common.cuh"

namespace
{
using namespace sb;

struct GArgs
{
    int N, G, C, K, H, W, Ho, Wo, Fh, Fw, stride, sh, pad_t, pad_l; // sh: stride along the height
    int accumulate, act;
    float slope;
    int zero_in, zero_filt, lshift, rshift, mult, k_zero;
};

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// fp32: thread = 4 group lanes x KT output channels of one output pixel.
// flat index over [N][G/16][K/KT][Ho][Wo][4 quads]
template <int KT>
__global__ void __launch_bounds__(256)
groupconv2d_f32_kernel(const GArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                       const float *__restrict__ bias, float *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int kts = a.K / KT;
    const long long total = (long long)a.N * (a.G / CB) * kts * a.Ho * a.Wo * 4;
    if (i >= total)
        return;
    const int q = (int)(i & 3); i >>= 2;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho;
    const int kt = (int)(i % kts); i /= kts;
    const int gb = (int)(i % (a.G / CB));
    const int n = (int)(i / (a.G / CB));
    const int k0 = kt * KT;
    const size_t plane = (size_t)a.H * a.W * CB;
    const float *src = in + ((size_t)n * (a.G / CB) + gb) * a.C * plane + q * 4;
    const size_t fstride_k = (size_t)a.C * a.Fh * a.Fw * CB;
    const float *fk = filt + ((size_t)gb * a.K + k0) * fstride_k + q * 4;
    const size_t oplane = (size_t)a.Ho * a.Wo * CB;
    float *dst = out + (((size_t)n * (a.G / CB) + gb) * a.K + k0) * oplane + ((size_t)oh * a.Wo + ow) * CB + q * 4;
    const int h0 = oh * a.sh - a.pad_t, w0 = ow * a.stride - a.pad_l;
    float4 acc[KT];
#pragma unroll
    for (int j = 0; j < KT; ++j)
    {
        acc[j] = a.accumulate ? ld4(dst + j * oplane) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias)
        {
            const float4 b = ld4(bias + ((size_t)gb * a.K + k0 + j) * CB + q * 4);
            acc[j].x += b.x; acc[j].y += b.y; acc[j].z += b.z; acc[j].w += b.w;
        }
    }
    for (int c = 0; c < a.C; ++c)
    {
        const float *pc = src + c * plane;
        const float *fc = fk + (size_t)c * a.Fh * a.Fw * CB;
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
                const float4 x = ld4(pc + ((size_t)ih * a.W + iw) * CB);
                const float *ft = fc + (size_t)(kh * a.Fw + kw) * CB;
#pragma unroll
                for (int j = 0; j < KT; ++j)
                {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(ft + j * fstride_k));
                    acc[j].x = fmaf(x.x, f.x, acc[j].x); acc[j].y = fmaf(x.y, f.y, acc[j].y);
                    acc[j].z = fmaf(x.z, f.z, acc[j].z); acc[j].w = fmaf(x.w, f.w, acc[j].w);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < KT; ++j)
    {
        float4 v = acc[j];
        v.x = apply_act(v.x, a.act, a.slope); v.y = apply_act(v.y, a.act, a.slope);
        v.z = apply_act(v.z, a.act, a.slope); v.w = apply_act(v.w, a.act, a.slope);
        *reinterpret_cast<float4 *>(dst + j * oplane) = v;
    }
}

__device__ __forceinline__ int gbyte(const uint4 &v, int i)
{
    const unsigned w = (i < 4) ? v.x : (i < 8) ? v.y : (i < 12) ? v.z : v.w;
    return (int)((w >> (8 * (i & 3))) & 0xffu);
}

// uint8: thread = the 16 group lanes of one output pixel and one output channel; one 128-bit
// load per tap for the activations and one (the same for every pixel of the CTA's channel,
// served by L1) for the weights.  flat index over [N][G/16][K][Ho][Wo].
__global__ void __launch_bounds__(256)
groupconv2d_u8_kernel(const GArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                      const int32_t *__restrict__ bias, uint8_t *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * (a.G / CB) * a.K * a.Ho * a.Wo;
    if (i >= total)
        return;
    const long long o = i;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho;
    const int k = (int)(i % a.K); i /= a.K; // i = n * (G/16) + gb
    const int gb = (int)(i % (a.G / CB));
    const size_t plane = (size_t)a.H * a.W * CB;
    const uint8_t *src = in + (size_t)i * a.C * plane;
    const uint8_t *fk = filt + ((size_t)gb * a.K + k) * a.C * a.Fh * a.Fw * CB;
    const int h0 = oh * a.sh - a.pad_t, w0 = ow * a.stride - a.pad_l;
    int acc[CB];
#pragma unroll
    for (int g = 0; g < CB; ++g)
        acc[g] = a.k_zero + (bias ? bias[((size_t)gb * a.K + k) * CB + g] : 0);
    for (int c = 0; c < a.C; ++c)
    {
        const uint8_t *pc = src + c * plane;
        const uint8_t *fc = fk + (size_t)c * a.Fh * a.Fw * CB;
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
                const uint4 v = *reinterpret_cast<const uint4 *>(pc + ((size_t)ih * a.W + iw) * CB);
                const uint4 f = __ldg(reinterpret_cast<const uint4 *>(fc + (size_t)(kh * a.Fw + kw) * CB));
#pragma unroll
                for (int g = 0; g < CB; ++g)
                    acc[g] += (gbyte(v, g) + a.zero_in) * (gbyte(f, g) + a.zero_filt);
            }
        }
    }
    *reinterpret_cast<uint4 *>(out + o * CB) = requant_pack16(acc, a.lshift, a.rshift, a.mult);
}

// Block-diagonal convolution: `groups` independent dense convolutions from 16 to 16 channels, group g
// on channel block g -- the second stage of the reference's fused grouped forms
// (fused_interface_abstract.hpp:2740-2760: G = output_groups, K = C_ob, F_c = C_ib):
//     in [N][G][H][W][16 c]   filt [G][Fh][Fw][16 c][16 k]   out [N][G][Ho][Wo][16 k]
// thread = four output channels of one output pixel of one group; flat index over [N][G][Ho][Wo][4].
__global__ void __launch_bounds__(256)
blockconv2d_f32_kernel(const GArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                       const float *__restrict__ bias, float *__restrict__ out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * a.G * a.Ho * a.Wo * 4;
    if (i >= total)
        return;
    const long long o = i;
    const int q = (int)(i & 3); i >>= 2;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n * G + g
    const int g = (int)(i % a.G);
    const float *src = in + (size_t)i * a.H * a.W * CB;
    const float *fg = filt + (size_t)g * a.Fh * a.Fw * CB * CB + q * 4;
    float *dst = out + o * 4;
    float4 acc = a.accumulate ? ld4(dst) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias)
    {
        const float4 b = ld4(bias + (size_t)g * CB + q * 4);
        acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    const int h0 = oh * a.sh - a.pad_t, w0 = ow * a.stride - a.pad_l;
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
            const float *px = src + ((size_t)ih * a.W + iw) * CB;
            const float *ft = fg + (size_t)(kh * a.Fw + kw) * CB * CB;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
            {
                const float4 x = ld4(px + c4 * 4);
                const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(ft + (c4 * 4 + j) * CB));
                    acc.x = fmaf(xs[j], f.x, acc.x); acc.y = fmaf(xs[j], f.y, acc.y);
                    acc.z = fmaf(xs[j], f.z, acc.z); acc.w = fmaf(xs[j], f.w, acc.w);
                }
            }
        }
    }
    acc.x = apply_act(acc.x, a.act, a.slope); acc.y = apply_act(acc.y, a.act, a.slope);
    acc.z = apply_act(acc.z, a.act, a.slope); acc.w = apply_act(acc.w, a.act, a.slope);
    *reinterpret_cast<float4 *>(dst) = acc;
}

int check_group(const small_b200_layer *L, int groups, const char *name, GArgs &a)
{
    if (!L)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: null layer.");
    if ((L->stride != 1 && L->stride != 2) || L->stride_h < 0 || L->stride_h > 2)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: stride unsupported.");
    if (L->C <= 0 || L->K <= 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: in_channels unsupported.");
    if (groups <= 0 || groups % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: output_groups unsupported.");
    if (L->N < 0 || L->H <= 0 || L->W <= 0 || L->Fh <= 0 || L->Fw <= 0 || L->pad_t < 0 ||
        L->pad_b < 0 || L->pad_l < 0 || L->pad_r < 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: bad shape.");
    a.N = L->N; a.G = groups; a.C = L->C; a.K = L->K; a.H = L->H; a.W = L->W; a.Fh = L->Fh; a.Fw = L->Fw;
    a.stride = L->stride; a.sh = row_stride(L); a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, a.sh);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    a.accumulate = L->accumulate; a.act = L->act; a.slope = L->slope;
    a.zero_in = L->zero_in; a.zero_filt = L->zero_filt; a.lshift = L->lshift; a.rshift = L->rshift;
    a.mult = L->multiplier; a.k_zero = L->k_zero;
    return SMALL_B200_OK;
}
} // namespace

extern "C"
{
int small_b200_groupconv2d_f32(const small_b200_layer *L, int32_t groups, const float *in, const float *filt,
                               const float *bias, float *out, void *stream)
{
    GArgs a{};
    if (int rc = check_group(L, groups, "GroupConv2D<float>", a))
        return rc;
    const int kt = a.K % 4 == 0 ? 4 : 1;
    const long long items = (long long)a.N * (a.G / CB) * (a.K / kt) * a.Ho * a.Wo * 4;
    if (items == 0)
        return SMALL_B200_OK;
    const unsigned blocks = (unsigned)((items + 255) / 256);
    if (kt == 4)
        groupconv2d_f32_kernel<4><<<blocks, 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    else
        groupconv2d_f32_kernel<1><<<blocks, 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("groupconv2d_f32_kernel");
}

int small_b200_blockconv2d_f32(const small_b200_layer *L, int32_t groups, const float *in, const float *filt,
                               const float *bias, float *out, void *stream)
{
    if (!L)
        return fail(SMALL_B200_INVALID_ARGUMENT, "GroupConv2D<float> (fused forms) ERROR: null layer.");
    small_b200_layer B = *L;
    B.C = B.K = CB;
    GArgs a{};
    if (groups <= 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "GroupConv2D<float> (fused forms) ERROR: output_groups unsupported.");
    if (int rc = check_group(&B, CB, "GroupConv2D<float> (fused forms)", a)) // the group count has no block here
        return rc;
    a.G = groups;
    const long long items = (long long)a.N * a.G * a.Ho * a.Wo * 4;
    if (items == 0)
        return SMALL_B200_OK;
    blockconv2d_f32_kernel<<<(unsigned)((items + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("blockconv2d_f32_kernel");
}

int small_b200_groupconv2d_u8(const small_b200_layer *L, int32_t groups, const uint8_t *in, const uint8_t *filt,
                              const int32_t *bias, uint8_t *out, void *stream)
{
    GArgs a{};
    if (int rc = check_group(L, groups, "GroupConv2D<quint8>", a))
        return rc;
    if (a.lshift < 0 || a.lshift > 31 || a.rshift < 0 || a.rshift > 31)
        return fail(SMALL_B200_INVALID_ARGUMENT, "GroupConv2D<quint8> ERROR: shift out of range.");
    if (a.sh != a.stride)
        return fail(SMALL_B200_INVALID_ARGUMENT, "GroupConv2D<quint8> ERROR: stride unsupported.");
    if (a.accumulate)
        // The int32 partial sums of output channel k of the groups start at byte k * Ho*Wo*16 of the
        // output buffer and are four times as long as the channel's bytes (interface_abstract.hpp:1470,
        // q_abstract_layer.hpp:1135-1144), so they overlap unless a group has ONE output channel -- and
        // the interface accepts multiples of 16 channels per group only.  No shape has a defined result.
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "PartialGroupConv2D<quint8> ERROR: the int32 partial sums of different output channels overlap "
                    "inside the output buffer for every shape the interface accepts.");
    const long long items = (long long)a.N * (a.G / CB) * a.K * a.Ho * a.Wo;
    if (items == 0)
        return SMALL_B200_OK;
    groupconv2d_u8_kernel<<<(unsigned)((items + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("groupconv2d_u8_kernel");
}
} // extern "C"
