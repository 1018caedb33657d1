// conv_f32.cu -- fp32 dense convolution on the CUDA cores (FFMA), implicit GEMM over the
// packed layout.  Replaces small::detail::abstract_layer<FloatBuffer,1,C_ob,C_ib,W_ob,
// stride,UNROLL,OP_CONV,2,rewrite> (include/small/abstract_layer.hpp:1368-1823) and its
// FLOAT_CONV_TILE_C microkernel (platforms/reference/intrinsics_float.h:262-281).
//
// Work decomposition
//   CTA  : TH x TW = 128 output pixels of one image  x  BN output channels
//   loop : input-channel block (16 ch) -> kernel row -> kernel col -> channel, the same
//          order in which the reference adds terms (abstract_layer.hpp:1630, :542-563)
//   stage: per input-channel block, the input patch (with halo, zero-filled outside the
//          image) and that block's filter slice are staged in shared memory with
//          cp.async, double buffered
//   thread: 8 consecutive pixels of one tile row x CH output channels in registers
#include <mutex>

#include "common.cuh"

namespace
{
using namespace sb;

constexpr int TH = 8, TW = 16; // output tile (rows x cols); one thread owns 8 cols of one row
constexpr int PXT = 8;         // pixels per thread

struct ConvArgs
{
    int N, C, K, H, W, Ho, Wo, Fh, Fw, stride, pad_t, pad_l;
    int sh;           // stride along the height (`stride` and the kernels' STRIDE are along the width)
    int cbs;          // input channel blocks
    int PH, PW;       // patch rows / cols
    int tiles_h, tiles_w, kblocks; // kblocks = K / BN
    int accumulate, act;
    float slope;
    int pool; // 1 = a 2x2 stride-2 max pool follows inside the kernel (output is Ho/2 x Wo/2)
};

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid)
{
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0; // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// BN: output channels per CTA; CH: output channels per thread (two groups of CH/2... for
// CH = 8 the thread owns channels [4g,4g+4) and [BN/2+4g, BN/2+4g+4) so that a quarter
// warp reads 128 contiguous bytes of the filter slice; for CH = 4 just [4g,4g+4)).
//
// POOL: the 2x2 stride-2 max pool that follows the convolution (fused_interface_abstract.hpp:463,
// Conv2D_Bias_ReLU_Maxpool2D) is taken in registers: a thread's 8 pixels hold four horizontal
// pairs, and the two rows of a pair of rows sit 16 lanes apart in the same warp.
template <int BN, int CH, int STRIDE, bool POOL>
__global__ void __launch_bounds__(16 * BN / CH)
conv2d_f32_kernel(const ConvArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                  const float *__restrict__ bias, float *__restrict__ out)
{
    constexpr int NT = 16 * BN / CH; // threads
    constexpr int CG = BN / CH;      // channel groups
    extern __shared__ __align__(16) float smem[];
    const int taps = a.Fh * a.Fw;
    const int patch_f = a.PH * a.PW * CB;  // floats per patch
    const int wts_f = taps * CB * BN;      // floats per filter slice
    const int stage_f = patch_f + wts_f;

    // tile coordinates: kb fastest so CTAs that share an input patch run together
    int bid = blockIdx.x;
    const int kb = bid % a.kblocks; bid /= a.kblocks;
    const int tw = bid % a.tiles_w; bid /= a.tiles_w;
    const int th = bid % a.tiles_h; bid /= a.tiles_h;
    const int n = bid;
    const int oh0 = th * TH, ow0 = tw * TW;
    const int ih0 = oh0 * a.sh - a.pad_t, iw0 = ow0 * STRIDE - a.pad_l;

    const int tid = threadIdx.x;
    const int cg = tid % CG;       // channel group (fast: lanes of a quarter warp share pixels)
    const int pg = tid / CG;       // pixel group 0..15
    const int r = pg >> 1;         // tile row
    const int c0 = (pg & 1) * PXT; // first tile col

    const float *in_img = in + (size_t)n * a.C * a.H * a.W;
    const size_t in_cb_stride = (size_t)a.H * a.W * CB;
    // filter: [K/16][C/16][taps][16][16]
    const size_t f_kb16_stride = (size_t)a.cbs * taps * CB * CB;

    auto load_stage = [&](int cb, int buf) {
        float *patch = smem + buf * stage_f;
        float *wts = patch + patch_f;
        // input patch: PH*PW pixels x 4 chunks of 16 B
        const float *src_cb = in_img + (size_t)cb * in_cb_stride;
        const int nchunk = a.PH * a.PW * 4;
        for (int i = tid; i < nchunk; i += NT)
        {
            const int q = i & 3, pix = i >> 2;
            const int pr = pix / a.PW, pc = pix - pr * a.PW;
            const int ih = ih0 + pr, iw = iw0 + pc;
            const bool ok = (ih >= 0) && (ih < a.H) && (iw >= 0) && (iw < a.W);
            const float *src = ok ? src_cb + ((size_t)ih * a.W + iw) * CB + q * 4 : in;
            cp_async16(patch + pix * CB + q * 4, src, ok);
        }
        // filter slice -> smem [tap][c][BN]
        const int wchunk = taps * CB * (BN / 4);
        for (int i = tid; i < wchunk; i += NT)
        {
            const int k4 = i % (BN / 4);
            const int tc = i / (BN / 4); // tap*16 + c
            const int kk = k4 * 4;       // channel inside the CTA's BN
            const int kb16 = (kb * BN + kk) / CB;
            const float *src = filt + (size_t)kb16 * f_kb16_stride + (size_t)cb * taps * CB * CB +
                               (size_t)tc * CB + (kk % CB);
            cp_async16(wts + tc * BN + kk, src, true);
        }
    };

    float acc[PXT][CH];
#pragma unroll
    for (int j = 0; j < PXT; ++j)
#pragma unroll
        for (int c = 0; c < CH; ++c)
            acc[j][c] = 0.f;

    // channel offsets owned by this thread inside the CTA's BN
    const int ko0 = cg * 4;
    const int ko1 = (CH == 8) ? BN / 2 + cg * 4 : 0;

    const int oh = oh0 + r;
    const bool row_ok = oh < a.Ho;

    // seed: existing output (Partial*) and/or bias, as Bias -> PartialConv2D does
    // (include/small/Conv2DLayer.hpp:827-835)
#pragma unroll
    for (int half = 0; half < CH / 4; ++half)
    {
        const int kg = kb * BN + (half ? ko1 : ko0);
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias)
            bv = *reinterpret_cast<const float4 *>(bias + kg);
#pragma unroll
        for (int j = 0; j < PXT; ++j)
        {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            const int ow = ow0 + c0 + j;
            if (a.accumulate && row_ok && ow < a.Wo)
                s = *reinterpret_cast<const float4 *>(
                    out + (((size_t)n * (a.K / CB) + kg / CB) * a.Ho * a.Wo + (size_t)oh * a.Wo + ow) * CB + (kg % CB));
            if (bias)
            {
                s.x += bv.x; s.y += bv.y; s.z += bv.z; s.w += bv.w;
            }
            acc[j][half * 4 + 0] = s.x; acc[j][half * 4 + 1] = s.y;
            acc[j][half * 4 + 2] = s.z; acc[j][half * 4 + 3] = s.w;
        }
    }

    load_stage(0, 0);
    cp_async_commit();

    for (int cb = 0; cb < a.cbs; ++cb)
    {
        const int buf = cb & 1;
        if (cb + 1 < a.cbs)
            load_stage(cb + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const float *patch = smem + buf * stage_f;
        const float *wts = patch + patch_f;
        const float *prow = patch + ((r * a.sh) * a.PW + c0 * STRIDE) * CB;
        for (int kh = 0; kh < a.Fh; ++kh)
        {
            for (int kw = 0; kw < a.Fw; ++kw)
            {
                const float *ap = prow + (kh * a.PW + kw) * CB;
                const float *wp = wts + (kh * a.Fw + kw) * CB * BN;
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4)
                {
                    float4 av[PXT];
#pragma unroll
                    for (int j = 0; j < PXT; ++j)
                        av[j] = *reinterpret_cast<const float4 *>(ap + j * STRIDE * CB + c4 * 4);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                    {
                        const float *wrow = wp + (c4 * 4 + cc) * BN;
                        const float4 b0 = *reinterpret_cast<const float4 *>(wrow + ko0);
                        float4 b1 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (CH == 8)
                            b1 = *reinterpret_cast<const float4 *>(wrow + ko1);
#pragma unroll
                        for (int j = 0; j < PXT; ++j)
                        {
                            const float x = (cc == 0) ? av[j].x : (cc == 1) ? av[j].y : (cc == 2) ? av[j].z : av[j].w;
                            acc[j][0] = fmaf(x, b0.x, acc[j][0]);
                            acc[j][1] = fmaf(x, b0.y, acc[j][1]);
                            acc[j][2] = fmaf(x, b0.z, acc[j][2]);
                            acc[j][3] = fmaf(x, b0.w, acc[j][3]);
                            if (CH == 8)
                            {
                                acc[j][4] = fmaf(x, b1.x, acc[j][4]);
                                acc[j][5] = fmaf(x, b1.y, acc[j][5]);
                                acc[j][6] = fmaf(x, b1.z, acc[j][6]);
                                acc[j][7] = fmaf(x, b1.w, acc[j][7]);
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();
    }

    if (POOL)
    {
        // bias and activation are already in; rows r and r^1 live in lanes l and l^(2*CG)
        static_assert(!POOL || CG == 8, "the pooled epilogue pairs rows 16 lanes apart");
        const int Hp = a.Ho / 2, Wp = a.Wo / 2;
#pragma unroll
        for (int half = 0; half < CH / 4; ++half)
        {
            const int kg = kb * BN + (half ? ko1 : ko0);
            float *obase = out + (((size_t)n * (a.K / CB) + kg / CB) * Hp * Wp + (size_t)(oh >> 1) * Wp) * CB + (kg % CB);
#pragma unroll
            for (int j = 0; j < PXT; j += 2)
            {
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                {
                    const float x0 = apply_act_ns(acc[j][half * 4 + q], act_neg_scale(a.act, a.slope));
                    const float x1 = apply_act_ns(acc[j + 1][half * 4 + q], act_neg_scale(a.act, a.slope));
                    const float m = fmaxf(x0, x1);
                    v[q] = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2 * CG));
                }
                const int pw = (ow0 + c0 + j) >> 1;
                if ((r & 1) == 0 && row_ok && pw < Wp)
                    *reinterpret_cast<float4 *>(obase + (size_t)pw * CB) = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
        return;
    }
    if (!row_ok)
        return;
#pragma unroll
    for (int half = 0; half < CH / 4; ++half)
    {
        const int kg = kb * BN + (half ? ko1 : ko0);
        float *obase = out + (((size_t)n * (a.K / CB) + kg / CB) * a.Ho * a.Wo + (size_t)oh * a.Wo) * CB + (kg % CB);
#pragma unroll
        for (int j = 0; j < PXT; ++j)
        {
            const int ow = ow0 + c0 + j;
            if (ow < a.Wo)
            {
                float4 v;
                v.x = apply_act_ns(acc[j][half * 4 + 0], act_neg_scale(a.act, a.slope));
                v.y = apply_act_ns(acc[j][half * 4 + 1], act_neg_scale(a.act, a.slope));
                v.z = apply_act_ns(acc[j][half * 4 + 2], act_neg_scale(a.act, a.slope));
                v.w = apply_act_ns(acc[j][half * 4 + 3], act_neg_scale(a.act, a.slope));
                *reinterpret_cast<float4 *>(obase + (size_t)ow * CB) = v;
            }
        }
    }
}

// First layer: C in {1,2,3}, the image is HWC-interleaved (buffers.hpp:52-57).  One thread
// per output pixel and 16-channel block; the filter slice [taps][C][16] sits in shared memory.
__global__ void __launch_bounds__(256)
conv2d_first_f32_kernel(const ConvArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                        const float *__restrict__ bias, float *__restrict__ out)
{
    extern __shared__ __align__(16) float w[]; // [taps][C][16]
    const int taps = a.Fh * a.Fw;
    const int kb = blockIdx.y;
    const int n = blockIdx.z;
    const int wn = taps * a.C * CB;
    const float *fsrc = filt + (size_t)kb * wn;
    for (int i = threadIdx.x; i < wn; i += blockDim.x)
        w[i] = fsrc[i];
    __syncthreads();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= a.Ho * a.Wo)
        return;
    const int oh = p / a.Wo, ow = p - oh * a.Wo;
    float *o = out + (((size_t)n * (a.K / CB) + kb) * a.Ho * a.Wo + p) * CB;
    float acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
    {
        float s = a.accumulate ? o[k] : 0.f;
        if (bias)
            s += bias[kb * CB + k];
        acc[k] = s;
    }
    const float *img = in + (size_t)n * a.C * a.H * a.W;
    for (int kh = 0; kh < a.Fh; ++kh)
    {
        const int ih = oh * a.sh - a.pad_t + kh;
        if (ih < 0 || ih >= a.H)
            continue;
        for (int kw = 0; kw < a.Fw; ++kw)
        {
            const int iw = ow * a.stride - a.pad_l + kw;
            if (iw < 0 || iw >= a.W)
                continue;
            const float *px = img + ((size_t)ih * a.W + iw) * a.C;
            const float *wt = w + (kh * a.Fw + kw) * a.C * CB;
            for (int c = 0; c < a.C; ++c)
            {
                const float x = __ldg(px + c);
#pragma unroll
                for (int k = 0; k < CB; ++k)
                    acc[k] = fmaf(x, wt[c * CB + k], acc[k]);
            }
        }
    }
#pragma unroll
    for (int k4 = 0; k4 < CB; k4 += 4)
    {
        float4 v;
        v.x = apply_act_ns(acc[k4 + 0], act_neg_scale(a.act, a.slope));
        v.y = apply_act_ns(acc[k4 + 1], act_neg_scale(a.act, a.slope));
        v.z = apply_act_ns(acc[k4 + 2], act_neg_scale(a.act, a.slope));
        v.w = apply_act_ns(acc[k4 + 3], act_neg_scale(a.act, a.slope));
        *reinterpret_cast<float4 *>(o + k4) = v;
    }
}

// First layer followed by a 2x2 stride-2 max pool: one thread per POOLED pixel and 16-channel
// block computes the four convolution outputs under it (64 accumulators), so the full-size
// activation never reaches memory.  Stride-1 convolution, even Ho and Wo.
__global__ void __launch_bounds__(128)
conv2d_first_pool_f32_kernel(const ConvArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                             const float *__restrict__ bias, float *__restrict__ out)
{
    extern __shared__ __align__(16) float w[]; // [taps][C][16]
    const int taps = a.Fh * a.Fw;
    const int kb = blockIdx.y;
    const int n = blockIdx.z;
    const int wn = taps * a.C * CB;
    const float *fsrc = filt + (size_t)kb * wn;
    for (int i = threadIdx.x; i < wn; i += blockDim.x)
        w[i] = fsrc[i];
    __syncthreads();
    const int Hp = a.Ho / 2, Wp = a.Wo / 2;
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= Hp * Wp)
        return;
    const int ph = p / Wp, pw = p - ph * Wp;
    float acc[4][CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
    {
        const float s = bias ? bias[kb * CB + k] : 0.f;
        acc[0][k] = s; acc[1][k] = s; acc[2][k] = s; acc[3][k] = s;
    }
    const float *img = in + (size_t)n * a.C * a.H * a.W;
    const int ih0 = 2 * ph - a.pad_t, iw0 = 2 * pw - a.pad_l;
    // input rows ih0 .. ih0+Fh and columns iw0 .. iw0+Fw feed the 2x2 outputs
    for (int dr = 0; dr <= a.Fh; ++dr)
    {
        const int ih = ih0 + dr;
        if (ih < 0 || ih >= a.H)
            continue;
        for (int dc = 0; dc <= a.Fw; ++dc)
        {
            const int iw = iw0 + dc;
            if (iw < 0 || iw >= a.W)
                continue;
            const float *px = img + ((size_t)ih * a.W + iw) * a.C;
            for (int c = 0; c < a.C; ++c)
            {
                const float x = __ldg(px + c);
                // output (oy, ox) of the 2x2 block sees this pixel through tap (dr-oy, dc-ox)
#pragma unroll
                for (int oy = 0; oy < 2; ++oy)
                {
                    const int kh = dr - oy;
                    if (kh < 0 || kh >= a.Fh)
                        continue;
#pragma unroll
                    for (int ox = 0; ox < 2; ++ox)
                    {
                        const int kw = dc - ox;
                        if (kw < 0 || kw >= a.Fw)
                            continue;
                        const float4 *wt = reinterpret_cast<const float4 *>(w + ((kh * a.Fw + kw) * a.C + c) * CB);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                        {
                            const float4 wv = wt[k4];
                            float *ac = acc[oy * 2 + ox] + k4 * 4;
                            ac[0] = fmaf(x, wv.x, ac[0]); ac[1] = fmaf(x, wv.y, ac[1]);
                            ac[2] = fmaf(x, wv.z, ac[2]); ac[3] = fmaf(x, wv.w, ac[3]);
                        }
                    }
                }
            }
        }
    }
    float *o = out + (((size_t)n * (a.K / CB) + kb) * Hp * Wp + p) * CB;
#pragma unroll
    for (int k4 = 0; k4 < CB; k4 += 4)
    {
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            v[q] = fmaxf(fmaxf(apply_act_ns(acc[0][k4 + q], act_neg_scale(a.act, a.slope)), apply_act_ns(acc[1][k4 + q], act_neg_scale(a.act, a.slope))),
                         fmaxf(apply_act_ns(acc[2][k4 + q], act_neg_scale(a.act, a.slope)), apply_act_ns(acc[3][k4 + q], act_neg_scale(a.act, a.slope))));
        *reinterpret_cast<float4 *>(o + k4) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// The same for compile-time shapes (the 3-channel 3x3 first layer of the image networks): the
// (FH+1) x (FW+1) x C input patch of the 2x2 block sits in registers and every filter vector
// fetched from shared memory feeds all four outputs (16 FMAs per 128-bit load).
// POOL = false: the same register patch without the pool (the first layer on its own): the four
// outputs of a thread's 2x2 block are stored.  A thread's two outputs of a row are 128 contiguous
// bytes and a warp's are 4 KB, but written straight from the registers every store instruction
// would touch 32 separate 16-byte pieces; the warp passes each row through its own 4.5 KB of shared
// memory (144-byte pitch: conflict-free both ways) and writes 512 contiguous bytes per instruction.
// SLOT >= 0: the filter of the layer's ONE block of 16 output channels sits in constant memory
// (c_first_w[SLOT], copied there by the launch on the same stream), and every multiply-add takes its
// weight straight from the constant bank.  With the filter in shared memory each 128-bit weight
// fetch feeds only 16 multiply-adds, and those broadcast fetches, not the FMA pipe, set the pace
// (the kernel ran at half the pipe's rate whatever its occupancy).
constexpr int FIRST_W_SLOTS = 4;
constexpr int FIRST_W_FLOATS = 3 * 3 * 3 * CB;
__constant__ float c_first_w[FIRST_W_SLOTS][FIRST_W_FLOATS];

template <int C, int FH, int FW, bool POOL = true, int SLOT = -1>
__global__ void __launch_bounds__(128)
conv2d_first_pool_fixed_f32_kernel(const ConvArgs a, const float *__restrict__ in, const float *__restrict__ filt,
                                   const float *__restrict__ bias, float *__restrict__ out)
{
    constexpr int wn = FH * FW * C * CB;
    __shared__ __align__(16) float w_s[SLOT < 0 ? wn : 4]; // [taps][C][16]
    const int kb = blockIdx.y;
    const int n = blockIdx.z;
    if (SLOT < 0)
    {
        const float *fsrc = filt + (size_t)kb * wn;
        for (int i = threadIdx.x; i < wn; i += blockDim.x)
            w_s[i] = fsrc[i];
        __syncthreads();
    }
    const float *w = SLOT < 0 ? w_s : c_first_w[SLOT < 0 ? 0 : SLOT];
    const int Hp = a.Ho / 2, Wp = a.Wo / 2;
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = p < Hp * Wp;
    if (!live)
    {
        if (POOL)
            return;
        p = Hp * Wp - 1; // computes a pixel it will not store: the warp's staging needs every lane
    }
    const int ph = p / Wp, pw = p - ph * Wp;
    const float *img = in + (size_t)n * C * a.H * a.W;
    const int ih0 = 2 * ph - a.pad_t, iw0 = 2 * pw - a.pad_l;
    float x[FH + 1][FW + 1][C];
#pragma unroll
    for (int dr = 0; dr <= FH; ++dr)
    {
        const int ih = ih0 + dr;
        const bool rok = ih >= 0 && ih < a.H;
#pragma unroll
        for (int dc = 0; dc <= FW; ++dc)
        {
            const int iw = iw0 + dc;
            const bool ok = rok && iw >= 0 && iw < a.W;
            const float *px = img + ((size_t)(ok ? ih : 0) * a.W + (ok ? iw : 0)) * C;
#pragma unroll
            for (int c = 0; c < C; ++c)
                x[dr][dc][c] = ok ? __ldg(px + c) : 0.f; // a padded tap adds nothing
        }
    }
    float acc[4][CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
    {
        const float s = bias ? bias[kb * CB + k] : 0.f;
        acc[0][k] = s; acc[1][k] = s; acc[2][k] = s; acc[3][k] = s;
    }
#pragma unroll
    for (int kh = 0; kh < FH; ++kh)
#pragma unroll
        for (int kw = 0; kw < FW; ++kw)
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                const float *wt = w + ((kh * FW + kw) * C + c) * CB;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)
                {
                    const float4 wv = SLOT < 0 ? reinterpret_cast<const float4 *>(wt)[k4]
                                               : make_float4(wt[4 * k4], wt[4 * k4 + 1], wt[4 * k4 + 2], wt[4 * k4 + 3]);
#pragma unroll
                    for (int o = 0; o < 4; ++o)
                    {
                        const float xv = x[(o >> 1) + kh][(o & 1) + kw][c];
                        float *ac = acc[o] + k4 * 4;
                        ac[0] = fmaf(xv, wv.x, ac[0]); ac[1] = fmaf(xv, wv.y, ac[1]);
                        ac[2] = fmaf(xv, wv.z, ac[2]); ac[3] = fmaf(xv, wv.w, ac[3]);
                    }
                }
            }
    if (!POOL)
    {
        __shared__ __align__(16) float stage[4][32 * 36]; // per warp: 32 threads x (128 bytes + 16 of padding)
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        float *mine = stage[warp] + lane * 36;
        const float ns = act_neg_scale(a.act, a.slope);
        float *plane = out + ((size_t)n * (a.K / CB) + kb) * a.Ho * a.Wo * CB;
#pragma unroll
        for (int dr = 0; dr < 2; ++dr)
        {
#pragma unroll
            for (int dc = 0; dc < 2; ++dc)
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)
                {
                    const float *ac = acc[dr * 2 + dc] + k4 * 4;
                    *reinterpret_cast<float4 *>(mine + dc * 16 + k4 * 4) =
                        make_float4(apply_act_ns(ac[0], ns), apply_act_ns(ac[1], ns), apply_act_ns(ac[2], ns),
                                    apply_act_ns(ac[3], ns));
                }
            __syncwarp();
            // piece j of the warp's 32 x 8 pieces belongs to thread j / 8: pooled pixel p0 + j / 8
#pragma unroll
            for (int it = 0; it < 8; ++it)
            {
                const int j = it * 32 + lane, t = j >> 3, piece = j & 7;
                const int pt = blockIdx.x * blockDim.x + warp * 32 + t;
                if (pt < Hp * Wp)
                {
                    const int pht = pt / Wp, pwt = pt - pht * Wp;
                    const float4 v = *reinterpret_cast<const float4 *>(stage[warp] + t * 36 + piece * 4);
                    *reinterpret_cast<float4 *>(plane + ((size_t)(2 * pht + dr) * a.Wo + 2 * pwt) * CB + piece * 4) = v;
                }
            }
            __syncwarp();
        }
        return;
    }
    float *o = out + (((size_t)n * (a.K / CB) + kb) * Hp * Wp + p) * CB;
#pragma unroll
    for (int k4 = 0; k4 < CB; k4 += 4)
    {
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            v[q] = fmaxf(fmaxf(apply_act_ns(acc[0][k4 + q], act_neg_scale(a.act, a.slope)), apply_act_ns(acc[1][k4 + q], act_neg_scale(a.act, a.slope))),
                         fmaxf(apply_act_ns(acc[2][k4 + q], act_neg_scale(a.act, a.slope)), apply_act_ns(acc[3][k4 + q], act_neg_scale(a.act, a.slope))));
        *reinterpret_cast<float4 *>(o + k4) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

template <int BN, int CH, int STRIDE, bool POOL = false>
int launch_conv(const ConvArgs &a, size_t smem_bytes, const float *in, const float *filt,
                const float *bias, float *out, cudaStream_t st)
{
    auto kern = conv2d_f32_kernel<BN, CH, STRIDE, POOL>;
    static PerDeviceOnce configured; // one attribute call per instantiation and device
    int dev;
    if (configured.needed(&dev))
    {
        SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured.mark(dev);
    }
    const long long blocks = (long long)a.N * a.tiles_h * a.tiles_w * a.kblocks;
    kern<<<(unsigned)blocks, 16 * BN / CH, smem_bytes, st>>>(a, in, filt, bias, out);
    return launched("conv2d_f32_kernel");
}
} // namespace

namespace
{
// pool: 0 = plain convolution; 1 = fused 2x2 stride-2 max pool (the caller has checked the shape)
// Constant-memory slot of a first-layer filter: a filter pointer keeps the slot it got, for the life of
// the process, and the filter's bytes are copied into it again on every call, on the call's stream.
// Slots are never taken away, so a kernel in flight on another stream can only meet a copy of the
// same filter; the fifth distinct filter of a device (and every later one) gets -1 and runs the
// shared-memory form.
int first_layer_slot(const float *filt)
{
    static std::mutex mu;
    static const float *owner[16][FIRST_W_SLOTS] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16)
        return -1;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < FIRST_W_SLOTS; ++i)
        if (owner[dev][i] == filt)
            return i;
    for (int i = 0; i < FIRST_W_SLOTS; ++i)
        if (!owner[dev][i])
        {
            owner[dev][i] = filt;
            return i;
        }
    return -1;
}

template <bool POOL>
int launch_first_fixed(const ConvArgs &a, dim3 grid, const float *in, const float *filt, const float *bias, float *out,
                       cudaStream_t st)
{
    const int slot = a.K == CB ? first_layer_slot(filt) : -1;
    if (slot >= 0)
        SB_CUDA(cudaMemcpyToSymbolAsync(c_first_w, filt, FIRST_W_FLOATS * sizeof(float),
                                        (size_t)slot * FIRST_W_FLOATS * sizeof(float), cudaMemcpyDeviceToDevice, st));
    switch (slot)
    {
    case 0: conv2d_first_pool_fixed_f32_kernel<3, 3, 3, POOL, 0><<<grid, 128, 0, st>>>(a, in, filt, bias, out); break;
    case 1: conv2d_first_pool_fixed_f32_kernel<3, 3, 3, POOL, 1><<<grid, 128, 0, st>>>(a, in, filt, bias, out); break;
    case 2: conv2d_first_pool_fixed_f32_kernel<3, 3, 3, POOL, 2><<<grid, 128, 0, st>>>(a, in, filt, bias, out); break;
    case 3: conv2d_first_pool_fixed_f32_kernel<3, 3, 3, POOL, 3><<<grid, 128, 0, st>>>(a, in, filt, bias, out); break;
    default: conv2d_first_pool_fixed_f32_kernel<3, 3, 3, POOL><<<grid, 128, 0, st>>>(a, in, filt, bias, out); break;
    }
    return launched(POOL ? "conv2d_first_pool_fixed_f32_kernel" : "conv2d_first_fixed_f32_kernel");
}

int conv2d_f32_impl(const small_b200_layer *L, int pool, const float *in, const float *filt,
                    const float *bias, float *out, void *stream)
{
    if (int rc = check_window_layer(L, "Conv2D<float>", true, 2))
        return rc;
    ConvArgs a;
    a.pool = pool;
    a.N = L->N; a.C = L->C; a.K = L->K; a.H = L->H; a.W = L->W;
    a.Fh = L->Fh; a.Fw = L->Fw; a.stride = L->stride; a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.sh = row_stride(L);
    if (pool && a.sh != L->stride)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D+MaxPool2D<float> ERROR: shape not covered by the fused kernel.");
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, a.sh);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    a.accumulate = L->accumulate; a.act = L->act; a.slope = L->slope;
    if (a.N == 0 || a.Ho == 0 || a.Wo == 0)
        return SMALL_B200_OK;
    cudaStream_t st = as_stream(stream);

    if (L->C < CB)
    {
        a.cbs = 1; a.PH = a.PW = 0; a.tiles_h = a.tiles_w = a.kblocks = 0;
        const size_t smem = (size_t)L->Fh * L->Fw * L->C * CB * sizeof(float);
        if (smem > 48 * 1024)
            return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> ERROR: first-layer window too large.");
        if (pool)
        {
            dim3 grid(((a.Ho / 2) * (a.Wo / 2) + 127) / 128, a.K / CB, a.N);
            if (L->C == 3 && L->Fh == 3 && L->Fw == 3)
            {
                return launch_first_fixed<true>(a, grid, in, filt, bias, out, st);
            }
            conv2d_first_pool_f32_kernel<<<grid, 128, smem, st>>>(a, in, filt, bias, out);
            return launched("conv2d_first_pool_f32_kernel");
        }
        if (L->C == 3 && L->Fh == 3 && L->Fw == 3 && L->stride == 1 && a.sh == 1 && !L->accumulate && a.Ho % 2 == 0 &&
            a.Wo % 2 == 0 && a.Ho > 0 && a.Wo > 0)
        {
            // 2x2 output blocks from a register patch, rows written through shared memory
            dim3 grid(((a.Ho / 2) * (a.Wo / 2) + 127) / 128, a.K / CB, a.N);
            return launch_first_fixed<false>(a, grid, in, filt, bias, out, st);
        }
        dim3 grid((a.Ho * a.Wo + 255) / 256, a.K / CB, a.N);
        conv2d_first_f32_kernel<<<grid, 256, smem, st>>>(a, in, filt, bias, out);
        return launched("conv2d_first_f32_kernel");
    }

    a.cbs = L->C / CB;
    a.PH = (TH - 1) * a.sh + L->Fh;
    a.PW = (TW - 1) * L->stride + L->Fw;
    a.tiles_h = (a.Ho + TH - 1) / TH;
    a.tiles_w = (a.Wo + TW - 1) / TW;
    const size_t patch_b = (size_t)a.PH * a.PW * CB * sizeof(float);
    auto smem_for = [&](int bn) { return 2 * (patch_b + (size_t)L->Fh * L->Fw * CB * bn * sizeof(float)); };
    const size_t limit = 200 * 1024;
    int bn = 0;
    if (pool)
    {
        // the pooled epilogue is written for 8 channel groups per pixel group
        if (a.K % 64 == 0 && smem_for(64) <= limit)
            return launch_conv<64, 8, 1, true>(((a.kblocks = a.K / 64), a), smem_for(64), in, filt, bias, out, st);
        if (a.K % 32 == 0 && smem_for(32) <= limit)
            return launch_conv<32, 4, 1, true>(((a.kblocks = a.K / 32), a), smem_for(32), in, filt, bias, out, st);
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D+MaxPool2D<float> ERROR: shape not covered by the fused kernel.");
    }
    if (a.K % 64 == 0 && smem_for(64) <= limit)
        bn = 64;
    else if (a.K % 32 == 0 && smem_for(32) <= limit)
        bn = 32;
    else if (smem_for(16) <= limit)
        bn = 16;
    else
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> ERROR: window too large for the staged kernel.");
    a.kblocks = a.K / bn;
    const size_t smem = smem_for(bn);
    const bool s2 = L->stride == 2;
    if (bn == 64)
        return s2 ? launch_conv<64, 8, 2>(a, smem, in, filt, bias, out, st)
                  : launch_conv<64, 8, 1>(a, smem, in, filt, bias, out, st);
    if (bn == 32)
        return s2 ? launch_conv<32, 4, 2>(a, smem, in, filt, bias, out, st)
                  : launch_conv<32, 4, 1>(a, smem, in, filt, bias, out, st);
    return s2 ? launch_conv<16, 4, 2>(a, smem, in, filt, bias, out, st)
              : launch_conv<16, 4, 1>(a, smem, in, filt, bias, out, st);
}
} // namespace

extern "C"
{
int small_b200_conv2d_f32(const small_b200_layer *L, const float *in, const float *filt, const float *bias,
                          float *out, void *stream)
{
    return conv2d_f32_impl(L, 0, in, filt, bias, out, stream);
}

int small_b200_conv2d_maxpool_f32_supported(const small_b200_layer *conv, const small_b200_layer *pool)
{
    if (!conv || !pool || conv->stride != 1 || row_stride(conv) != 1 || row_stride(pool) != pool->stride || conv->accumulate)
        return 0;
    if (conv->K % (conv->C < CB ? 16 : 32) != 0) // the staged kernel pairs rows inside a warp: 32 or 64 channels per CTA
        return 0;
    if (pool->Fh != 2 || pool->Fw != 2 || pool->stride != 2 || pool->pad_t || pool->pad_b || pool->pad_l || pool->pad_r)
        return 0;
    const int Ho = out_dim(conv->H, conv->pad_t, conv->pad_b, conv->Fh, 1);
    const int Wo = out_dim(conv->W, conv->pad_l, conv->pad_r, conv->Fw, 1);
    if (Ho <= 0 || Wo <= 0 || Ho % 2 || Wo % 2 || pool->H != Ho || pool->W != Wo || pool->C != conv->K ||
        pool->N != conv->N)
        return 0;
    return 1;
}

int small_b200_conv2d_maxpool_f32(const small_b200_layer *conv, const small_b200_layer *pool, const float *in,
                                  const float *filt, const float *bias, float *out, void *stream)
{
    if (!small_b200_conv2d_maxpool_f32_supported(conv, pool))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D+MaxPool2D<float> ERROR: shape not covered by the fused kernel.");
    return conv2d_f32_impl(conv, 1, in, filt, bias, out, stream);
}
} // extern "C"
