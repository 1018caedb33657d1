// conv_u8_ring.cu -- small::Conv2D<QUInt8Buffer> (include/small/interface_abstract.hpp:229-404, loop nest
// include/small/q_abstract_layer.hpp:894-1571) for every window, stride and padding as an implicit GEMM on
// tcgen05.mma.kind::i8.
//
// A tile is 128 consecutive output pixels of the batch (pixel index = image * Ho*Wo + oh * Wo + ow) times
// NT output channels; the reduction runs over (kernel row, kernel column, pair of input channel blocks)
// in steps of K = 32 bytes.  For each step the producer warps gather the 128 x 32-byte slice of the
// im2col matrix (a pixel's 16 channels of one block are 16 contiguous bytes of the packed activation)
// and the 32 x NT slice of the packed filter into one stage of a ring in shared memory; one thread
// issues the MMAs, whose completion hands the stage back; four warps requantise the finished tile out
// of tensor memory while the next tile accumulates into the other half of it.
//
// Zero points (the reference ADDS them: (a + zero_in) * (b + zero_filt), and skips taps outside the image):
//   * filter zero point -128 with activation zero point 0 or -128 -- every quantised network here: the
//     operands enter as signed / unsigned bytes already shifted, a tap outside the image is a zero byte,
//     and the accumulator needs no correction at all;
//   * anything else: both operands enter as unsigned bytes with zero bytes outside the image, so the MMA
//     gives sum(a * b) over the valid taps.  zero_filt * sum(a) comes from sixteen extra accumulator
//     columns whose filter column is all ones; zero_in * sum(b) + n * zero_in * zero_filt is a
//     per-channel constant for interior pixels, and pixels at the border take away the per-tap channel
//     sums (a table in shared memory, built once per CTA) of the taps they do not have.
// The int32 partial-sum form stays on the CUDA-core kernel.
//
// First layers (1 to 3 channels, [H][W][C] activation, filter [K/16][1][Fh][Fw][C][16]) take the same
// route with the reduction index running over (kernel row, kernel column, channel) byte by byte.
#include "tc_common.cuh"

namespace
{
using namespace sb;

constexpr int TILE_M = 128;
constexpr int EPI_WARPS = 4, PROD_WARPS = 8;
constexpr int THREADS = (EPI_WARPS + PROD_WARPS + 1) * 32;
constexpr int STAGES = 8;
constexpr int IN_FLIGHT = 4; // reduction steps whose loads a producer thread has outstanding

struct RingArgs
{
    int N, H, W, C, K, Ho, Wo, Fh, Fw, stride, row_stride, pad_t, pad_l;
    int cib;      // channels per input block: 16, or C for a first layer
    int cbs;      // input channel blocks (1 for a first layer)
    int steps;    // reduction steps of 32 bytes
    int tiles;    // ceil(N * Ho * Wo / 128)
    int nblocks;  // K / NT
    int zero_in, zero_filt;
    int lshift, rshift, mult, k_zero;
};

template <int NT, bool GENERAL>
struct Geometry
{
    static constexpr int NCOLS = GENERAL ? NT + 16 : NT;     // accumulator columns: NT channels (+ the row sums)
    static constexpr uint32_t A_BYTES = 2 * TILE_M * CB;     // [2 chunks][128 pixels][16 B], K-major
    static constexpr uint32_t B_BYTES = NCOLS * 2 * CB;      // [NCOLS/16][2 chunks][16 rows][16 B], MN-major
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * NCOLS <= 32 ? 32 : 2 * NCOLS <= 64 ? 64 : 2 * NCOLS <= 128 ? 128
                                          : 2 * NCOLS <= 256 ? 256 : 512;
    static constexpr size_t RING = (size_t)STAGES * STAGE;
};

template <int NT, bool FIRST, bool GENERAL>
__global__ void __launch_bounds__(THREADS)
conv_u8_ring_kernel(const RingArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                    const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int *status)
{
    using G = Geometry<NT, GENERAL>;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ __align__(16) int seed[NT];
    int *tapsum = reinterpret_cast<int *>(smem + G::RING); // GENERAL: [Fh * Fw][NT] channel sums of the filter

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long total_px = (long long)a.N * a.Ho * a.Wo;
    const int nb = blockIdx.y;
    const int taps = a.Fh * a.Fw;
    const int kmax = taps * a.C; // first layers: rows of the filter of one channel group

    if (warp == EPI_WARPS + PROD_WARPS)
    {
        if (lane == 0)
        {
            for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], PROD_WARPS); mbar_init(&empty_bar[i], 1); }
            for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], EPI_WARPS); }
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, G::TMEM_COLS);
        tmem_relinquish();
    }
    if (GENERAL)
    {
        // the sixteen extra filter columns: column 0 all ones (its accumulator is the sum of the
        // activation bytes under the window), the others zero; never rewritten
        for (int i = tid; i < STAGES * 32; i += THREADS)
        {
            const int st = i >> 5, r = i & 31;
            *reinterpret_cast<uint4 *>(smem + (size_t)st * G::STAGE + G::A_BYTES + (size_t)(NT / CB) * 2 * CB * CB + (size_t)r * CB) =
                make_uint4(1u, 0u, 0u, 0u);
        }
        // channel sums of the filter per tap, needed only where the activation zero point is not zero
        if (a.zero_in != 0)
            for (int i = tid; i < taps * NT; i += THREADS)
            {
                const int tap = i / NT, k = i - tap * NT;
                const int kg = nb * (NT / CB) + k / CB, k16 = k % CB;
                int sum = 0;
                if (FIRST)
                    for (int c = 0; c < a.C; ++c)
                        sum += filt[((size_t)kg * kmax + (size_t)tap * a.C + c) * CB + k16];
                else
                    for (int c = 0; c < a.C; ++c)
                        sum += filt[((((size_t)kg * a.cbs + c / CB) * taps) + tap) * (CB * CB) + (size_t)(c % CB) * CB + k16];
                tapsum[i] = sum;
            }
        fence_proxy_async();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid < NT)
    {
        int c = a.k_zero + (bias ? bias[nb * NT + tid] : 0);
        if (GENERAL && a.zero_in != 0)
        {
            int all = 0;
            for (int tap = 0; tap < taps; ++tap)
                all += tapsum[tap * NT + tid];
            c += a.zero_in * all + taps * a.C * a.zero_in * a.zero_filt;
        }
        seed[tid] = c;
    }
    __syncthreads();
    const uint32_t tmem = tmem_base_s;

    if (warp < EPI_WARPS)
    {
        // ---- epilogue: thread = one pixel of the tile = one lane of tensor memory
        bool ok = true;
        int i = 0;
        for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++i)
        {
            const int buf = i & 1;
            const long long g = (long long)tile * TILE_M + tid;
            const bool live = g < total_px;
            const int n = live ? (int)(g / ((long long)a.Ho * a.Wo)) : 0;
            const int px = live ? (int)(g - (long long)n * a.Ho * a.Wo) : 0;
            const int oh = px / a.Wo, ow = px - oh * a.Wo;
            const int ih0 = oh * a.row_stride - a.pad_t, iw0 = ow * a.stride - a.pad_l;
            const bool border = GENERAL && a.zero_in != 0 &&
                                (ih0 < 0 || iw0 < 0 || ih0 + a.Fh > a.H || iw0 + a.Fw > a.W);
            ok = mbar_wait(&acc_full[buf], (i >> 1) & 1, status, 31);
            if (!ok)
                break;
            tc_fence_after_sync();
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * G::NCOLS);
            int base = 0;
            if (GENERAL)
            {
                uint32_t r[16];
                tmem_ld16(lane_base + NT, r);
                tmem_ld_wait();
                base = a.zero_filt * (int)r[0];
            }
            uint8_t *orow = out + (((size_t)n * (a.K / CB) + (size_t)nb * (NT / CB)) * a.Ho * a.Wo + px) * CB;
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 16)
            {
                uint32_t r[16];
                tmem_ld16(lane_base + c0, r);
                tmem_ld_wait();
                int q[16];
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4)
                {
                    const int4 s4 = *reinterpret_cast<const int4 *>(seed + c0 + 4 * e4);
                    q[4 * e4 + 0] = (int)r[4 * e4 + 0] + s4.x + base;
                    q[4 * e4 + 1] = (int)r[4 * e4 + 1] + s4.y + base;
                    q[4 * e4 + 2] = (int)r[4 * e4 + 2] + s4.z + base;
                    q[4 * e4 + 3] = (int)r[4 * e4 + 3] + s4.w + base;
                }
                if (border) // take away what the taps outside the image added to the constant
                    for (int kh = 0; kh < a.Fh; ++kh)
                        for (int kw = 0; kw < a.Fw; ++kw)
                        {
                            const int ih = ih0 + kh, iw = iw0 + kw;
                            if (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                                continue;
                            const int *t = tapsum + (kh * a.Fw + kw) * NT + c0;
                            const int nzz = a.C * a.zero_in * a.zero_filt;
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                q[e] -= a.zero_in * t[e] + nzz;
                        }
                const uint4 o = requant_pack16(q, a.lshift, a.rshift, a.mult);
                if (live)
                    *reinterpret_cast<uint4 *>(orow + (size_t)(c0 / CB) * a.Ho * a.Wo * CB) = o;
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[buf]);
        }
    }
    else if (warp < EPI_WARPS + PROD_WARPS)
    {
        // ---- producers: thread = (pixel row of the tile, which 16-byte chunk of the step)
        const int pt = tid - EPI_WARPS * 32;
        const int row = pt & (TILE_M - 1), half = pt >> 7;
        const int jpairs = (a.cbs + 1) / 2;
        const unsigned flip_a = (!GENERAL && a.zero_in != 0) ? 0x80808080u : 0u;
        const unsigned flip_b = GENERAL ? 0u : 0x80808080u;
        // this thread's piece of the filter slice: 16-byte row `brow` of chunk `bhalf` of channel group `bgrp`
        const bool has_b = pt < NT * 2;
        const int bgrp = pt >> 5, bhalf = (pt >> 4) & 1, brow = pt & 15;
        bool ok = true;
        // The (tile, reduction step) pairs of this CTA form one sequence; a thread keeps the loads of
        // IN_FLIGHT consecutive pairs outstanding, across tile boundaries, before it stores any of them.
        const unsigned my_tiles = ((unsigned)a.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
        const unsigned units = my_tiles * (unsigned)a.steps;
        const unsigned hw_out = (unsigned)(a.Ho * a.Wo);
        const int fwc = a.Fw * a.C;
        for (unsigned w0 = 0; w0 < units && ok; w0 += IN_FLIGHT)
        {
            uint4 va[IN_FLIGHT], vb[IN_FLIGHT];
#pragma unroll
            for (int u = 0; u < IN_FLIGHT; ++u)
            {
                va[u] = make_uint4(0u, 0u, 0u, 0u);
                vb[u] = make_uint4(0u, 0u, 0u, 0u);
                const unsigned w = w0 + u;
                if (w >= units)
                    continue;
                const unsigned ti = w / (unsigned)a.steps;
                const int q = (int)(w - ti * (unsigned)a.steps);
                const unsigned g = (blockIdx.x + ti * gridDim.x) * TILE_M + row;
                const bool live = g < total_px;
                const unsigned n = live ? g / hw_out : 0u;
                const unsigned px = live ? g - n * hw_out : 0u;
                const int oh = (int)(px / (unsigned)a.Wo), ow = (int)px - oh * a.Wo;
                const int ih0 = oh * a.row_stride - a.pad_t, iw0 = ow * a.stride - a.pad_l;
                const uint8_t *img = in + (size_t)n * a.C * a.H * a.W;
                if (FIRST)
                {
                    // reduction index k = (kh * Fw + kw) * C + c, 16 of them per chunk; the three
                    // counters advance byte by byte
                    const int k0 = q * 32 + half * 16;
                    unsigned wv[4] = {0u, 0u, 0u, 0u};
                    if (live && k0 < kmax)
                    {
                        int kh = k0 / fwc;
                        const int r = k0 - kh * fwc;
                        int kw = r / a.C, c = r - kw * a.C;
#pragma unroll
                        for (int b = 0; b < 16; ++b)
                        {
                            const int ih = ih0 + kh, iw = iw0 + kw;
                            if (kh < a.Fh && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                            {
                                const unsigned v = (unsigned)img[((size_t)ih * a.W + iw) * a.C + c] ^ (flip_a & 0xffu);
                                wv[b >> 2] |= v << (8 * (b & 3));
                            }
                            if (++c == a.C)
                            {
                                c = 0;
                                if (++kw == a.Fw)
                                {
                                    kw = 0;
                                    ++kh;
                                }
                            }
                        }
                    }
                    va[u] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    if (has_b)
                    {
                        const int k = q * 32 + bhalf * 16 + brow;
                        if (k < kmax) // filter [K/16][Fh*Fw*C rows][16]
                        {
                            const uint4 v = *reinterpret_cast<const uint4 *>(
                                filt + (((size_t)(nb * (NT / CB) + bgrp)) * kmax + k) * CB);
                            vb[u] = make_uint4(v.x ^ flip_b, v.y ^ flip_b, v.z ^ flip_b, v.w ^ flip_b);
                        }
                    }
                }
                else
                {
                    const int tap = q / jpairs, j = q - tap * jpairs;
                    const int kh = tap / a.Fw, kw = tap - kh * a.Fw;
                    const int cb = 2 * j + half;
                    const int ih = ih0 + kh, iw = iw0 + kw;
                    if (live && cb < a.cbs && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
                    {
                        const uint4 v = *reinterpret_cast<const uint4 *>(img + (((size_t)cb * a.H + ih) * a.W + iw) * CB);
                        va[u] = make_uint4(v.x ^ flip_a, v.y ^ flip_a, v.z ^ flip_a, v.w ^ flip_a);
                    }
                    const int cbb = 2 * j + bhalf;
                    if (has_b && cbb < a.cbs) // filter [K/16][C/16][Fh][Fw][16 c][16 k]
                    {
                        const uint4 v = *reinterpret_cast<const uint4 *>(
                            filt + ((((size_t)(nb * (NT / CB) + bgrp)) * a.cbs + cbb) * taps + tap) * (CB * CB) +
                            (size_t)brow * CB);
                        vb[u] = make_uint4(v.x ^ flip_b, v.y ^ flip_b, v.z ^ flip_b, v.w ^ flip_b);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < IN_FLIGHT; ++u)
            {
                const unsigned w = w0 + u;
                if (w >= units || !ok)
                    continue;
                const unsigned s = w % STAGES, use = w / STAGES;
                if (use > 0) // every lane waits; the outcome is made the same for the whole warp
                    ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (use - 1) & 1u, status, 32));
                if (ok)
                {
                    uint8_t *st = smem + (size_t)s * G::STAGE;
                    *reinterpret_cast<uint4 *>(st + (size_t)half * TILE_M * CB + (size_t)row * CB) = va[u];
                    if (has_b)
                        *reinterpret_cast<uint4 *>(st + G::A_BYTES + (size_t)bgrp * 2 * CB * CB + (size_t)bhalf * CB * CB +
                                                   (size_t)brow * CB) = vb[u];
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&full_bar[s]);
                }
            }
        }
    }
    else if (lane == 0)
    {
        // ---- MMA issue
        const uint32_t afmt = (!GENERAL && a.zero_in != 0) ? 1u : 0u, bfmt = GENERAL ? 0u : 1u; // 1 = signed bytes
        const uint32_t idesc = make_idesc(2 /*s32*/, afmt, bfmt, 0 /*A K-major*/, 1 /*B MN-major*/, TILE_M, G::NCOLS);
        bool ok = true;
        unsigned consumed = 0;
        int i = 0;
        for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++i)
        {
            const int buf = i & 1;
            if (i >= 2)
                ok = mbar_wait(&acc_empty[buf], ((i >> 1) - 1) & 1, status, 33);
            if (!ok)
                break;
            tc_fence_after_sync();
            for (int q = 0; q < a.steps && ok; ++q, ++consumed)
            {
                const unsigned s = consumed % STAGES;
                ok = mbar_wait(&full_bar[s], (consumed / STAGES) & 1u, status, 34);
                if (!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(smem + (size_t)s * G::STAGE);
                const uint64_t da = make_smem_desc(sa, TILE_M * CB, 8 * CB, 0);
                const uint64_t db = make_smem_desc(sa + G::A_BYTES, 8 * CB, 2 * CB * CB, 0);
                tc_mma_i8(tmem + (uint32_t)(buf * G::NCOLS), da, db, idesc, q > 0 ? 1u : 0u);
                tc_commit(&empty_bar[s]);
            }
            if (ok)
                tc_commit(&acc_full[buf]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == EPI_WARPS + PROD_WARPS)
        tmem_dealloc(tmem, G::TMEM_COLS);
}

template <int NT, bool FIRST, bool GENERAL>
int launch_ring(const RingArgs &a, const uint8_t *in, const uint8_t *filt, const int32_t *bias, uint8_t *out,
                cudaStream_t st)
{
    using G = Geometry<NT, GENERAL>;
    auto kern = conv_u8_ring_kernel<NT, FIRST, GENERAL>;
    const size_t smem = G::RING + (GENERAL ? (size_t)a.Fh * a.Fw * NT * sizeof(int) : 0);
    if (smem > 200 * 1024)
        return -1;
    static PerDeviceOnce configured;
    int dev;
    if (configured.needed(&dev))
    {
        SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured.mark(dev);
    }
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    // CTAs resident per SM: what registers, shared memory and threads allow (the runtime's count) and
    // tensor memory (512 columns).  The grid is TWO such waves: measured on a 16 -> 32 channel 1x1 layer
    // (24x24 pixels, batch 2048) 0.052 ms against 0.066 ms for one wave of CTAs that each walk twice
    // as many tiles -- the second wave's CTAs start as the first ones drain, which evens out the tail.
    int per_sm = 1;
    SB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem));
    if (per_sm > 512 / (int)G::TMEM_COLS) per_sm = 512 / (int)G::TMEM_COLS;
    if (per_sm < 1) per_sm = 1;
    per_sm *= 2;
    long long gx = (long long)num_sms() * per_sm / a.nblocks;
    if (gx < 1)
        gx = 1;
    if (gx > a.tiles)
        gx = a.tiles;
    dim3 grid((unsigned)gx, (unsigned)a.nblocks);
    kern<<<grid, THREADS, smem, st>>>(a, in, filt, bias, out, status);
    return launched("conv_u8_ring_kernel");
}
} // namespace

namespace sb
{
// Returns -1 when the layer is not covered by this kernel, otherwise a SMALL_B200_* code.
int conv2d_u8_ring(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt, const int32_t *bias, uint8_t *out,
                   cudaStream_t st)
{
    if (L->accumulate)
        return -1;
    const bool general = !(L->zero_filt == -128 && (L->zero_in == 0 || L->zero_in == -128));
    if (L->K <= 0 || L->K % CB != 0 || L->C <= 0)
        return -1;
    const bool first = L->C < CB;
    if (!first && L->C % CB != 0)
        return -1;
    if ((!first && reinterpret_cast<uintptr_t>(in) % 16 != 0) || reinterpret_cast<uintptr_t>(filt) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(out) % 16 != 0 || (bias && reinterpret_cast<uintptr_t>(bias) % 16 != 0))
        return -1;
    RingArgs a;
    a.N = L->N; a.H = L->H; a.W = L->W; a.C = L->C; a.K = L->K; a.Fh = L->Fh; a.Fw = L->Fw;
    a.stride = L->stride; a.row_stride = row_stride(L); a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, a.row_stride);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    if (a.N <= 0 || a.Ho <= 0 || a.Wo <= 0)
        return SMALL_B200_OK;
    a.cib = first ? L->C : CB;
    a.cbs = first ? 1 : L->C / CB;
    a.steps = first ? (a.Fh * a.Fw * a.C + 31) / 32 : a.Fh * a.Fw * ((a.cbs + 1) / 2);
    const long long px = (long long)a.N * a.Ho * a.Wo;
    if (px + TILE_M >= 0x7fffffffLL || ((px + TILE_M - 1) / TILE_M) * a.steps >= 0x7fffffffLL)
        return -1; // 32-bit pixel and step counters in the kernel
    a.tiles = (int)((px + TILE_M - 1) / TILE_M);
    a.zero_in = L->zero_in; a.zero_filt = L->zero_filt;
    a.lshift = L->lshift; a.rshift = L->rshift; a.mult = L->multiplier; a.k_zero = L->k_zero;
    const int nt = (L->K % 128 == 0) ? 128 : (L->K % 64 == 0) ? 64 : (L->K % 32 == 0) ? 32 : 16;
    a.nblocks = L->K / nt;
#define SB_RING(NT_)                                                                                                  \
    (first ? (general ? launch_ring<NT_, true, true>(a, in, filt, bias, out, st)                                     \
                      : launch_ring<NT_, true, false>(a, in, filt, bias, out, st))                                   \
           : (general ? launch_ring<NT_, false, true>(a, in, filt, bias, out, st)                                    \
                      : launch_ring<NT_, false, false>(a, in, filt, bias, out, st)))
    switch (nt)
    {
    case 128: return SB_RING(128);
    case 64: return SB_RING(64);
    case 32: return SB_RING(32);
    default: return SB_RING(16);
    }
#undef SB_RING
}
} // namespace sb
