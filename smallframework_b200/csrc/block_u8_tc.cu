// block_u8_tc.cu -- two (or three) uint8 layers of a small-image network as ONE kernel, with the
// intermediate activation kept in shared memory.
//
//   stage 1   a dense layer on the tensor core: a 1x1 convolution (activations arrive by one bulk
//             copy per image) or the one-channel first layer as an im2col GEMM (built in shared
//             memory, see conv_u8_tc.cu).  Its int32 sums are requantised by four epilogue warps
//             and written, as uint8, into shared memory -- never to global memory.
//   stage 2   DW:   a 3x3 stride-1 'same' depthwise convolution of that intermediate, ALSO on the
//                   tensor core: a depthwise tap is a GEMM whose weight matrix is diagonal, and the
//                   tensor pipe is idle anyway while the integer ALUs requantise.  Per tap (kh, kw)
//                   and 32 channels one tcgen05.mma.kind::i8 with M = 128 pixels, N = K = 32 and a
//                   diagonal 32x32 weight block adds  D[p][ch] += X[p + (kh-1)W + (kw-1)][ch] * w[ch].
//                   The shift is only a different start address of the A operand ("linear shift"):
//                   the intermediate is stored three times, once per kernel column kw, each copy
//                   displaced by (1 - kw) pixels and with the image column that would wrap around
//                   to the neighbouring row zeroed, plus W + 1 zero pixels above and below; so tap
//                   (kh, kw) of output pixel p is entry p + kh*W of copy kw for every p, and padded
//                   taps read zeros, which for operands already shifted by their zero points is
//                   the reference's "padded taps are skipped".
//             POOL: the global average pool of the intermediate followed by a dense layer on the
//                   pooled vector (the tail of the keyword-spotting network), on the CUDA cores:
//                   per image it is 64 sums and a 64 x 16 matrix-vector product.
//
// Per-channel constants (bias, k_zero, zero-point terms) also go through the tensor core: both stages
// start their accumulation with one extra MMA whose A operand is a constant tile (31 bytes of 127 and one
// byte of 1 in every row) and whose B operand holds, per output channel, 32 signed digits d_i with
// 127 * (d_0 + ... + d_30) + d_31 = the constant.  The epilogues then need no per-channel value at all
// (four register-only instructions per output); reading 8 bytes of constant per output from shared
// memory instead cost as much shared-memory bandwidth as all the MMA operands together, and shared-memory
// bandwidth is what bounds this kernel.  A constant beyond +-500000 (a bias of that size is possible, the
// biases are data) switches that stage to the shared-memory form; the decision is made once per CTA.
//
// This is the reference's Conv2D_ReLU_DepthwiseConv2D_ReLU fusion
// (include/small/fused_interface_abstract.hpp:1840) for quint8 buffers, where the clamp of the
// requantisation is the ReLU; the reference keeps an intermediate buffer per output tile in
// cache for the same purpose.
//
// Roles: EW (8) warps stage-1 epilogue (thread = pixel = tensor-memory lane, the channel blocks split
// between the two warps of a lane quarter), EW warps stage-2 epilogue, then the bulk-copy producer
// (and owner of the tensor-memory allocation), the MMA issuer of stage 1 and the MMA issuers of stage 2.  A CTA walks over images n = blockIdx.x, + gridDim.x, ...;
// activations, the intermediate and both accumulators are double-buffered, so stage 1 of image
// j + 1 overlaps the stage-1 epilogue of image j and stage 2 of image j - 1.
// Requirements (else the layers run as separate kernels): H*W <= 128; filter zero points -128
// (weights enter the tensor core as signed bytes); zero point of the intermediate 0 or -128.
#include "tc_common.cuh"

namespace
{
using namespace sb;

constexpr int BM = 128;            // pixels per image tile = tensor-memory lanes
// Warps: EW epilogue warps per stage, then the producer, the stage-1 issuer and up to two stage-2 issuers.
__host__ __device__ constexpr int block_threads(int EW) { return (2 * EW + 4) * 32; }

struct Requant
{
    int lshift, rshift, mult, k_zero;
};

struct BlockArgs
{
    int N, H, W, HW;   // images; size of the intermediate (= output of stage 1 = output of a DW stage 2)
    int C;             // stage-1 input channels (1x1 form: multiple of 32; first-layer form: 1)
    int E;             // entries (pixels) per channel block of one shifted copy of the intermediate
    // first-layer form only: the raw image and its window
    int H0, W0, Fh, Fw, stride, pad_t, pad_l, pitch, prow;
    int zero_in1;      // input zero point of stage 1
    int mid_signed;    // 1: the intermediate's zero point is -128 (stored as signed bytes)
    Requant q1, q2;    // stage 1; stage 2 (DW: the depthwise layer, POOL: the average pool)
    // POOL form: the dense layer
    int Kd, zero_pool, zero_in_d, zero_filt_d;
    Requant qd;
};

// Role-uniform give-up: a thread whose bounded wait ran out raises the role's flag; everybody
// looks at it after the role's next named barrier and leaves the image loop together, so nobody
// waits at a barrier for a warp that has left.
struct RoleFlag
{
    int v;
};

// 16 accumulators of one pixel (one channel block) -> 16 output bytes.  in_acc: the per-channel
// constants are already inside the accumulators (they came through the tensor core, see the kernel), so
// the common quantiser is four register-only instructions per output; otherwise they are read from shared
// memory, as seeds of the wide multiply (common.cuh) or, for any other quantiser, as plain addends.
__device__ __forceinline__ uint4 requant16(const uint32_t *r, const int *corr, const long long *seed, const Requant &q,
                                           bool in_acc)
{
    if (requant_is_fast(q.lshift, q.rshift, q.mult))
    {
        const int bit = 1 << (q.rshift - 2), sh1 = q.rshift - 1;
        uint32_t w[4];
        if (in_acc)
        {
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4)
                w[e4] = pack4_sat(requant_seeded_raw((int)r[4 * e4], q.mult, 1ll << 30, bit, sh1),
                                  requant_seeded_raw((int)r[4 * e4 + 1], q.mult, 1ll << 30, bit, sh1),
                                  requant_seeded_raw((int)r[4 * e4 + 2], q.mult, 1ll << 30, bit, sh1),
                                  requant_seeded_raw((int)r[4 * e4 + 3], q.mult, 1ll << 30, bit, sh1));
            return make_uint4(w[0], w[1], w[2], w[3]);
        }
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4)
        {
            int x[4];
#pragma unroll
            for (int e2 = 0; e2 < 2; ++e2)
            {
                const longlong2 sd = *reinterpret_cast<const longlong2 *>(seed + 4 * e4 + 2 * e2);
                x[2 * e2] = requant_seeded_raw((int)r[4 * e4 + 2 * e2], q.mult, sd.x, bit, sh1);
                x[2 * e2 + 1] = requant_seeded_raw((int)r[4 * e4 + 2 * e2 + 1], q.mult, sd.y, bit, sh1);
            }
            w[e4] = pack4_sat(x[0], x[1], x[2], x[3]);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    int v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e)
        v[e] = (int)r[e] + (in_acc ? 0 : corr[e]);
    return requant_pack16(v, q.lshift, q.rshift, q.mult);
}

__device__ __forceinline__ int dp4a_u8_s8(unsigned a, unsigned b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// EW: epilogue warps per stage, 4 or 8.  A warp covers the 32 pixels of tensor-memory lane quarter
// (warp % 4); with 8 warps the channel blocks of an image are split between the two warps of a quarter.
// The epilogues are long chains of dependent integer instructions: what keeps the SM's schedulers busy
// is the number of such warps in flight, so the default is 8 per stage and two CTAs per SM.
template <int K, bool STEM, bool POOL, bool SIGNED_IN, int EW>
__global__ void __launch_bounds__(block_threads(EW), 2)
block_u8_tc_kernel(const BlockArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt1,
                   const int32_t *__restrict__ bias1, const uint8_t *__restrict__ filt2,
                   const int32_t *__restrict__ bias2, uint8_t *__restrict__ out, int *status)
{
    constexpr int KB = K / CB;                       // channel blocks of the intermediate
    constexpr int KCH = 4;                           // first-layer form: 16-byte chunks of the im2col K = 64
    constexpr uint32_t TMEM_COLS = POOL ? (2 * K < 32 ? 32 : 2 * K) : 4 * K;
    constexpr int TAPS = 9;
    constexpr int BLOCK_THREADS = block_threads(EW), EPI_THREADS = EW * 32;
    constexpr int PARTS = EW / 4;                    // warps per lane quarter
    constexpr int CBW = KB / PARTS;                  // channel blocks per epilogue warp
    constexpr int W_PROD = 2 * EW, W_ISS1 = 2 * EW + 1, W_ISS2 = 2 * EW + 2;
    constexpr int PPARTS = EW / KB;                  // POOL: warps that share the pixels of a channel block
    constexpr int DPITCH = K + 4;                    // POOL: bytes per row of the dense filter in shared memory
    static_assert(KB % PARTS == 0 && EW % KB == 0, "epilogue warps must divide the channel blocks");
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t a_full[2], d1_full[2], d1_free[2], p_full[2], p_free[2], d2_full[2], d2_free[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ __align__(16) int corr1[K], corr2[K];         // per-channel constants added to every accumulator
    __shared__ __align__(16) long long seed1[K], seed2[K];  // the same as seeds of the wide multiply (common.cuh)
    __shared__ __align__(16) uint8_t pooled[2][K];
    __shared__ int pool_part[POOL ? PPARTS : 1][K];          // POOL: partial channel sums
    __shared__ __align__(16) uint8_t dense_w[POOL ? 128 * DPITCH : 16]; // POOL: dense filter [k][c] as signed bytes
    __shared__ int dense_c[POOL ? 128 : 1];                  // POOL: per-output constant of the dense layer
    __shared__ RoleFlag failed1, failed2;
    __shared__ int big1, big2; // a stage's constants do not fit the digit form: its epilogue adds them itself

    const int cbs = a.C / CB;
    const uint32_t a_stage = STEM ? (uint32_t)(KCH * BM * CB) : (uint32_t)(a.C * BM);
    const uint32_t b1_bytes = STEM ? (uint32_t)(KCH * K * CB) : (uint32_t)(K * a.C);
    const uint32_t b2_bytes = POOL ? 0u : (uint32_t)(TAPS * (K / 32) * 1024);
    const uint32_t copy_bytes = (uint32_t)(KB * a.E * CB);
    const uint32_t p_stage = (POOL ? 1u : 3u) * copy_bytes;
    uint8_t *sA = smem;                          // [stage][...]
    uint8_t *sB1 = sA + 2 * a_stage;
    uint8_t *sB2 = sB1 + b1_bytes;               // [tap][K/32][2 k-chunks][32 n][16 B], diagonal
    uint8_t *sP = sB2 + b2_bytes;                // [stage][copy kw][cb][entry][16 B]
    uint8_t *sI = sP + 2 * p_stage;              // first-layer form: [stage][prow][pitch] padded image
    const int img_bytes = STEM ? a.prow * a.pitch : 0;
    uint8_t *sOnes = sI + ((2 * img_bytes + 15) & ~15); // [2 chunks][128 rows][16 B]: 127 ... 127 1
    uint8_t *sC1 = sOnes + 2 * BM * CB;          // digits of the stage-1 constants, laid out like sB1 with 32 "input channels"
    uint8_t *sC2 = sC1 + 32 * K;                 // digits of the stage-2 constants: [K/32][2 chunks][32 n][16 B]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int first = blockIdx.x, step = gridDim.x;
    const int count = first < a.N ? (a.N - first + step - 1) / step : 0;

    if (warp == W_PROD)
    {
        if (lane == 0)
        {
            for (int i = 0; i < 2; ++i)
            {
                mbar_init(&a_full[i], STEM ? EW : 1);
                mbar_init(&d1_full[i], 1); mbar_init(&d1_free[i], EW);
                mbar_init(&p_full[i], EW); mbar_init(&p_free[i], POOL ? EW : K / 32);
                mbar_init(&d2_full[i], K / 32); mbar_init(&d2_free[i], EW);
            }
            failed1.v = 0; failed2.v = 0; big1 = 0; big2 = 0;
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, TMEM_COLS);
        tmem_relinquish();
    }
    // ---- operands that stay for the life of the CTA
    if (STEM)
    {
        // filter -> K-major [chunk][n][16 B]: byte k = kh*4 + kw of output channel n, as signed bytes
        for (int i = tid; i < KCH * K * CB; i += BLOCK_THREADS)
        {
            const int b = i % CB, n = (i / CB) % K, j = i / (CB * K);
            const int k = j * CB + b, kh = k >> 2, kw = k & 3;
            uint8_t v = 0;
            if (kh < a.Fh && kw < a.Fw) // filter [K/16][1][Fh][Fw][1][16]
                v = filt1[((((size_t)(n / CB)) * a.Fh + kh) * a.Fw + kw) * CB + (n % CB)] ^ 0x80u;
            sB1[i] = v;
        }
        for (int i = tid; i < (int)(2 * a_stage / 16); i += BLOCK_THREADS) // rows of missing pixels / taps stay zero
            reinterpret_cast<uint4 *>(sA)[i] = make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid; i < 2 * img_bytes / 4; i += BLOCK_THREADS)
            reinterpret_cast<unsigned *>(sI)[i] = 0u;
    }
    else
    {
        // filter slabs [K/16][C/16][16 c][16 k] as they lie in memory, as signed bytes (w - 128)
        const unsigned *src = reinterpret_cast<const unsigned *>(filt1);
        for (int i = tid; i < (int)(b1_bytes / 4); i += BLOCK_THREADS)
            reinterpret_cast<unsigned *>(sB1)[i] = __ldg(src + i) ^ 0x80808080u;
    }
    for (int i = tid; i < (int)((b2_bytes + 2 * p_stage) / 16); i += BLOCK_THREADS) // sB2 and sP are adjacent
        reinterpret_cast<uint4 *>(sB2)[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int i = tid; i < 2 * BM; i += BLOCK_THREADS)
        reinterpret_cast<uint4 *>(sOnes)[i] = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, i < BM ? 0x7f7f7f7fu : 0x017f7f7fu);
    for (int i = tid; i < (32 * K + (POOL ? 0 : (K / 32) * 1024)) / 16; i += BLOCK_THREADS) // sC1 and sC2 are adjacent
        reinterpret_cast<uint4 *>(sC1)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (!POOL)
    {
        // depthwise filter [K/16][3][3][16] -> per tap and 32 channels a diagonal 32 x 32 block, K-major
        for (int i = tid; i < TAPS * K; i += BLOCK_THREADS)
        {
            const int ch = i % K, tap = i / K;
            const uint8_t w = filt2[((size_t)(ch / CB) * TAPS + tap) * CB + (ch % CB)] ^ 0x80u;
            const int c32 = ch & 31;
            sB2[(size_t)(tap * (K / 32) + (ch >> 5)) * 1024 + (c32 >> 4) * 512 + c32 * 16 + (c32 & 15)] = w;
        }
    }
    if (tid < K)
    {
        int c = a.q1.k_zero + (bias1 ? bias1[tid] : 0);
        if (!STEM && a.zero_in1 != 0)
        {
            int wsum = 0; // sum over input channels of (w + zero_filt), from the signed copy
            const int8_t *col = reinterpret_cast<const int8_t *>(sB1) + (size_t)(tid / CB) * cbs * CB * CB + (tid % CB);
            for (int i = 0; i < a.C; ++i)
                wsum += col[i * CB];
            c += a.zero_in1 * wsum;
        }
        corr1[tid] = c;
        seed1[tid] = requant_seed(c, a.q1.mult);
        const int c2 = POOL ? 0 : a.q2.k_zero + (bias2 ? bias2[tid] : 0);
        corr2[tid] = c2;
        seed2[tid] = requant_seed(c2, a.q2.mult);
        if (c / 127 > 31 * 127 || c / 127 < -31 * 127)
            big1 = 1;
        if (c2 / 127 > 31 * 127 || c2 / 127 < -31 * 127)
            big2 = 1;
    }
    __syncthreads();
    if (tid < 2 * K)
    {
        // digits of constant c: 31 digits worth 127 each, one worth 1 (the remainder of c / 127)
        const int n = tid % K, stage2 = tid / K;
        if (!(stage2 ? (POOL || big2) : big1))
        {
            const int c = stage2 ? corr2[n] : corr1[n];
            int rest = c / 127;
            const int last = c - 127 * rest;
            for (int i = 0; i < 32; ++i)
            {
                int d = last;
                if (i < 31)
                {
                    d = rest > 127 ? 127 : (rest < -127 ? -127 : rest);
                    rest -= d;
                }
                uint8_t *dst;
                if (stage2)
                    dst = sC2 + (n >> 5) * 1024 + (i >> 4) * 512 + (n & 31) * CB + (i & 15);
                else if (STEM) // K-major [chunk][n][16 B], like the first-layer filter
                    dst = sC1 + (i >> 4) * K * CB + n * CB + (i & 15);
                else           // MN-major slabs [n / 16][2][16 i][16 n], like the 1x1 filter
                    dst = sC1 + (n >> 4) * 2 * CB * CB + (i >> 4) * CB * CB + (i & 15) * CB + (n & 15);
                *dst = (uint8_t)(int8_t)d;
            }
        }
    }
    if (POOL)
    {
        // dense filter [Kd/16][K/16][16 c][16 k] -> rows [k][c] of signed bytes (w - 128), and per output
        // k_zero + bias + zero_in * sum_c (w - 128)
        for (int i = tid; i < a.Kd * K; i += BLOCK_THREADS)
        {
            const int c = i % K, k = i / K;
            dense_w[k * DPITCH + c] = filt2[((size_t)(k / CB) * KB + c / CB) * CB * CB + (c % CB) * CB + (k % CB)] ^ 0x80u;
        }
        __syncthreads();
        if (tid < a.Kd)
        {
            int wsum = 0;
            for (int c = 0; c < K; ++c)
                wsum += (int)(int8_t)dense_w[tid * DPITCH + c];
            dense_c[tid] = a.qd.k_zero + (bias2 ? bias2[tid] : 0) + a.zero_in_d * wsum;
        }
    }
    fence_proxy_async();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == W_PROD)
    {
        // ---------------- producer (1x1 form): one bulk copy per image ----------------
        if (!STEM && lane == 0)
        {
            const uint32_t bytes = (uint32_t)(a.C * a.HW);
            bool ok = true;
            for (int j = 0; j < count && ok; ++j)
            {
                const int s = j & 1;
                if (j >= 2) // the MMAs that read this stage two images ago are done
                    ok = mbar_wait(&d1_full[s], ((j >> 1) - 1) & 1, status, 31);
                if (!ok)
                    break;
                mbar_expect_tx(&a_full[s], bytes);
                tma_load_1d(sA + (size_t)s * a_stage, in + (size_t)(first + j * step) * bytes, bytes, &a_full[s]);
            }
        }
    }
    else if (warp == W_ISS1)
    {
        // ---------------- MMA issuer, stage 1 ----------------
        // Issuing one tcgen05.mma costs its thread about 150 cycles whatever the size of the MMA
        // (measured here: 20 MMAs of an image took one thread 3000 cycles, with every descriptor
        // precomputed), far longer than these small MMAs occupy the pipe.  So the MMAs of an image
        // are spread over threads: this one issues stage 1, and each block of 32 depthwise channels
        // (its own accumulator columns) has an issuing thread of its own in the warps that follow.
        if (lane == 0)
        {
            const uint32_t idesc1 = STEM ? make_idesc(2, SIGNED_IN ? 1u : 0u, 1, 0, 0, BM, K)
                                         : make_idesc(2, 0 /*u8*/, 1 /*s8*/, 0 /*A K-major*/, 1 /*B MN-major*/, BM, K);
            const uint32_t a16 = a_stage >> 4;
            const uint64_t da1_0 = STEM ? make_smem_desc(smem_u32(sA), BM * CB, 8 * CB, 0)
                                        : make_smem_desc(smem_u32(sA), (uint32_t)(a.HW * CB), 8 * CB, 0);
            const uint64_t db1_0 = STEM ? make_smem_desc(smem_u32(sB1), K * CB, 8 * CB, 0)
                                        : make_smem_desc(smem_u32(sB1), 8 * CB, (uint32_t)(cbs * CB * CB), 0);
            // 32 bytes of K per MMA = two 16-byte chunks of A (first-layer form: 128 rows each; 1x1 form:
            // channel block cb of the image lies HW pixels after block cb - 1, the image being one
            // contiguous run -- lanes >= HW read into the next block, their sums are never used)
            const uint32_t a_step = STEM ? (uint32_t)(2 * BM) : (uint32_t)(2 * a.HW);
            const uint32_t b_step = STEM ? (uint32_t)(2 * K) : (uint32_t)(2 * CB);
            const int n1 = STEM ? KCH / 2 : cbs / 2;
            // the MMA that seeds the accumulators with the per-channel constants (all-zero digits when the
            // stage adds them in its epilogue)
            const uint64_t d_ones = make_smem_desc(smem_u32(sOnes), BM * CB, 8 * CB, 0);
            const uint64_t d_c1 = STEM ? make_smem_desc(smem_u32(sC1), K * CB, 8 * CB, 0)
                                       : make_smem_desc(smem_u32(sC1), 8 * CB, 2 * CB * CB, 0);
            bool ok = true;
            for (int j = 0; j < count && ok; ++j)
            {
                const int s = j & 1;
                ok = mbar_wait(&a_full[s], (j >> 1) & 1, status, 32);
                if (ok && j >= 2)
                    ok = mbar_wait(&d1_free[s], ((j >> 1) - 1) & 1, status, 35);
                if (!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t d1 = tmem + (uint32_t)(s * K);
                const uint64_t da_s = da1_0 + (uint64_t)(s ? a16 : 0u);
                tc_mma_i8(d1, d_ones, d_c1, idesc1, 0u);
                for (int i = 0; i < n1; ++i)
                    tc_mma_i8(d1, da_s + (uint64_t)(i * a_step), db1_0 + (uint64_t)(i * b_step), idesc1, 1u);
                tc_commit(&d1_full[s]);
            }
        }
    }
    else if (warp >= W_ISS2)
    {
        // ---------------- MMA issuers, stage 2: each owns channels 32*c32 .. 32*c32 + 31 ----------------
        const int c32 = warp - W_ISS2;
        if (!POOL && lane == 0 && c32 < K / 32)
        {
            const uint32_t idesc2 = make_idesc(2, a.mid_signed ? 1u : 0u, 1, 0, 0, BM, 32);
            // all descriptor fields are fixed; an operand position is the base descriptor plus a
            // precomputed count of 16-byte units
            const uint64_t db2_0 = make_smem_desc(smem_u32(sB2), 32 * CB, 8 * CB, 0) + (uint64_t)(c32 * 64);
            const uint64_t da2_0 = make_smem_desc(smem_u32(sP), (uint32_t)(a.E * CB), 8 * CB, 0) + (uint64_t)(c32 * 2 * a.E);
            const uint32_t copy16 = copy_bytes >> 4, stage16 = p_stage >> 4;
            uint32_t dA[3][3]; // [kh][kw]: entries of copy kw shifted by kh rows
#pragma unroll
            for (int kh = 0; kh < 3; ++kh)
#pragma unroll
                for (int kw = 0; kw < 3; ++kw)
                    dA[kh][kw] = (uint32_t)kw * copy16 + (uint32_t)(kh * a.W);
            const uint64_t d_ones = make_smem_desc(smem_u32(sOnes), BM * CB, 8 * CB, 0);
            const uint64_t d_c2 = make_smem_desc(smem_u32(sC2) + (uint32_t)(c32 * 1024), 32 * CB, 8 * CB, 0);
            bool ok = true;
            for (int jj = 0; jj < count && ok; ++jj)
            {
                const int t = jj & 1;
                ok = mbar_wait(&p_full[t], (jj >> 1) & 1, status, 33);
                if (ok && jj >= 2)
                    ok = mbar_wait(&d2_free[t], ((jj >> 1) - 1) & 1, status, 34);
                if (!ok)
                    break;
                tc_fence_after_sync();
                const uint64_t da_t = da2_0 + (uint64_t)(t ? stage16 : 0u);
                const uint32_t d = tmem + (uint32_t)(2 * K + t * K + c32 * 32);
                tc_mma_i8(d, d_ones, d_c2, idesc2, 0u);
#pragma unroll
                for (int tap = 0; tap < TAPS; ++tap)
                    tc_mma_i8(d, da_t + (uint64_t)dA[tap / 3][tap % 3], db2_0 + (uint64_t)(tap * (K / 32) * 64), idesc2, 1u);
                tc_commit(&d2_full[t]); // this block's sums are complete ...
                tc_commit(&p_free[t]);  // ... and its reads of the intermediate are done
            }
        }
    }
    else if (warp < EW)
    {
        // ---------------- stage-1 epilogue: requantise into the shifted copies ----------------
        const int quarter = warp & 3, part = warp >> 2;
        const int q = quarter * 32 + lane;         // this thread's pixel = tensor-memory lane
        const int cb0 = part * CBW;                // its channel blocks: cb0 .. cb0 + CBW - 1
        const int cq = q % a.W;
        const bool wraps_left = cq == a.W - 1;     // copy kw = 0 must not show this pixel to the next row
        const bool wraps_right = cq == 0;          // copy kw = 2 must not show it to the previous row
        const uint32_t sx = a.mid_signed ? 0x80808080u : 0u;
        const bool in_acc = big1 == 0;
        bool ok = true;
        // first-layer form: the im2col tile of an image is built by these warps (see conv_u8_tc.cu)
        const int oh = q / a.W, ow = q - oh * a.W;
        auto build = [&](int n, int s) {
            uint8_t *img = sI + (size_t)s * img_bytes;
            const uint8_t *src = in + (size_t)n * a.H0 * a.W0;
            for (int i = tid; i < a.H0 * a.W0; i += EPI_THREADS)
            {
                const int h = i / a.W0, w = i - h * a.W0;
                const uint8_t v = src[i];
                img[(h + a.pad_t) * a.pitch + (w + a.pad_l)] = SIGNED_IN ? (uint8_t)(v ^ 0x80u) : v;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            if (q < a.HW)
            {
                const uint8_t *row = img + (oh * a.stride) * a.pitch + ow * a.stride;
                uint8_t *arow = sA + (size_t)s * a_stage + (size_t)q * CB;
                for (int j4 = part; j4 * 4 < a.Fh; j4 += PARTS) // the warps of a quarter share the pixel's chunks
                {
                    unsigned wv[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                    {
                        const int kh = j4 * 4 + t;
                        if (kh < a.Fh)
                        {
                            const uint8_t *pw = row + kh * a.pitch;
                            const unsigned *al = reinterpret_cast<const unsigned *>(pw - ((size_t)pw & 3));
                            wv[t] = __funnelshift_r(al[0], al[1], 8 * (unsigned)((size_t)pw & 3));
                            if (a.Fw < 4)
                                wv[t] &= (1u << (8 * a.Fw)) - 1u;
                        }
                    }
                    *reinterpret_cast<uint4 *>(arow + (size_t)j4 * BM * CB) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            // one arrival per warp: hundreds of arrivals on one barrier word are serialised by the hardware
            // and were a sizeable part of an image's time
            fence_proxy_async();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&a_full[s]);
        };
        if (STEM && count > 0)
            build(first, 0);
        for (int j = 0; j < count; ++j)
        {
            const int s = j & 1;
            if (STEM)
            {
                // everyone is done with the padded copy of image j - 1 (and agrees on whether to go on)
                if (!ok)
                    *reinterpret_cast<volatile int *>(&failed1.v) = 1;
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (*reinterpret_cast<volatile int *>(&failed1.v))
                    break;
                if (j + 1 < count)
                    build(first + (j + 1) * step, s ^ 1); // stage s^1 was read by the MMAs of image j - 1: waited for below, last turn
            }
            else if (!ok)
                break;
            ok = mbar_wait(&d1_full[s], (j >> 1) & 1, status, 36);
            if (ok && j >= 2)
                ok = mbar_wait(&p_free[s], ((j >> 1) - 1) & 1, status, 37);
            if (!ok)
                continue; // leaves at the top of the loop, together with the other warps
            tc_fence_after_sync();
            // this pixel in the copy for kw = 1 (entry q + W); the DW form keeps it between the other two
            uint8_t *pc = sP + (size_t)s * p_stage + (POOL ? 0u : copy_bytes) + (size_t)(q + a.W) * CB;
            // the load of channel block cb + 1 is in flight while block cb is requantised
            uint32_t ra[16], rb[16];
            const uint32_t d1 = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(s * K + cb0 * CB);
            tmem_ld16(d1, ra);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < CBW; ++i)
            {
                uint32_t *cur = (i & 1) ? rb : ra, *nxt = (i & 1) ? ra : rb;
                const int cb = cb0 + i;
                if (i + 1 < CBW)
                    tmem_ld16(d1 + (uint32_t)((i + 1) * CB), nxt);
                uint4 o = requant16(cur, corr1 + cb * CB, seed1 + cb * CB, a.q1, in_acc);
                o.x ^= sx; o.y ^= sx; o.z ^= sx; o.w ^= sx;
                if (q < a.HW)
                {
                    uint8_t *p1 = pc + (size_t)cb * a.E * CB;
                    *reinterpret_cast<uint4 *>(p1) = o;
                    if (!POOL)
                    {
                        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4 *>(p1 - copy_bytes + CB) = wraps_left ? z : o;   // copy kw = 0, entry q + W + 1
                        *reinterpret_cast<uint4 *>(p1 + copy_bytes - CB) = wraps_right ? z : o;  // copy kw = 2, entry q + W - 1
                    }
                }
                if (i + 1 < CBW)
                    tmem_ld_wait();
            }
            tc_fence_before_sync();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0)
            {
                mbar_arrive(&p_full[s]);
                mbar_arrive(&d1_free[s]);
            }
        }
    }
    else
    {
        // ---------------- stage-2 epilogue ----------------
        const int w2 = warp - EW, quarter = w2 & 3, part = w2 >> 2;
        const int p = quarter * 32 + lane, cb0 = part * CBW;
        const int rt = tid - EPI_THREADS; // thread index inside this role
        const bool in_acc = big2 == 0;
        bool ok = true;
        if (!POOL)
        {
            for (int j = 0; j < count && ok; ++j)
            {
                const int t = j & 1;
                ok = mbar_wait(&d2_full[t], (j >> 1) & 1, status, 38);
                if (!ok)
                    break;
                tc_fence_after_sync();
                uint8_t *o = out + ((size_t)(first + j * step) * KB * a.HW + p) * CB;
                uint32_t ra[16], rb[16];
                const uint32_t d2 = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(2 * K + t * K + cb0 * CB);
                tmem_ld16(d2, ra);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < CBW; ++i)
                {
                    uint32_t *cur = (i & 1) ? rb : ra, *nxt = (i & 1) ? ra : rb;
                    const int cb = cb0 + i;
                    if (i + 1 < CBW)
                        tmem_ld16(d2 + (uint32_t)((i + 1) * CB), nxt);
                    const uint4 ov = requant16(cur, corr2 + cb * CB, seed2 + cb * CB, a.q2, in_acc);
                    if (p < a.HW)
                        *reinterpret_cast<uint4 *>(o + (size_t)cb * a.HW * CB) = ov;
                    if (i + 1 < CBW)
                        tmem_ld_wait();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&d2_free[t]);
            }
        }
        else
        {
            // Warp w2 sums channel block w2 % KB over every PPARTS-th group of 32 pixels.  A lane owns one
            // 32-bit word (four channels) of eight-pixel-strided pixels, so a warp reads 128 contiguous
            // bytes at a time; the eight lanes that share a word add up by three shuffles.
            const int cbp = w2 % KB, ppart = w2 / KB;
            const int quad = lane & 3, pg = lane >> 2;
            for (int j = 0; j < count; ++j)
            {
                const int t = j & 1;
                if (ok)
                    ok = mbar_wait(&p_full[t], (j >> 1) & 1, status, 39);
                if (ok)
                {
                    unsigned s4[4] = {0u, 0u, 0u, 0u};
                    const uint8_t *col = sP + (size_t)t * p_stage + ((size_t)cbp * a.E + a.W) * CB + quad * 4;
                    for (int px = ppart * 8 + pg; px < a.HW; px += PPARTS * 8)
                    {
                        const unsigned wv = *reinterpret_cast<const unsigned *>(col + (size_t)px * CB);
                        s4[0] = __dp4a(wv, 0x00000001u, s4[0]);
                        s4[1] = __dp4a(wv, 0x00000100u, s4[1]);
                        s4[2] = __dp4a(wv, 0x00010000u, s4[2]);
                        s4[3] = __dp4a(wv, 0x01000000u, s4[3]);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e)
#pragma unroll
                        for (int m = 16; m >= 4; m >>= 1)
                            s4[e] += __shfl_xor_sync(0xffffffffu, s4[e], m);
                    if (lane < 4)
                        *reinterpret_cast<int4 *>(&pool_part[ppart][cbp * CB + quad * 4]) =
                            make_int4((int)s4[0], (int)s4[1], (int)s4[2], (int)s4[3]);
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&p_free[t]); // this warp's reads of the intermediate are done
                }
                if (!ok)
                    *reinterpret_cast<volatile int *>(&failed2.v) = 1;
                asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
                if (*reinterpret_cast<volatile int *>(&failed2.v))
                    break;
                if (rt < K)
                {
                    int v = a.q2.k_zero + a.HW * a.zero_pool; // k_zero + sum over the window of (a + zero point)
#pragma unroll
                    for (int pp = 0; pp < PPARTS; ++pp)
                        v += pool_part[pp][rt];
                    pooled[t][rt] = (uint8_t)requant_dev(v, a.q2.lshift, a.q2.rshift, a.q2.mult);
                }
                asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
                // dense layer on the pooled vector: four channels per dp4a (unsigned activations, signed weights)
                if (rt < a.Kd)
                {
                    int acc = dense_c[rt];
                    const unsigned *wrow = reinterpret_cast<const unsigned *>(dense_w + rt * DPITCH);
                    const unsigned *pv = reinterpret_cast<const unsigned *>(pooled[t]);
#pragma unroll
                    for (int c4 = 0; c4 < K / 4; ++c4)
                        acc = dp4a_u8_s8(pv[c4], wrow[c4], acc);
                    out[(size_t)(first + j * step) * a.Kd + rt] =
                        (uint8_t)requant_dev(acc, a.qd.lshift, a.qd.rshift, a.qd.mult);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == W_PROD)
        tmem_dealloc(tmem, TMEM_COLS);
}

bool quant_ok(const small_b200_layer *L)
{
    return L->lshift >= 0 && L->lshift < 32 && L->rshift >= 0 && L->rshift < 32 && row_stride(L) == L->stride;
}

// Fills the arguments of stage 1 and the geometry; false when the pair is not covered.
bool plan_first(const small_b200_layer *c, BlockArgs &a, bool &stem)
{
    if (!c || c->N < 0 || c->K % 32 != 0 || c->K > 64 || c->zero_filt != -128 || !quant_ok(c) || c->accumulate)
        return false;
    a = BlockArgs{};
    a.N = c->N; a.C = c->C;
    a.H = out_dim(c->H, c->pad_t, c->pad_b, c->Fh, c->stride);
    a.W = out_dim(c->W, c->pad_l, c->pad_r, c->Fw, c->stride);
    a.HW = a.H * a.W;
    if (a.HW <= 0 || a.HW > BM)
        return false;
    a.zero_in1 = c->zero_in;
    a.q1 = Requant{c->lshift, c->rshift, c->multiplier, c->k_zero};
    stem = c->C == 1;
    if (stem)
    {
        if (c->Fw > 4 || c->Fh > 16 || (c->zero_in != 0 && c->zero_in != -128) || c->stride < 1)
            return false;
        a.H0 = c->H; a.W0 = c->W; a.Fh = c->Fh; a.Fw = c->Fw; a.stride = c->stride; a.pad_t = c->pad_t; a.pad_l = c->pad_l;
        a.pitch = ((c->W + c->pad_l + c->pad_r + 12) + 3) & ~3; // room for the unaligned window read
        a.prow = c->H + c->pad_t + c->pad_b + 1;
    }
    else
    {
        if (c->Fh != 1 || c->Fw != 1 || c->stride != 1 || c->pad_t || c->pad_b || c->pad_l || c->pad_r)
            return false;
        if (c->C % 32 != 0 || c->C > 128)
            return false;
    }
    a.E = (BM + 2 * a.W + 7) & ~7;
    return true;
}

size_t smem_need(const BlockArgs &a, int K, bool stem, bool pool)
{
    const size_t a_stage = stem ? (size_t)4 * BM * CB : (size_t)a.C * BM;
    const size_t b1 = stem ? (size_t)4 * K * CB : (size_t)K * a.C;
    const size_t b2 = pool ? 0 : (size_t)9 * (K / 32) * 1024;
    const size_t p_stage = (size_t)(pool ? 1 : 3) * (K / CB) * a.E * CB;
    const size_t img = stem ? (size_t)2 * a.prow * a.pitch : 0;
    const size_t consts = (size_t)2 * BM * CB + (size_t)32 * K + (pool ? 0 : (size_t)(K / 32) * 1024);
    return 2 * a_stage + b1 + b2 + 2 * p_stage + ((img + 15) & ~(size_t)15) + consts + 64;
}

template <int K, bool STEM, bool POOL, bool SIGNED_IN, int EW = 8>
int launch_block(const BlockArgs &a, size_t smem, const uint8_t *in, const uint8_t *f1, const int32_t *b1, const uint8_t *f2,
                 const int32_t *b2, uint8_t *out, cudaStream_t st)
{
    auto kern = block_u8_tc_kernel<K, STEM, POOL, SIGNED_IN, EW>;
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
    // CTAs per SM: tensor memory (4K or 2K of 512 columns) and shared memory
    int per_sm = 512 / (POOL ? (2 * K < 32 ? 32 : 2 * K) : 4 * K);
    const int by_smem = (int)((224 * 1024) / (smem + 4096));
    if (per_sm > by_smem) per_sm = by_smem;
    const int by_threads = 2048 / block_threads(EW); // and the register file: 48 registers per thread at EW = 8
    if (per_sm > by_threads) per_sm = by_threads;
    if (per_sm > (EW == 8 ? 2 : 4)) per_sm = (EW == 8 ? 2 : 4);
    if (per_sm < 1) per_sm = 1;
    long long grid = (long long)num_sms() * per_sm;
    if (grid > a.N) grid = a.N;
    kern<<<(unsigned)grid, block_threads(EW), smem, st>>>(a, in, f1, b1, f2, b2, out, status);
    return launched("block_u8_tc_kernel");
}

template <bool POOL>
int dispatch(const BlockArgs &a, int K, bool stem, size_t smem, const uint8_t *in, const uint8_t *f1, const int32_t *b1,
             const uint8_t *f2, const int32_t *b2, uint8_t *out, cudaStream_t st)
{
    const bool sgn = a.zero_in1 != 0;
#define SB_BLOCK_CASE(KK)                                                                                        \
    if (K == KK)                                                                                                 \
    {                                                                                                            \
        if (!stem)                                                                                               \
            return launch_block<KK, false, POOL, false>(a, smem, in, f1, b1, f2, b2, out, st);                   \
        return sgn ? launch_block<KK, true, POOL, true>(a, smem, in, f1, b1, f2, b2, out, st)                    \
                   : launch_block<KK, true, POOL, false>(a, smem, in, f1, b1, f2, b2, out, st);                  \
    }
    SB_BLOCK_CASE(32)
    SB_BLOCK_CASE(64)
#undef SB_BLOCK_CASE
    return fail(SMALL_B200_INVALID_ARGUMENT, "fused uint8 block: channel count not covered");
}

bool plan_dw(const small_b200_layer *c, const small_b200_layer *d, BlockArgs &a, bool &stem)
{
    if (!plan_first(c, a, stem) || !d)
        return false;
    if (d->C != c->K || d->H != a.H || d->W != a.W || d->N != c->N || d->Fh != 3 || d->Fw != 3 || d->stride != 1 ||
        d->pad_t != 1 || d->pad_b != 1 || d->pad_l != 1 || d->pad_r != 1 || d->accumulate || !quant_ok(d))
        return false;
    if (d->zero_filt != -128 || (d->zero_in != 0 && d->zero_in != -128))
        return false;
    a.mid_signed = d->zero_in != 0;
    a.q2 = Requant{d->lshift, d->rshift, d->multiplier, d->k_zero};
    return smem_need(a, c->K, stem, false) <= 200 * 1024;
}

bool plan_pool(const small_b200_layer *c, const small_b200_layer *pl, const small_b200_layer *dn, BlockArgs &a, bool &stem)
{
    if (!plan_first(c, a, stem) || !pl || !dn)
        return false;
    if (pl->C != c->K || pl->H != a.H || pl->W != a.W || pl->Fh != a.H || pl->Fw != a.W || pl->pad_t || pl->pad_b ||
        pl->pad_l || pl->pad_r || pl->N != c->N || !quant_ok(pl))
        return false;
    if (dn->C != c->K || dn->H != 1 || dn->W != 1 || dn->Fh != 1 || dn->Fw != 1 || dn->stride != 1 || dn->pad_t ||
        dn->pad_b || dn->pad_l || dn->pad_r || dn->K % CB != 0 || dn->K <= 0 || dn->K > 128 || dn->N != c->N ||
        dn->accumulate || !quant_ok(dn) || dn->zero_filt != -128)
        return false;
    a.mid_signed = 0;
    a.zero_pool = pl->zero_in;
    a.q2 = Requant{pl->lshift, pl->rshift, pl->multiplier, pl->k_zero};
    a.Kd = dn->K; a.zero_in_d = dn->zero_in; a.zero_filt_d = dn->zero_filt;
    a.qd = Requant{dn->lshift, dn->rshift, dn->multiplier, dn->k_zero};
    return smem_need(a, c->K, stem, true) <= 200 * 1024;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
} // namespace

extern "C"
{
int small_b200_conv2d_dwconv2d_u8_supported(const small_b200_layer *conv, const small_b200_layer *dw)
{
    BlockArgs a;
    bool stem;
    return plan_dw(conv, dw, a, stem) ? 1 : 0;
}

int small_b200_conv2d_dwconv2d_u8(const small_b200_layer *conv, const small_b200_layer *dw, const uint8_t *in,
                                  const uint8_t *conv_filt, const int32_t *conv_bias, const uint8_t *dw_filt,
                                  const int32_t *dw_bias, uint8_t *out, void *stream)
{
    BlockArgs a;
    bool stem;
    if (!plan_dw(conv, dw, a, stem))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D_DepthwiseConv2D<quint8> ERROR: this pair of layers is not covered by the "
                                                 "one-kernel form; call the two layers separately.");
    if (a.N == 0)
        return SMALL_B200_OK;
    if (!aligned16(in) || !aligned16(out) || !aligned16(conv_filt))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D_DepthwiseConv2D<quint8> ERROR: buffers must be 16-byte aligned.");
    return dispatch<false>(a, conv->K, stem, smem_need(a, conv->K, stem, false), in, conv_filt, conv_bias, dw_filt, dw_bias, out,
                           as_stream(stream));
}

int small_b200_conv2d_avgpool_dense_u8_supported(const small_b200_layer *conv, const small_b200_layer *pool,
                                                 const small_b200_layer *dense)
{
    BlockArgs a;
    bool stem;
    return plan_pool(conv, pool, dense, a, stem) ? 1 : 0;
}

int small_b200_conv2d_avgpool_dense_u8(const small_b200_layer *conv, const small_b200_layer *pool,
                                       const small_b200_layer *dense, const uint8_t *in, const uint8_t *conv_filt,
                                       const int32_t *conv_bias, const uint8_t *dense_filt, const int32_t *dense_bias,
                                       uint8_t *out, void *stream)
{
    BlockArgs a;
    bool stem;
    if (!plan_pool(conv, pool, dense, a, stem))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D_AveragePool2D_Dense<quint8> ERROR: these layers are not covered by the "
                                                 "one-kernel form; call them separately.");
    if (a.N == 0)
        return SMALL_B200_OK;
    if (!aligned16(in) || !aligned16(conv_filt))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D_AveragePool2D_Dense<quint8> ERROR: buffers must be 16-byte aligned.");
    return dispatch<true>(a, conv->K, stem, smem_need(a, conv->K, stem, true), in, conv_filt, conv_bias, dense_filt, dense_bias, out,
                          as_stream(stream));
}
} // extern "C"
