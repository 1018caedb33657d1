// conv_tf32x3.cu -- fp32 dense convolution (stride 1) on the 5th-generation tensor cores with
// the 3xTF32 split: every fp32 operand x is fed as hi = x (the tensor core ignores the low 13
// mantissa bits) and lo = x - trunc_tf32(x) (exact in fp32), and each product is accumulated as
// a_lo*b_hi + a_hi*b_lo + a_hi*b_hi in fp32 tensor memory.  The dropped a_lo*b_lo term is
// 2^-22 relative, so the result stays within the 1e-5 gate against the reference's fp32 loop
// nest (include/small/abstract_layer.hpp:1368-1823, FLOAT_CONV_TILE_C).
//
// Implicit GEMM without im2col ("linear shift"):
//   For one image and one block of 16 input channels, TMA copies a patch of the packed
//   activations [rows][PW columns][16 ch] into shared memory split into four 16-byte channel
//   chunks: [chunk][row][col][4 floats].  PW = W + max(pad_l, pad_r): the zero column(s) that
//   TMA's out-of-bounds fill produces at the left edge of every row also serve as the right
//   padding of the row above.  Output pixel (r, c) is GEMM row m = r*PW + c, and filter tap
//   (kh, kw) of that pixel sits at patch entry m + kh*PW + kw.  Consecutive GEMM rows are
//   consecutive 16-byte entries, i.e. 8 rows = one 128-byte core matrix of the K-major
//   no-swizzle canonical layout, for EVERY tap: a tap only moves the descriptor's start
//   address.  Rows with c >= Wo are junk and are not stored.
//   The filter [K/16][C/16][tap][16 c][16 k] has the output channel contiguous (MN-major).
//   kind::tf32 did not accept an MN-major no-swizzle B operand on this hardware (a one-MMA
//   experiment returned zeros, while the K-major form was exact), so the filter is re-laid
//   once per set of weights into [K/NT][C/16][tap][c/4][NT k][4 c] (prepare_filter_kernel,
//   which also produces the lo copy), NT = output channels per CTA.  One tap of one CTA is
//   then a single contiguous run of NT*64 bytes that IS the K-major no-swizzle canonical
//   layout ([c/4][k][4 c], like the activations) and arrives by one bulk copy.
//
// The lo parts are produced outside this kernel into caller-provided scratch: the filter once
// per set of weights (prepare), the activations once per call (split_tf32_kernel).
#include "tc_common.cuh"

namespace
{
using namespace sb;

constexpr int MAX_MT = 4;  // accumulator tiles per CTA
constexpr int B_STAGES = 4;
constexpr int A_SLOTS_MAX = 4;

struct TcArgs
{
    int N, C, K, H, W, Ho, Wo, Fh, Fw, pad_t, pad_l;
    int cbs, taps;
    int PW, PR;          // patch width / rows
    int MT;              // GEMM rows per CTA
    int n_mtiles;        // accumulator tiles: 128-row tiles then an optional 64-row tile
    int mtile_rows[MAX_MT];
    int m_tiles_per_img; // CTAs along M per image
    int NT;              // output channels per CTA
    int n_tiles;         // K / NT
    int a_slots;         // activation patches in flight (1..4)
    int group;           // filter taps summed in tensor memory before a flush (1 or Fw)
    int accumulate, act;
    float slope;
};

__global__ void __launch_bounds__(256)
split_tf32_kernel(long long n4, const float4 *__restrict__ x, float4 *__restrict__ lo)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
    {
        const float4 v = x[i];
        float4 r;
        r.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
        r.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
        r.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
        r.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
        lo[i] = r;
    }
}

// Output channels per CTA, a function of K alone so that filter preparation and the
// convolution agree: two tensor-memory buffers x two accumulator tiles x NT columns must fit
// the 512 columns, and a thread keeps 64 columns of each tile in registers.
__host__ __device__ inline int pick_nt(int K)
{
    return (K % 128 == 0) ? 128 : (K % 64 == 0) ? 64 : (K % 32 == 0) ? 32 : 16;
}

// packed filter [K/16][slab][16 c][16 k] -> hi and lo copies in [K/NT][slab][c/4][NT k][4 c]
__global__ void __launch_bounds__(256)
prepare_filter_kernel(long long n, int slabs, int NT, const float *__restrict__ w, float *__restrict__ hi,
                      float *__restrict__ lo)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int k16 = (int)(i & 15), c = (int)((i >> 4) & 15);
    const long long t = i >> 8;            // kb16 * slabs + slab
    const int slab = (int)(t % slabs);
    const int k = (int)(t / slabs) * 16 + k16;
    const float v = w[i];
    const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    const long long o = (((long long)(k / NT) * slabs + slab) * 4 + (c >> 2)) * NT * 4 + (long long)(k % NT) * 4 + (c & 3);
    hi[o] = v;
    lo[o] = v - h;
}

// Tensor-core accumulation truncates: every MMA adds into the fp32 accumulator with
// round-toward-zero, a one-sided error that grows with the number of accumulations (measured
// here: 3e-5 of the output range after 1700 MMAs).  So tensor memory only ever holds the sum
// of ONE filter tap (6 MMAs per accumulator tile); eight accumulation warps pull each tap's
// partial sums out with tcgen05.ld and add them into fp32 registers with round-to-nearest,
// while the tensor core already works on the next tap in the second half of tensor memory.
//
// warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: accumulation + epilogue (lane quarter
// = warp % 4, column half = (warp - 2) / 4)
constexpr int ACC_WARPS = 8;
constexpr int MAX_NT = 128;        // output channels per CTA
constexpr int COLS_PER_THREAD = 64; // of one accumulator tile

__global__ void __launch_bounds__(320, 1)
conv_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                   const float *__restrict__ filt_hi, const float *__restrict__ filt_lo,
                   const TcArgs a, const float *__restrict__ bias, float *__restrict__ out, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t a_full[A_SLOTS_MAX], a_empty[A_SLOTS_MAX], b_full[B_STAGES], b_empty[B_STAGES];
    __shared__ __align__(8) uint64_t t_full[2], t_empty[2];
    __shared__ uint32_t tmem_base_s;

    const uint32_t a_bytes = (uint32_t)a.PR * a.PW * 64;      // bytes of one hi (or lo) patch
    const uint32_t a_part = (a_bytes + 127u) & ~127u;         // its 128-byte aligned footprint
    const uint32_t a_chunk = (uint32_t)a.PR * a.PW * 16;      // bytes between channel chunks
    const uint32_t b_part = (uint32_t)a.NT * 64;              // bytes of one hi (or lo) tap tile
    const uint32_t b_chunk = (uint32_t)a.NT * 16;             // bytes between 4-channel chunks
    uint8_t *sA = smem;                                        // [slot][hi|lo][chunk][PR][PW][16 B]
    uint8_t *sB = smem + (size_t)a.a_slots * 2 * a_part;      // [stage][hi|lo][c/4][NT k][16 B]

    int bid = blockIdx.x;
    const int nt = bid % a.n_tiles; bid /= a.n_tiles;
    const int mt = bid % a.m_tiles_per_img;
    const int n = bid / a.m_tiles_per_img;
    const int m0 = mt * a.MT;
    const int r_first = m0 / a.PW;
    const int m_local0 = m0 - r_first * a.PW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int buf_cols = a.n_mtiles * a.NT; // columns of one tensor-memory buffer
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * buf_cols)
        tmem_cols <<= 1;

    if (warp == 0)
    {
        if (lane == 0)
        {
            for (int i = 0; i < A_SLOTS_MAX; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
            for (int i = 0; i < 2; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], ACC_WARPS); }
            for (int i = 0; i < B_STAGES; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    const int steps = a.cbs * a.taps;

    if (warp == 0 && lane == 0)
    {
        // ---------------- producer ----------------
        bool ok = true;
        int bs = 0;
        for (int cb = 0; cb < a.cbs && ok; ++cb)
        {
            const int slot = cb % a.a_slots;
            const int use = cb / a.a_slots;
            if (use > 0)
                ok = mbar_wait(&a_empty[slot], (use - 1) & 1, status, 11);
            if (!ok)
                break;
            uint8_t *dst = sA + (size_t)slot * 2 * a_part;
            mbar_expect_tx(&a_full[slot], 2 * a_bytes);
            tma_load_5d(dst, &map_a_hi, 0, -a.pad_l, r_first - a.pad_t, 0, n * a.cbs + cb, &a_full[slot]);
            tma_load_5d(dst + a_part, &map_a_lo, 0, -a.pad_l, r_first - a.pad_t, 0, n * a.cbs + cb, &a_full[slot]);
            for (int tap = 0; tap < a.taps && ok; ++tap, ++bs)
            {
                const int st = bs % B_STAGES, buse = bs / B_STAGES;
                if (buse > 0)
                    ok = mbar_wait(&b_empty[st], (buse - 1) & 1, status, 12);
                if (!ok)
                    break;
                uint8_t *bd = sB + (size_t)st * 2 * b_part;
                mbar_expect_tx(&b_full[st], 2 * b_part);
                const size_t off = ((size_t)nt * steps + (size_t)(cb * a.taps + tap)) * (b_part / 4);
                tma_load_1d(bd, filt_hi + off, b_part, &b_full[st]);
                tma_load_1d(bd + b_part, filt_lo + off, b_part, &b_full[st]);
            }
        }
    }
    else if (warp == 1 && lane == 0)
    {
        // ---------------- MMA issuer ----------------
        // One thread feeds the tensor core, so the per-MMA instruction count matters: all
        // descriptor fields except the 16-byte-granular start address are fixed per CTA, and
        // a new operand position is one 64-bit add on a precomputed descriptor.
        bool ok = true;
        int bs = 0;
        const uint64_t a_desc0 = make_smem_desc(smem_u32(sA), a_chunk, 128, 0);
        const uint64_t b_desc0 = make_smem_desc(smem_u32(sB), b_chunk, 128, 0);
        const uint32_t idesc0 = make_idesc(1 /*f32*/, 2 /*tf32*/, 2 /*tf32*/, 0 /*A K-major*/, 0 /*B K-major*/,
                                           (uint32_t)a.mtile_rows[0], (uint32_t)a.NT);
        const uint32_t idesc1 = make_idesc(1, 2, 2, 0, 0, (uint32_t)(a.n_mtiles > 1 ? a.mtile_rows[1] : 128),
                                           (uint32_t)a.NT);
        const uint64_t a_lo_off = a_part >> 4, b_lo_off = b_part >> 4;
        const uint64_t a_half = (2 * a_chunk) >> 4, b_half = (2 * b_chunk) >> 4;
        const uint64_t a_tile1 = (uint64_t)a.mtile_rows[0];          // rows of tile 0 = 16-byte entries
        const bool two_tiles = a.n_mtiles > 1;
        for (int cb = 0; cb < a.cbs && ok; ++cb)
        {
            const int slot = cb % a.a_slots;
            ok = mbar_wait(&a_full[slot], (cb / a.a_slots) & 1, status, 13);
            if (!ok)
                break;
            const uint64_t a_slot = a_desc0 + ((uint64_t)(slot * 2 * a_part) >> 4) + (uint64_t)m_local0;
            int kh = 0, kw = 0;
            for (int tap = 0; tap < a.taps && ok; ++tap, ++bs)
            {
                const int st = bs % B_STAGES;
                const int chunk = bs / a.group, in_chunk = bs - chunk * a.group;
                const int tb = chunk & 1; // tensor-memory buffer of this group of taps
                ok = mbar_wait(&b_full[st], (bs / B_STAGES) & 1, status, 14);
                if (ok && in_chunk == 0 && chunk >= 2)
                    ok = mbar_wait(&t_empty[tb], ((chunk >> 1) - 1) & 1, status, 16);
                if (!ok)
                    break;
                tc_fence_after_sync();
                const uint64_t ah = a_slot + (uint64_t)(kh * a.PW + kw), al = ah + a_lo_off;
                const uint64_t bh = b_desc0 + ((uint64_t)(st * 2 * b_part) >> 4), bl = bh + b_lo_off;
                const uint32_t d0 = tmem + (uint32_t)(tb * buf_cols), d1 = d0 + (uint32_t)a.NT;
                const uint32_t fresh = in_chunk == 0 ? 0u : 1u;
                // tile 0
                tc_mma_tf32(d0, al, bh, idesc0, fresh);
                tc_mma_tf32(d0, ah, bl, idesc0, 1u);
                tc_mma_tf32(d0, ah, bh, idesc0, 1u);
                tc_mma_tf32(d0, al + a_half, bh + b_half, idesc0, 1u);
                tc_mma_tf32(d0, ah + a_half, bl + b_half, idesc0, 1u);
                tc_mma_tf32(d0, ah + a_half, bh + b_half, idesc0, 1u);
                if (two_tiles)
                {
                    const uint64_t ah1 = ah + a_tile1, al1 = al + a_tile1;
                    tc_mma_tf32(d1, al1, bh, idesc1, fresh);
                    tc_mma_tf32(d1, ah1, bl, idesc1, 1u);
                    tc_mma_tf32(d1, ah1, bh, idesc1, 1u);
                    tc_mma_tf32(d1, al1 + a_half, bh + b_half, idesc1, 1u);
                    tc_mma_tf32(d1, ah1 + a_half, bl + b_half, idesc1, 1u);
                    tc_mma_tf32(d1, ah1 + a_half, bh + b_half, idesc1, 1u);
                }
                tc_commit(&b_empty[st]); // the tap's filter tile is free once these MMAs retire
                if (in_chunk == a.group - 1)
                    tc_commit(&t_full[tb]); // the group's partial sums are complete
                if (tap == a.taps - 1)
                    tc_commit(&a_empty[slot]);
                if (++kw == a.Fw) { kw = 0; ++kh; }
            }
        }
    }
    else if (warp >= 2)
    {
        // ---------------- accumulation + epilogue ----------------
        const int quarter = warp & 3;          // TMEM lanes [32*quarter, 32*quarter+32)
        const int chalf = (warp - 2) >> 2;     // which half of the tile's columns
        const int my_cols = (a.NT >= 32) ? a.NT / 2 : a.NT;
        const bool active = (a.NT >= 32) || chalf == 0;
        const int col0 = chalf * my_cols;      // first column inside a tile (0 when NT < 32)
        float acc[2][COLS_PER_THREAD];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < COLS_PER_THREAD; ++c)
                acc[j][c] = 0.f;
        bool ok = true;
        for (int g = 0; g < steps / a.group && ok; ++g)
        {
            const int tb = g & 1;
            ok = mbar_wait(&t_full[tb], (g >> 1) & 1, status, 15, 1u << 24);
            if (!ok)
                break;
            tc_fence_after_sync();
            if (active)
            {
                // four pieces of 32 columns (2 tiles x 2); a tile's two loads are in flight
                // together, so a flush costs two tensor-memory round trips
                const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(tb * buf_cols + col0);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                {
                    if (j < a.n_mtiles)
                    {
                        uint32_t v0[32], v1[32];
                        if (my_cols >= 64)
                        {
                            tmem_ld32(tbase + (uint32_t)(j * a.NT), v0);
                            tmem_ld32(tbase + (uint32_t)(j * a.NT + 32), v1);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                            {
                                acc[j][e] += __uint_as_float(v0[e]);
                                acc[j][32 + e] += __uint_as_float(v1[e]);
                            }
                        }
                        else if (my_cols == 32)
                        {
                            tmem_ld32(tbase + (uint32_t)(j * a.NT), v0);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                acc[j][e] += __uint_as_float(v0[e]);
                        }
                        else
                        {
                            tmem_ld16(tbase + (uint32_t)(j * a.NT), v0);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                acc[j][e] += __uint_as_float(v0[e]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&t_empty[tb]);
        }
        if (ok && active)
        {
            int row_off = 0;
#pragma unroll
            for (int j = 0; j < 2; ++j)
            {
                if (j < a.n_mtiles)
                {
                    const int rows = a.mtile_rows[j];
                    // 128-row tile: lane l of quarter q holds row 32q + l; 64-row tile: rows
                    // 16q + l in lanes 0..15 of each quarter
                    const int trow = (rows == 128) ? quarter * 32 + lane : quarter * 16 + lane;
                    const bool lane_has_row = (rows == 128) || (lane < 16);
                    const int m = m0 + row_off + trow;
                    const int r = m / a.PW, c = m - r * a.PW;
                    const bool valid = lane_has_row && r < a.Ho && c < a.Wo;
#pragma unroll
                    for (int cg = 0; cg < COLS_PER_THREAD / 16; ++cg)
                    {
                        if (valid && cg * 16 < my_cols)
                        {
                            const int kg = nt * a.NT + col0 + cg * 16;
                            float *o = out + ((((size_t)n * (a.K / CB) + kg / CB) * a.Ho + r) * a.Wo + c) * CB;
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                            {
                                float4 x;
                                x.x = acc[j][cg * 16 + q * 4 + 0]; x.y = acc[j][cg * 16 + q * 4 + 1];
                                x.z = acc[j][cg * 16 + q * 4 + 2]; x.w = acc[j][cg * 16 + q * 4 + 3];
                                if (a.accumulate)
                                {
                                    const float4 s = *reinterpret_cast<const float4 *>(o + q * 4);
                                    x.x += s.x; x.y += s.y; x.z += s.z; x.w += s.w;
                                }
                                if (bias)
                                {
                                    const float4 b = *reinterpret_cast<const float4 *>(bias + kg + q * 4);
                                    x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
                                }
                                x.x = apply_act(x.x, a.act, a.slope); x.y = apply_act(x.y, a.act, a.slope);
                                x.z = apply_act(x.z, a.act, a.slope); x.w = apply_act(x.w, a.act, a.slope);
                                *reinterpret_cast<float4 *>(o + q * 4) = x;
                            }
                        }
                    }
                    row_off += rows;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0)
        tmem_dealloc(tmem, tmem_cols);
}
} // namespace

extern "C"
{
int small_b200_split_tf32(int64_t n, const float *x, float *lo, void *stream)
{
    if (n < 0 || n % 4 != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "split_tf32 ERROR: element count must be a multiple of 4.");
    if (n == 0)
        return SMALL_B200_OK;
    long long blocks = (n / 4 + 255) / 256;
    const long long cap = (long long)num_sms() * 16;
    if (blocks > cap)
        blocks = cap;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(n / 4, (const float4 *)x, (float4 *)lo);
    return launched("split_tf32_kernel");
}

int small_b200_conv2d_f32_tf32x3_supported(const small_b200_layer *L)
{
    if (!L || L->stride != 1 || L->C % CB != 0 || L->K % CB != 0 || L->C <= 0 || L->K <= 0)
        return 0;
    const int PW = L->W + (L->pad_l > L->pad_r ? L->pad_l : L->pad_r);
    return (PW <= 256 && L->Fw <= 16 && L->Fh <= 16) ? 1 : 0;
}

int small_b200_filter_prepare_tf32x3(const small_b200_layer *L, const float *filt, float *prepared, void *stream)
{
    if (!small_b200_conv2d_f32_tf32x3_supported(L))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: shape not covered by the tensor-core path.");
    const long long n = (long long)L->K * L->C * L->Fh * L->Fw;
    prepare_filter_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
        n, (L->C / CB) * L->Fh * L->Fw, pick_nt(L->K), filt, prepared, prepared + n);
    return launched("prepare_filter_kernel");
}

int small_b200_conv2d_f32_tf32x3(const small_b200_layer *L, const float *in, const float *in_lo,
                                 const float *filt_prepared, const float *bias, float *out, void *stream)
{
    const float *filt = filt_prepared;
    const float *filt_lo = filt_prepared ? filt_prepared + (size_t)L->K * L->C * L->Fh * L->Fw : nullptr;
    if (int rc = check_window_layer(L, "Conv2D<float>", true, 2))
        return rc;
    if (!small_b200_conv2d_f32_tf32x3_supported(L))
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: shape not covered by the tensor-core path.");
    TcArgs a{};
    a.N = L->N; a.C = L->C; a.K = L->K; a.H = L->H; a.W = L->W; a.Fh = L->Fh; a.Fw = L->Fw;
    a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, 1);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, 1);
    a.cbs = L->C / CB; a.taps = L->Fh * L->Fw;
    a.accumulate = L->accumulate; a.act = L->act; a.slope = L->slope;
    if (a.N == 0 || a.Ho == 0 || a.Wo == 0)
        return SMALL_B200_OK;
    a.PW = L->W + (L->pad_l > L->pad_r ? L->pad_l : L->pad_r);

    a.NT = pick_nt(a.K);
    a.group = a.Fw; // one kernel row per flush: taps = Fh * Fw is a multiple of it
    // GEMM rows of one image: the last valid row is (Ho-1)*PW + Wo-1
    const int m_img = (a.Ho - 1) * a.PW + a.Wo;
    const int MT = (m_img <= 128) ? 128 : (m_img <= 192) ? 192 : 256;
    a.MT = MT;
    a.n_mtiles = 0;
    for (int left = MT; left > 0;)
    {
        const int rows = left >= 128 ? 128 : 64;
        a.mtile_rows[a.n_mtiles++] = rows;
        left -= rows;
    }
    a.m_tiles_per_img = (m_img + MT - 1) / MT;
    a.n_tiles = a.K / a.NT;
    const int need = (a.PW - 1) + MT + (a.Fh - 1) * a.PW + (a.Fw - 1) + 1;
    a.PR = (need + a.PW - 1) / a.PW;
    if (a.PR > 256)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: patch too tall.");
    const size_t a_part = (((size_t)a.PR * a.PW * 64) + 127) & ~(size_t)127, b_part = (size_t)a.NT * 64;
    const size_t limit = 220 * 1024;
    // as many activation slots as fit (a layer with few taps per channel block, e.g. 1x1,
    // needs several patches in flight to cover the TMA latency)
    size_t smem = 0;
    for (a.a_slots = (a.cbs < A_SLOTS_MAX ? (a.cbs > 0 ? a.cbs : 1) : A_SLOTS_MAX); a.a_slots >= 1; --a.a_slots)
    {
        smem = (size_t)a.a_slots * 2 * a_part + (size_t)B_STAGES * 2 * b_part;
        if (smem <= limit)
            break;
    }
    if (a.a_slots < 1)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: patch does not fit in shared memory.");

    CUtensorMap ma_hi, ma_lo;
    {
        // activations [N*cbs][H][W][4 chunks][4 floats]
        const uint64_t dims[5] = {4, (uint64_t)a.W, (uint64_t)a.H, 4, (uint64_t)a.N * a.cbs};
        const uint64_t strides[4] = {64, (uint64_t)a.W * 64, 16, (uint64_t)a.H * a.W * 64};
        const uint32_t box[5] = {4, (uint32_t)a.PW, (uint32_t)a.PR, 4, 1};
        if (int rc = make_tensor_map(&ma_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, in, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return rc;
        if (int rc = make_tensor_map(&ma_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, in_lo, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return rc;
    }
    static bool configured = false;
    if (!configured)
    {
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        configured = true;
    }
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    const long long blocks = (long long)a.N * a.m_tiles_per_img * a.n_tiles;
    conv_tf32x3_kernel<<<(unsigned)blocks, 320, smem, as_stream(stream)>>>(ma_hi, ma_lo, filt, filt_lo, a, bias, out, status);
    return launched("conv_tf32x3_kernel");
}
} // extern "C"

// ---------------------------------------------------------------------------------------------
// The same tensor-core convolution for callers that must not allocate device memory.
//
// small_b200_conv2d_f32_tf32x3 needs two pieces of scratch from its caller: the lo half of the
// activations and the re-laid filter.  Some callers cannot provide them: code that runs inside
// a region where cudaMalloc is forbidden or would synchronise the device (a real-time loop, a
// plug-in that only ever receives its input and output pointers, a host that has handed all of
// its device memory to another allocator).  For them the scratch lives in this fixed array
// inside the library image.  Every GPU that loads the library carries these 16 MiB until the
// process exits, which is why the limit is modest.
constexpr size_t STATIC_SCRATCH_FLOATS = (size_t)4 << 20; // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_FLOATS];

namespace
{
// In host code `g_static_scratch` is only a stand-in for the device symbol, not an address a
// kernel could use; the device address is looked up once per device, with that device current.
int static_scratch_ptr(float **ptr)
{
    static float *ptrs[64] = {nullptr};
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64)
        return fail(SMALL_B200_CUDA_ERROR, "device index out of range for the static scratch table");
    if (!ptrs[dev])
    {
        float *p = nullptr;
        SB_CUDA(cudaGetSymbolAddress((void **)&p, g_static_scratch));
        ptrs[dev] = p;
    }
    *ptr = ptrs[dev];
    return SMALL_B200_OK;
}
} // namespace

extern "C" int small_b200_conv2d_f32_tf32x3_noalloc(const small_b200_layer *L, const float *in,
                                                    const float *filt, const float *bias, float *out,
                                                    void *stream)
{
    if (int rc = check_window_layer(L, "Conv2D<float>", true, 2))
        return rc;
    if (!small_b200_conv2d_f32_tf32x3_supported(L))
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "Conv2D<float> (3xTF32, no-alloc) ERROR: shape not covered by the tensor-core path.");
    const size_t in_elems = (size_t)L->N * L->C * L->H * L->W;
    const size_t filt_elems = (size_t)L->K * L->C * L->Fh * L->Fw;
    // lo half of the input (rounded up so the filter copies stay 256-byte aligned), then the
    // re-laid filter and its lo copy
    const size_t in_slot = (in_elems + 63) & ~(size_t)63;
    const size_t need = in_slot + 2 * filt_elems;
    if (need > STATIC_SCRATCH_FLOATS)
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "Conv2D<float> (3xTF32, no-alloc) ERROR: this call needs " + std::to_string(need * 4) +
                        " bytes of scratch (input elements + 2 x filter elements, 4 bytes each) but the "
                        "built-in scratch holds " + std::to_string(STATIC_SCRATCH_FLOATS * 4) +
                        " bytes; use small_b200_conv2d_f32_tf32x3 with caller-provided scratch.");
    float *scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch))
        return rc;
    float *in_lo = scratch, *prepared = scratch + in_slot;
    // Nothing in the scratch has to start from zero: both regions are completely rewritten for
    // the sizes of this call before the convolution reads them.
    if (int rc = small_b200_split_tf32((int64_t)in_elems, in, in_lo, stream))
        return rc;
    if (int rc = small_b200_filter_prepare_tf32x3(L, filt, prepared, stream))
        return rc;
    return small_b200_conv2d_f32_tf32x3(L, in, in_lo, prepared, bias, out, stream);
}
