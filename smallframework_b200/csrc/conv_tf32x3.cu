// conv_tf32x3.cu -- fp32 dense convolution (stride 1) on the 5th-generation tensor cores with
// the 3xTF32 split: every fp32 operand x is fed as hi = x (the tensor core ignores the low 13
// mantissa bits) and lo = x - trunc_tf32(x) (exact in fp32), and each product is accumulated as
// a_lo*b_hi + a_hi*b_lo + a_hi*b_hi in fp32 tensor memory.  The dropped a_lo*b_lo term is
// 2^-22 relative, so the result stays within the 1e-5 gate against the reference's fp32 loop
// nest (include/small/abstract_layer.hpp:1368-1823, FLOAT_CONV_TILE_C).
//
// GEMM orientation: D[k][pixel] = sum_c W[k][c] * X[pixel][c].  The output channels are the
// tensor core's M (one tile of 128, or 64 for layers with fewer channels), the pixels its N
// (64..256 per CTA).  One tcgen05.mma of kind::tf32 covers only 8 input channels and occupies
// the tensor pipe for N/2 cycles whatever M is, with a floor of about 80 cycles (measured with
// two issuing threads: 83 cycles at N = 128, 96 at N = 192, 128 at N = 256), so wide-N instructions
// are what keeps the pipe busy.  Every MMA reads its operands from shared memory (10 KB at N = 192):
// at full rate that alone is 107 of the 128 bytes per cycle shared memory delivers, which makes
// shared-memory bandwidth, not the tensor pipe, the ceiling of the wide layers.
//
// Layers with 32 or 64 output channels turn the GEMM around (PIXM): 128 pixels are the M of one MMA
// and all output channels its N, D[pixel][k].  Both dimensions of the instruction are then used in
// full (a 64-row M costs the same pipe time as 128 rows), an MMA takes N/2 = 16 or 32 cycles, and a
// thread of the accumulation warps owns one pixel with all its channels: its sums go to the packed
// output as 64-byte runs without any transposition.  Three threads issue the MMAs there.
// Variants of the pixel-major kernel (template arguments MERGED, POOL): for 16 / 32 output channels
// [W_hi | W_lo] is one operand of 2K columns (four MMAs per tap instead of six, TcArgs::merged); layers of
// one 16-channel block then sum the whole window in tensor memory (TcArgs::row_skip); for 32 / 64 output
// channels on wide images a following 2x2 stride-2 max pool can run in the epilogue (TcArgs::pool).
//
// Implicit GEMM without im2col ("linear shift"):
//   For one image and one block of 16 input channels, TMA copies a patch of the packed
//   activations [rows][PW columns][16 ch] (64 bytes per pixel) into shared memory.
//   PW = W + max(pad_l, pad_r): the zero column(s) that TMA's out-of-bounds fill produces at the
//   left edge of every row also serve as the right padding of the row above.  The copy writes
//   the patch in the 64-byte swizzle, and that IS a K-major operand of the tensor core: rows of
//   64 bytes (one pixel's 16 channels), 8-pixel groups 512 bytes apart; the hardware applies the
//   swizzle to absolute shared-memory addresses, so a descriptor may start at any pixel.  The raw
//   fp32 patch serves as the hi operand as it is; four splitter warps write the lo copy to the
//   same offsets of a second buffer.  Output pixel (r, c) is GEMM column m = r*PW + c, and filter
//   tap (kh, kw) of that pixel sits at patch entry m + kh*PW + kw: consecutive pixels are
//   consecutive rows for EVERY tap, so a tap only moves the descriptor's start address by 64 bytes
//   per pixel.  Columns with c >= Wo are junk and are not stored.
//   (A no-swizzle K-major patch needs 16-byte box rows from TMA, which it moves at about one row
//   per 9 cycles, or a re-layout pass through shared memory: both were slower.)
//   The filter [K/16][C/16][tap][16 c][16 k] has the output channel contiguous (MN-major).
//   kind::tf32 did not accept an MN-major no-swizzle operand on this hardware (a one-MMA
//   experiment returned zeros, while the K-major form was exact), so the filter is re-laid once
//   per set of weights into [K/MT][C/16][tap][c/4][MT k][4 c] (prepare_filter_kernel), MT =
//   output channels per CTA.  One tap of one CTA is then a single contiguous run of MT*64 bytes
//   that IS the K-major canonical layout and arrives by one bulk copy; its lo copy is made by the
//   same preparation step and loaded next to it (making it in shared memory like the patch's
//   cost more shared-memory bandwidth than the tensor core could spare).
#include "tc_common.cuh"

namespace
{
using namespace sb;

constexpr int W_STAGES_MAX = 6; // filter stages, each one group of taps (a kernel row)
constexpr int X_SLOTS_MAX = 3;

// Division of a non-negative int below 2^31 by a divisor fixed per launch: one multiply-high, an add and a
// shift instead of the two dozen instructions of a 32-bit division.  Every role decodes a tile per tile and
// the accumulation warps turn a GEMM column into a pixel with a division by the patch width; these run on the
// schedulers the MMA-issuing threads need.
struct FastDiv
{
    uint32_t mul, shift;
    __host__ void set(int d)
    {
        uint32_t s = 0;
        while ((1ull << s) < (unsigned long long)d)
            ++s;
        shift = s;
        mul = (uint32_t)((((1ull << 32) * ((1ull << s) - (unsigned long long)d)) / (unsigned long long)d) + 1);
    }
    __device__ __forceinline__ int div(int x) const { return (int)((__umulhi((uint32_t)x, mul) + (uint32_t)x) >> shift); }
};

struct TcArgs
{
    int N, C, K, H, W, Ho, Wo, Fh, Fw, pad_t, pad_l;
    int cbs, taps;
    int PW, PR;        // patch width / rows
    int NPX;           // pixels (GEMM columns) per CTA: 64, 128, 192 or 256
    int px_tiles;      // CTAs along the pixel axis per image
    int tiled;         // 0: tiles are ranges of full-width rows; 1: TH x TW pixel tiles
    int TW, TH, tiles_x; // tiled mode: valid columns / rows of a tile, tiles per row of tiles
    int MT;            // output channels per CTA (tensor-core M): 128 or 64
    int k_tiles;       // ceil(K / MT)
    int x_slots, w_stages;
    int pixm;          // 1: pixels on the tensor core's M, output channels on its N (K = 32 or 64)
    int tbufs;         // accumulator buffers in tensor memory: 2, or 4 when 4 * NPX <= 512 columns
    int group;         // filter taps summed in tensor memory before a flush
    // 1x1 layers: `cg` channel blocks travel as ONE patch of cg planes and are summed in tensor memory
    // as if they were the cg taps of a kernel row (cbs and taps then count these bundles: cbs = C/16/cg,
    // taps = group = cg).  A group of a 1x1 layer would otherwise be six MMAs, a third of the hand-overs
    // between the roles that a 3x3 kernel row pays for eighteen.  tap_step: descriptor units (16 bytes)
    // between the operand positions of two taps of a group: 4 (one pixel) or one plane of the patch.
    int cg, tap_step;
    // Output addressing in floats: pixel (r, c) of channel block kb lies at kb * o_kb_stride +
    // r * o_row_stride + c * 16 behind the image's first element.  Normally Ho*Wo*16 and Wo*16.
    // rows_view: a 1x1 layer on small images (H*W <= 64) is planned as ONE image whose rows are the
    // images of the batch (N' = 1, H' = N, W' = H*W): a 1x1 layer has no neighbourhoods, so a tile may
    // run across images and no tile is mostly empty (a 3x3-pixel image would fill 9 of a tile's 64
    // columns).  Only the strides differ: input rows are a whole image apart, and so are output rows.
    int rows_view;
    long long o_kb_stride, o_row_stride;
    int accumulate, act;
    float slope;
    unsigned smem_bytes;
    unsigned stage_off;  // byte offset of the output staging rows (0: they alias the operand buffers)
    int total_tiles;     // N * px_tiles * k_tiles
    int persistent;      // 1: one CTA per SM walks over the tiles; 0: one tile per CTA
    int ksplit;          // 2: a cluster of two CTAs shares a tile, each reduces half of the channel blocks
    int tile_base;       // first tile of this launch (a layer may run as two launches, see the launch code)
    int w_resident;      // 1: every group of a tile has a filter stage of its own, loaded once per CTA (see fit_rings)
    // Filters with 16 or 32 output channels are prepared with the lo rows of every 4-channel chunk right
    // behind its hi rows ([slab][c/4][hi k | lo k][4 c], interleaved_filter()): a pixel-major MMA then
    // takes [W_hi | W_lo] as ONE operand of 2K columns (the MERGED kernel, see its issuer).
    int merged;
    // Layers of one 16-channel block with the merged operand sum a WHOLE window in tensor memory (group = taps,
    // at most 18 full-size accumulations): one flush and one round of hand-overs per tile instead of one per
    // kernel row, and the issuing threads take whole tiles in turn.  row_skip: descriptor units from the last
    // tap of a kernel row to the first tap of the next one, beyond the one-pixel step.
    int row_skip;
    // 1: a 2x2 stride-2 max pool follows in the epilogue (pixel-major tiled plans only); the output strides
    // then describe the pooled tensor and `stage_off` locates the exchange rows of the pooling step
    int pool;
    FastDiv by_px_tiles, by_N, by_tiles_x, by_PW;
};

// Output channels per CTA, a function of K alone so that filter preparation and the
// convolution agree.
__host__ __device__ inline int pick_mt(int K) { return K >= 128 ? 128 : 64; }
// Layout of the prepared filter, a function of K alone for the same reason.
__host__ __device__ inline bool interleaved_filter(int K) { return K == 16 || K == 32; }

// packed filter [K/16][slab][16 c][16 k] -> hi and lo copies in [K/MT][slab][c/4][kv k][4 c];
// kv = MT except in a last, partial tile (K % MT channels).  inter: one array [slab][c/4][hi K | lo K][4 c].
__global__ void __launch_bounds__(256)
prepare_filter_kernel(long long n, int slabs, int MT, int K, int inter, const float *__restrict__ w,
                      float *__restrict__ hi, float *__restrict__ lo)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int k16 = (int)(i & 15), c = (int)((i >> 4) & 15);
    const long long t = i >> 8;            // kb16 * slabs + slab
    const int slab = (int)(t % slabs);
    const int k = (int)(t / slabs) * 16 + k16;
    const int tile = k / MT;
    const int kv = (K - tile * MT) < MT ? (K - tile * MT) : MT;
    const long long o = (long long)tile * MT * slabs * 16 + ((long long)slab * 4 + (c >> 2)) * kv * 4 +
                        (long long)(k - tile * MT) * 4 + (c & 3);
    const float v = w[i];
    const float vl = v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    if (inter)
    {
        const long long oi = (((long long)slab * 4 + (c >> 2)) * 2 * K + k) * 4 + (c & 3);
        hi[oi] = v;
        hi[oi + (long long)K * 4] = vl;
        return;
    }
    hi[o] = v;
    lo[o] = vl;
}

// Tensor-core accumulation truncates: every MMA adds into the fp32 accumulator with
// round-toward-zero, a one-sided error that grows with the number of accumulations (measured
// here: 3e-5 of the output range after 1700 MMAs).  So tensor memory only ever holds the sum
// of one kernel row of one channel block (6 MMAs per tap); eight accumulation warps pull
// these partial sums out with tcgen05.ld and add them into fp32 registers with
// round-to-nearest, while the tensor core already works on the next groups of taps in the other
// accumulator buffers of tensor memory (two of 192 or 256 columns, four when a buffer needs at
// most 128).
//
// warp 0: TMA producer, warps 1..2: MMA issuers (warp 3 idle), warps 4..11: accumulation +
// epilogue (lane quarter = warp % 4, pixel half = (warp - 4) / 4), warps 12..15: operand
// splitters (lo copy of every patch).  The first and last warpgroups give registers
// back (setmaxnreg) so that the accumulation warps can hold 128 running sums per thread
// without spilling.
//
// The unit of the filter pipeline is a GROUP of taps (one kernel row): one bulk copy and one
// tcgen05.commit, which frees the filter stage for the producer and hands the partial sums to
// the accumulation warps.
constexpr int ACC_WARPS = 8;
constexpr int FIRST_ACC_WARP = 4;
constexpr int FIRST_SPLIT_WARP = 12;
constexpr int SPLIT_THREADS = 128;
constexpr int NUM_THREADS = 512;
constexpr int COLS_PER_THREAD = 128;

__device__ __forceinline__ float4 lo_of(const float4 v)
{
    float4 r;
    r.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
    r.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
    r.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
    r.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
    return r;
}

// One tile of work: an image, a range of pixels and a block of MT output channels.
struct Tile
{
    int n, kt, kv;             // image, channel tile, channels this tile really has
    int row_base, col_base;    // first patch row / column in image coordinates (before padding)
    int m_local0;              // first GEMM column inside the patch
    int tw_valid, th_valid;    // real outputs per patch row / patch rows that hold outputs
};

// FAST = false keeps the plain divisions: the whole-window instantiations (MERGED == 2) are at the edge of their
// register budget, and with the multiply-high form the compiler's spill landed in their MMA issue loop
// (16 -> 32 channels at 208x208: 0.203 -> 0.225 ms), so they divide the slow way.
template <bool FAST = true>
__device__ __forceinline__ Tile decode_tile(const TcArgs &a, int t)
{
    // Pixel tile fastest, then the image, channel tile slowest.  The CTAs that run at the same time then
    // share one or two filter slices (a slice of a 1024 -> 1024 3x3 layer is 9.4 MB with its lo copy),
    // which stay in L2 while every image's tiles pass over them, and the activations of the whole batch
    // (44 MB there) stay in L2 from one slice to the next; neighbouring tiles of an image, whose patches
    // share their halo rows, still run side by side.  With the channel tile fastest, every 9 images streamed
    // all 75 MB of filter again: 541 MB of DRAM reads per launch for 126 MB of algorithmic bytes (176 MB
    // now, and the layer 3 % faster).
    Tile T;
    const int t1 = FAST ? a.by_px_tiles.div(t) : t / a.px_tiles, pt = t - t1 * a.px_tiles;
    T.kt = FAST ? a.by_N.div(t1) : t1 / a.N;
    T.n = t1 - T.kt * a.N;
    if (!a.tiled)
    {
        const int m0 = pt * a.NPX;
        T.row_base = FAST ? a.by_PW.div(m0) : m0 / a.PW; T.col_base = 0; T.m_local0 = m0 - T.row_base * a.PW;
        T.tw_valid = a.Wo; T.th_valid = a.Ho;
    }
    else
    {
        const int ty = FAST ? a.by_tiles_x.div(pt) : pt / a.tiles_x, tx = pt - ty * a.tiles_x;
        T.row_base = ty * a.TH; T.col_base = tx * a.TW; T.m_local0 = 0;
        T.tw_valid = (a.Wo - T.col_base) < a.TW ? (a.Wo - T.col_base) : a.TW; T.th_valid = a.TH;
    }
    T.kv = (a.K - T.kt * a.MT) < a.MT ? (a.K - T.kt * a.MT) : a.MT;
    return T;
}

// A CTA walks over tiles blockIdx.x, blockIdx.x + gridDim.x, ...  With a grid of one CTA per SM the
// roles run ahead of one another across tile boundaries: the producer, the splitters and the MMA
// issuer start the next tile while the accumulation warps still write the previous one out, which
// hides the start-up and the epilogue of a tile (half the life of a CTA on layers with few channel
// blocks).  All ring positions and barrier phases therefore count patches and groups over the whole
// life of the CTA.  With one tile per CTA (grid = number of tiles) the loop runs once and the
// output staging may alias the operand buffers (stage_off = 0).
// PERSIST = false: exactly one tile per CTA, known at compile time.
#define SB_TILE_LOOP(cond_extra) \
    for (int t = first_tile, once_ = 0; (PERSIST ? (t < a.total_tiles) : (once_ == 0)) && (cond_extra); t += tile_step, ++once_)

template <bool PERSIST, bool SPLIT, bool PIXM = false, int MERGED = 0, bool POOL = false> // MERGED: 1 merged operand, 2 with whole-window groups
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_tf32x3_kernel(const __grid_constant__ CUtensorMap map_x, const float *__restrict__ filt,
                   const float *__restrict__ filt_lo, const TcArgs a, const float *__restrict__ bias, float *__restrict__ out, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t x_full[X_SLOTS_MAX], x_ready[X_SLOTS_MAX], x_empty[X_SLOTS_MAX];
    __shared__ __align__(8) uint64_t w_full[W_STAGES_MAX], g_done[W_STAGES_MAX];
    __shared__ __align__(8) uint64_t t_full[4], t_empty[4];
    __shared__ __align__(8) uint64_t peer_staged, peer_done; // split reduction: hand-over between the two CTAs
    __shared__ uint32_t tmem_base_s;
    __shared__ int acc_failed; // an accumulation warp gave up on a wait: all eight leave at the same tile

    const uint32_t entries = (uint32_t)a.PR * a.PW;
    const uint32_t x_bytes = entries * 64 * (uint32_t)a.cg;     // one patch [plane][entry][16 floats]
    const uint32_t x_part = (x_bytes + 1023u) & ~1023u;         // hi (or lo) copy; keeps the swizzle pattern anchored
    const uint32_t w_part = (uint32_t)a.MT * 64;               // one hi (or lo) tap tile
    uint8_t *sX = smem;                                              // [slot][hi|lo][entry][64 B, 64-byte swizzle]
    uint8_t *sW = sX + (size_t)a.x_slots * 2 * x_part;              // [stage][hi|lo][tap in group][c/4][MT k][16 B]
    const uint32_t w_half_stage = (uint32_t)a.group * w_part;       // hi (or lo) tiles of one stage

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < (PIXM ? a.tbufs * (a.NPX >> 7) * a.K * (MERGED ? 2 : 1) : a.tbufs * a.NPX))
        tmem_cols <<= 1;

    // Split reduction (one tile per CTA only): the two CTAs of a cluster take one half of the channel
    // blocks each; rank 1 hands its sums to rank 0 through shared memory at the end.  It turns the
    // 3.46 waves of the 13x13 layers at batch 64 into 7 half-waves.
    constexpr bool split = SPLIT && !PERSIST;
    const uint32_t crank = split ? cluster_ctarank() : 0u;
    const int cbs_l = split ? a.cbs / 2 : a.cbs;     // channel blocks this CTA reduces
    const int cb_begin = (int)crank * cbs_l;
    const int steps = a.cbs * a.taps;
    const int groups_per_cb = a.taps / a.group, groups = cbs_l * groups_per_cb;
    const int first_tile = a.tile_base + (split ? blockIdx.x / 2 : blockIdx.x), tile_step = gridDim.x;

    // patch number pc / group number gc count over every tile of this CTA
    auto issue_patch = [&](const Tile &T, int cb, int pc) {
        const int slot = pc % a.x_slots;
        mbar_expect_tx(&x_full[slot], x_bytes);
        tma_load_4d(sX + (size_t)slot * 2 * x_part, &map_x, 0, T.col_base - a.pad_l, T.row_base - a.pad_t,
                    (T.n * a.cbs + cb_begin + cb) * a.cg, &x_full[slot]);
    };
    auto issue_filter = [&](const Tile &T, int g, int gc) {
        const int st = gc % a.w_stages;
        uint8_t *wd = sW + (size_t)st * 2 * w_half_stage;
        const size_t off = (size_t)T.kt * a.MT * steps * 16 + (size_t)(g + cb_begin * groups_per_cb) * a.group * T.kv * 16;
        mbar_expect_tx(&w_full[st], 2u * a.group * T.kv * 64);
        if (MERGED)
        {
            // hi and lo rows of a chunk lie side by side in one array: one run of twice the length
            tma_load_1d(wd, filt + 2 * off, 2u * a.group * T.kv * 64, &w_full[st]);
            return;
        }
        // the group's taps are contiguous, [tap][c/4][kv k][4 c]: a partial last tile (kv < MT) simply
        // is a shorter run, and the MMA descriptors take kv * 16 bytes as the chunk stride
        tma_load_1d(wd, filt + off, (uint32_t)a.group * T.kv * 64, &w_full[st]);
        tma_load_1d(wd + w_half_stage, filt_lo + off, (uint32_t)a.group * T.kv * 64, &w_full[st]);
    };

    if (warp == 0)
    {
        if (lane == 0)
        {
            acc_failed = 0;
            for (int i = 0; i < X_SLOTS_MAX; ++i)
            {
                mbar_init(&x_full[i], 1); mbar_init(&x_ready[i], SPLIT_THREADS); mbar_init(&x_empty[i], PIXM ? 3 : 2);
            }
            for (int i = 0; i < W_STAGES_MAX; ++i)
            {
                mbar_init(&w_full[i], 1); mbar_init(&g_done[i], 1);
            }
            for (int i = 0; i < 4; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], ACC_WARPS); }
            mbar_init(&peer_staged, ACC_WARPS); mbar_init(&peer_done, ACC_WARPS);
            fence_barrier_init();
            // The first patch and the first filter stage only need their barriers: their round
            // trip to memory overlaps the tensor-memory allocation and the CTA-wide barrier.
            const Tile T = decode_tile<MERGED != 2>(a, first_tile);
            issue_patch(T, 0, 0);
            issue_filter(T, 0, 0);
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    if (split)
        cluster_sync_all(); // the peer's barriers exist before anybody can arrive on them
    else
        __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp < FIRST_ACC_WARP || warp >= FIRST_SPLIT_WARP)
    {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        if (warp == 0 && lane == 0)
        {
            // ---------------- producer ----------------
            bool ok = true;
            // Patches run ahead of the filter stages where a slot is free: a patch is a tiled copy of
            // a few hundred 64-byte rows from memory and takes several thousand cycles, more than
            // the MMAs of a tile with one or two channel blocks.  The look-ahead never waits (a wait
            // here would hold back the filter stages); only the patch of the group at hand does.
            // The patch cursor (p_t, p_cb) walks the same (tile, channel block) sequence as everybody else.
            int pc = 1, gc = 0, q = 0; // pc: patches issued (patch 0 already is), q: patches the groups have entered
            int p_t = first_tile, p_cb = 1;
            Tile PT = decode_tile<MERGED != 2>(a, p_t); // decoded once per tile (the decode divides)
            auto step_cursor = [&]() {
                if (p_cb == cbs_l)
                {
                    p_cb = 0;
                    p_t += tile_step;
                    if (PERSIST && p_t < a.total_tiles)
                        PT = decode_tile<MERGED != 2>(a, p_t);
                }
            };
            step_cursor();
            auto next_patch = [&]() {
                issue_patch(PT, p_cb, pc);
                ++pc;
                ++p_cb;
                step_cursor();
            };
            SB_TILE_LOOP(ok)
            {
                const Tile T = decode_tile<MERGED != 2>(a, t);
                for (int g = 0; g < groups && ok; ++g, ++gc)
                {
                    if (g % groups_per_cb == 0)
                    {
                        if (pc <= q) // the look-ahead has not reached this group's patch: now it must go
                        {
                            const int slot = pc % a.x_slots, xuse = pc / a.x_slots;
                            if (xuse > 0) // all issuers' MMAs on the slot's previous patch are done
                                ok = mbar_wait(&x_empty[slot], (xuse - 1) & 1, status, 11);
                            if (!ok)
                                break;
                            next_patch();
                        }
                        ++q;
                    }
                    while (pc < q - 1 + a.x_slots && (PERSIST ? p_t < a.total_tiles : p_t == first_tile) &&
                           (pc < a.x_slots || mbar_test(&x_empty[pc % a.x_slots], ((pc / a.x_slots) - 1) & 1)))
                        next_patch();
                    if (gc == 0)
                        continue; // so is filter stage 0
                    if (a.w_resident && gc >= a.w_stages)
                        continue; // the whole filter is in shared memory since the CTA's first tile
                    const int st = gc % a.w_stages, wuse = gc / a.w_stages;
                    if (wuse > 0)
                        ok = mbar_wait(&g_done[st], (wuse - 1) & 1, status, 12);
                    if (!ok)
                        break;
                    issue_filter(T, g, gc);
                }
            }
        }
        else if (warp >= 1 && warp <= (PIXM ? 3 : 2) && lane == 0)
        {
            // ---------------- MMA issuers ----------------
            // All descriptor fields except the 16-byte-granular start address are fixed per CTA,
            // and a new operand position is one 64-bit add on a precomputed descriptor.  A = filter
            // tap (M = channels), B = patch shifted by the tap (N = pixels).
            // Issuing one MMA costs a thread about as long as the tensor pipe needs for it
            // (measured: one thread sustains an N = 192 MMA every 122 cycles, the pipe takes 96;
            // two threads together reach the 96), and whatever the thread does between two groups
            // (three barrier waits of about 200 cycles each, the commit) is idle tensor time on top.
            // Two threads therefore take the groups in turn, one per tensor-memory buffer: while
            // one waits for its filter stage and its buffer, the other one's MMAs keep the pipe
            // busy.  The groups are independent sums, so the two threads need no order between them.
            // Pixel-major tiles (PIXM: M = 128 pixels, N = all 32 or 64 output channels) have cheap
            // MMAs (N/2 cycles each), so a third thread joins to keep up with the pipe.
            constexpr int NISS = PIXM ? 3 : 2;
            const int me = warp - 1; // this thread issues the groups with g % NISS == me
            int turn = 0;            // g % NISS
            const bool own_t_full = PIXM || a.tbufs > a.w_stages;
            const int mtiles = a.NPX >> 7; // PIXM: blocks of 128 pixels per tile
            const int tb_mask = a.tbufs - 1, tb_shift = a.tbufs == 4 ? 2 : 1; // group g sums in buffer g % tbufs
            bool ok = true;
            // patch: rows of 64 bytes (one pixel's 16 channels) in the 64-byte swizzle the bulk copy
            // wrote; 8-pixel groups are 512 bytes apart; a pixel further is 4 descriptor units
            const uint64_t x_desc_base = make_smem_desc(smem_u32(sX), 16, 512, 4);
            const uint32_t idesc = make_idesc(1 /*f32*/, 2 /*tf32*/, 2 /*tf32*/, 0 /*A K-major*/, 0 /*B K-major*/,
                                              PIXM ? 128u : (uint32_t)a.MT, PIXM ? (uint32_t)a.K : (uint32_t)a.NPX);
            const uint32_t idesc_wide = make_idesc(1, 2, 2, 0, 0, 128u, 2u * (uint32_t)a.K); // MERGED: N = [hi | lo]
            const uint64_t x_lo_off = x_part >> 4, w_lo_off = w_half_stage >> 4;
            constexpr uint32_t w_rows = MERGED ? 2u : 1u; // rows of a 4-channel chunk: kv, or kv hi + kv lo
            const uint64_t x_half = 2; // channels 8..15 of the block
            const uint64_t tap_step = (uint64_t)a.tap_step;
            const uint64_t w_stage_step = (uint64_t)2 * w_half_stage >> 4;
            const uint64_t x_slot_step = (uint64_t)2 * x_part >> 4;
            int slot = 0, xphase = 0, st = 0, wphase = 0, g = 0; // g counts groups over all tiles
            uint64_t x_slot_off = 0, w_stage_off = 0;
            SB_TILE_LOOP(ok)
            {
                // Of a tile the issuing threads need only its first GEMM column inside the patch and the channels
                // of its channel tile; 2-D pixel tiles of a layer with one channel tile always start at column 0
                // with all K channels, and the decode (three integer divisions per tile, for every issuing
                // thread and every tile, its own or not) is issue time taken from the MMAs.
                Tile T;
                if (a.tiled && a.k_tiles == 1)
                {
                    T.m_local0 = 0; T.kv = a.K;
                }
                else
                    T = decode_tile<MERGED != 2>(a, t);
                const uint64_t x_desc0 = x_desc_base + (uint64_t)T.m_local0 * 4;
                // filter stage: [tap][c/4][kv rows][16 B], kv = channels of this tile
                const uint64_t w_desc0 = make_smem_desc(smem_u32(sW), (uint32_t)T.kv * 16 * w_rows, 128, 0);
                const uint64_t w_tap = (uint64_t)T.kv * 4 * w_rows, w_half = (uint64_t)T.kv * 2 * w_rows;
                for (int cb = 0; cb < cbs_l && ok; ++cb)
                {
                    ok = mbar_wait(&x_ready[slot], xphase, status, 13);
                    if (!ok)
                        break;
                    uint64_t x_row = x_desc0 + x_slot_off; // patch position of tap (kh, 0)
                    for (int gi = 0; gi < groups_per_cb && ok; ++gi, ++g)
                    {
                        if (turn == me)
                        {
                            // resident stages complete phase 0 once and stay there; every issuer still has
                            // to observe that itself the first time it uses a stage (with 1, 2, 4 or 5
                            // stages a stage is not always the same thread's), and a completed phase
                            // answers at once
                            ok = mbar_wait(&w_full[st], a.w_resident ? 0u : (uint32_t)wphase, status, 14);
                            if (ok && g > tb_mask)
                                ok = mbar_wait(&t_empty[g & tb_mask], ((g >> tb_shift) - 1) & 1, status, 16);
                            if (!ok)
                                break;
                            tc_fence_after_sync();
                            uint64_t wh = w_desc0 + w_stage_off, xh = x_row;
                            if (PIXM && MERGED)
                            {
                                // [W_hi | W_lo] is one operand of 2K columns: x_hi times it gives the hi*hi sums in
                                // columns [0, K) and one cross term in [K, 2K), x_lo * W_hi adds the other cross
                                // term there.  Four instructions per tap and 128 pixels instead of six, the 128-pixel
                                // operand read from shared memory four times instead of six, and the small terms
                                // never meet a full-size accumulator; the accumulation warps add the two halves.
                                const uint32_t d0 = tmem + (uint32_t)((g & tb_mask) * mtiles * 2 * a.K);
                                int kw = 0;
                                for (int tp = 0; tp < a.group; ++tp, wh += w_tap, xh += tap_step)
                                {
                                    for (int mt = 0; mt < mtiles; ++mt)
                                    {
                                        const uint64_t xa = xh + (uint64_t)mt * 512, xl = xa + x_lo_off;
                                        const uint32_t d = d0 + (uint32_t)(mt * 2 * a.K);
                                        tc_mma_tf32(d, xa, wh, idesc_wide, tp == 0 ? 0u : 1u);
                                        tc_mma_tf32(d + (uint32_t)a.K, xl, wh, idesc, 1u);
                                        tc_mma_tf32(d, xa + x_half, wh + w_half, idesc_wide, 1u);
                                        tc_mma_tf32(d + (uint32_t)a.K, xl + x_half, wh + w_half, idesc, 1u);
                                    }
                                    if (MERGED == 2 && ++kw == a.Fw) // the group spans kernel rows: on to the next patch row
                                    {
                                        kw = 0;
                                        xh += (uint64_t)a.row_skip;
                                    }
                                }
                            }
                            else if (PIXM)
                            {
                                const uint32_t d0 = tmem + (uint32_t)((g & tb_mask) * mtiles * a.K);
                                // The small cross terms of the whole group first, the hi*hi terms last: the
                                // tensor core adds into its accumulator with truncation, an error of one ulp OF
                                // THE ACCUMULATOR per MMA, so only the MMAs issued while it holds full-size sums
                                // (two per tap instead of six) contribute a full-size error.
                                uint64_t wh2 = wh, xh2 = xh;
                                for (int tp = 0; tp < a.group; ++tp, wh += w_tap, xh += tap_step)
                                {
                                    const uint64_t wl = wh + w_lo_off;
                                    for (int mt = 0; mt < mtiles; ++mt)
                                    {
                                        const uint64_t xa = xh + (uint64_t)mt * 512, xl = xa + x_lo_off; // 128 pixels on
                                        const uint32_t d = d0 + (uint32_t)(mt * a.K);
                                        tc_mma_tf32(d, xa, wl, idesc, tp == 0 ? 0u : 1u);
                                        tc_mma_tf32(d, xl, wh, idesc, 1u);
                                        tc_mma_tf32(d, xa + x_half, wl + w_half, idesc, 1u);
                                        tc_mma_tf32(d, xl + x_half, wh + w_half, idesc, 1u);
                                    }
                                }
                                for (int tp = 0; tp < a.group; ++tp, wh2 += w_tap, xh2 += tap_step)
                                    for (int mt = 0; mt < mtiles; ++mt)
                                    {
                                        const uint64_t xa = xh2 + (uint64_t)mt * 512;
                                        const uint32_t d = d0 + (uint32_t)(mt * a.K);
                                        tc_mma_tf32(d, xa, wh2, idesc, 1u);
                                        tc_mma_tf32(d, xa + x_half, wh2 + w_half, idesc, 1u);
                                    }
                            }
                            const uint32_t d = tmem + (uint32_t)((g & tb_mask) * a.NPX);
                            uint64_t wh2 = wh, xh2 = xh; // cross terms first, hi*hi last (see the pixel-major loop)
                            for (int tp = 0; !PIXM && tp < a.group; ++tp, wh += w_tap, xh += tap_step)
                            {
                                const uint64_t xl = xh + x_lo_off, wl = wh + w_lo_off;
                                tc_mma_tf32(d, wl, xh, idesc, tp == 0 ? 0u : 1u);
                                tc_mma_tf32(d, wh, xl, idesc, 1u);
                                tc_mma_tf32(d, wl + w_half, xh + x_half, idesc, 1u);
                                tc_mma_tf32(d, wh + w_half, xl + x_half, idesc, 1u);
                            }
                            for (int tp = 0; !PIXM && tp < a.group; ++tp, wh2 += w_tap, xh2 += tap_step)
                            {
                                tc_mma_tf32(d, wh2, xh2, idesc, 1u);
                                tc_mma_tf32(d, wh2 + w_half, xh2 + x_half, idesc, 1u);
                            }
                            // the stage is free for the producer and the group's partial sums are
                            // complete for the accumulation warps: one commit serves both while the
                            // accumulator ring is no deeper than the filter ring (a waiter must not fall
                            // two phases behind its barrier)
                            tc_commit(&g_done[st]);
                            if (own_t_full)
                                tc_commit(&t_full[g & tb_mask]);
                        }
                        if (++turn == NISS)
                            turn = 0;
                        x_row += (uint64_t)(a.group == a.Fw ? a.PW : 1) * 4;
                        w_stage_off += w_stage_step;
                        if (++st == a.w_stages) { st = 0; wphase ^= 1; w_stage_off = 0; }
                    }
                    tc_commit(&x_empty[slot]); // both issuers: the slot is free once the MMAs of either are done
                    x_slot_off += x_slot_step;
                    if (++slot == a.x_slots) { slot = 0; xphase ^= 1; x_slot_off = 0; }
                }
            }
        }
        else if (warp >= FIRST_SPLIT_WARP)
        {
            // ---------------- operand splitters ----------------
            const int sid = tid - FIRST_SPLIT_WARP * 32;
            bool ok = true;
            int pc = 0;
            SB_TILE_LOOP(ok)
                for (int cb = 0; cb < cbs_l && ok; ++cb, ++pc)
                {
                    const int slot = pc % a.x_slots;
                    ok = mbar_wait(&x_full[slot], (pc / a.x_slots) & 1, status, 17);
                    if (!ok)
                        break;
                    {
                        // The patch as the bulk copy wrote it is the hi operand (the tensor core
                        // ignores the 13 low mantissa bits of an fp32 word read as tf32); the lo copy
                        // takes the same place in its own buffer, so the swizzle needs no thought.
                        const float4 *xh = reinterpret_cast<const float4 *>(sX + (size_t)slot * 2 * x_part);
                        float4 *xl = reinterpret_cast<float4 *>(sX + (size_t)slot * 2 * x_part + x_part);
                        const uint32_t total = x_bytes >> 4;
                        for (uint32_t i = (uint32_t)sid; i < total; i += SPLIT_THREADS)
                            xl[i] = lo_of(xh[i]);
                    }
                    fence_proxy_async();
                    mbar_arrive(&x_ready[slot]);
                }
        }
    }
    else
    {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
        const float act_ns = act_neg_scale(a.act, a.slope); // activation: v > 0 ? v : v * act_ns
        if (PIXM)
        {
            // ---------------- accumulation + epilogue, pixel-major ----------------
            // A thread owns one pixel (its tensor-memory lane) and all K <= 64 output channels of it:
            // the running sums need 64 registers, a flush is one or two loads, and the epilogue
            // writes 64 contiguous bytes per channel block straight from the registers (a warp
            // covers 32 consecutive pixels: no transposition through shared memory, no barrier).
            const int quarter = warp & 3, mt = (warp - FIRST_ACC_WARP) >> 2;
            const int mtiles = a.NPX >> 7;
            const bool active = mt < mtiles;
            const size_t plane = (size_t)a.o_kb_stride;
            bool ok = true;
            int gc = 0;
            SB_TILE_LOOP(ok)
            {
                const Tile T = decode_tile<MERGED != 2>(a, t);
                // the bias seeds the sums (these loads overlap the wait for the first group)
                constexpr int ACC = MERGED ? 32 : 64; // output channels a thread can hold
                float acc[ACC];
#pragma unroll
                for (int c4 = 0; c4 < ACC / 4; ++c4)
                {
                    const float4 b = (bias && c4 * 4 < a.K) ? __ldg(reinterpret_cast<const float4 *>(bias) + c4)
                                                            : make_float4(0.f, 0.f, 0.f, 0.f);
                    acc[4 * c4] = b.x; acc[4 * c4 + 1] = b.y; acc[4 * c4 + 2] = b.z; acc[4 * c4 + 3] = b.w;
                }
                for (int g = 0; g < groups && ok; ++g, ++gc)
                {
                    const int tb = gc & 3;
                    ok = mbar_wait(&t_full[tb], (gc >> 2) & 1, status, 15, 1u << 24);
                    if (!ok)
                        break;
                    tc_fence_after_sync();
                    if (active)
                    {
                        const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) +
                                               (uint32_t)((tb * mtiles + mt) * a.K * (MERGED ? 2 : 1));
                        if (MERGED)
                        {
                            // columns [0, K): the hi*hi sums, [K, 2K): the cross terms of the same channels
                            uint32_t v[32];
                            tmem_ld32(tbase, v);
                            tmem_ld_wait();
                            if (a.K == 16)
                            {
#pragma unroll
                                for (int e = 0; e < 16; ++e)
                                    acc[e] += __uint_as_float(v[e]) + __uint_as_float(v[16 + e]);
                            }
                            else
                            {
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    acc[e] += __uint_as_float(v[e]);
                                tmem_ld32(tbase + 32u, v);
                                tmem_ld_wait();
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    acc[e] += __uint_as_float(v[e]);
                            }
                        }
                        else // K = 64
                        {
#pragma unroll
                        for (int piece = 0; piece < 2; ++piece)
                            if (piece * 32 < a.K)
                            {
                                uint32_t v[32];
                                tmem_ld32(tbase + (uint32_t)(piece * 32), v);
                                tmem_ld_wait();
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    acc[piece * 32 + e] += __uint_as_float(v[e]);
                            }
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&t_empty[tb]);
                }
                if (POOL)
                {
                    // 2x2 max pool, stride 2, on the sums in registers (K = 32 or 64: a thread holds ACC = K
                    // sums).  Tiles have even heights and widths and an even patch width, so the horizontal
                    // neighbour of pixel (rl, cl) is the next lane of the same warp: the even lane of a pair keeps
                    // the lower half of the channels of BOTH pixels' maximum, the odd lane the upper half (one
                    // shuffle per kept channel).  The vertical neighbour is PW lanes further on, in another warp:
                    // odd rows leave their halves in shared memory, even rows pick them up behind a barrier of the
                    // eight accumulation warps, apply the activation (monotonic, so it commutes with the maximum;
                    // the launch code checks that) and store their half of the pooled pixel.  A first barrier
                    // keeps a warp from writing into the exchange rows while a slower one still reads the previous
                    // tile's.  Every instruction here competes with the MMA-issuing threads for the issue slots of
                    // the four schedulers, which is why the work is split between the lanes of a pair.
                    // Every warp comes to the first barrier at every tile; a warp whose wait ran out says so
                    // before it and all leave together (see the channel-major epilogue).
                    constexpr int HALF = ACC / 2;
                    const int ml = mt * 128 + quarter * 32 + lane; // tiled plans: m_local0 = 0
                    const int rl = (MERGED == 2 ? ml / a.PW : a.by_PW.div(ml)), cl = ml - rl * a.PW;
                    const int upper = lane & 1;
                    float *xrow = reinterpret_cast<float *>(smem + a.stage_off) +
                                  ((size_t)(rl >> 1) * (a.PW >> 1) + (cl >> 1)) * (ACC + 4) + upper * HALF;
                    if (!ok)
                        *reinterpret_cast<volatile int *>(&acc_failed) = 1;
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (*reinterpret_cast<volatile int *>(&acc_failed))
                        ok = false;
                    if (ok)
                    {
                        float keep[HALF];
                        if (active)
                        {
#pragma unroll
                            for (int e = 0; e < HALF; ++e)
                            {
                                const float mine = upper ? acc[HALF + e] : acc[e], theirs = upper ? acc[e] : acc[HALF + e];
                                keep[e] = fmaxf(mine, __shfl_xor_sync(0xffffffffu, theirs, 1));
                            }
                            if ((rl & 1) && rl < a.TH)
                            {
#pragma unroll
                                for (int j = 0; j < HALF / 4; ++j)
                                    reinterpret_cast<float4 *>(xrow)[j] = make_float4(keep[4 * j], keep[4 * j + 1], keep[4 * j + 2], keep[4 * j + 3]);
                            }
                        }
                        asm volatile("bar.sync 1, 256;" ::: "memory");
                        const int r = T.row_base + rl, c = T.col_base + (cl & ~1);
                        if (active && !(rl & 1) && (cl & ~1) < T.tw_valid && rl < a.TH && r < a.Ho)
                        {
                            float *o = out + ((size_t)T.n * (a.K / CB) + (size_t)upper * (HALF / CB)) * plane +
                                       (size_t)(r >> 1) * a.o_row_stride + (size_t)(c >> 1) * CB;
#pragma unroll
                            for (int j = 0; j < HALF / 4; ++j)
                            {
                                const float4 y = reinterpret_cast<const float4 *>(xrow)[j]; // row rl + 1 shares the slot
                                float4 x = make_float4(fmaxf(keep[4 * j], y.x), fmaxf(keep[4 * j + 1], y.y),
                                                       fmaxf(keep[4 * j + 2], y.z), fmaxf(keep[4 * j + 3], y.w));
                                x.x = apply_act_ns(x.x, act_ns); x.y = apply_act_ns(x.y, act_ns);
                                x.z = apply_act_ns(x.z, act_ns); x.w = apply_act_ns(x.w, act_ns);
                                *(reinterpret_cast<float4 *>(o + (size_t)(j >> 2) * plane) + (j & 3)) = x;
                            }
                        }
                    }
                }
                else if (ok && active)
                {
                    const int ml = T.m_local0 + mt * 128 + quarter * 32 + lane;
                    const int rl = (MERGED == 2 ? ml / a.PW : a.by_PW.div(ml)), cl = ml - rl * a.PW;
                    const int r = T.row_base + rl, c = T.col_base + cl;
                    if (cl < T.tw_valid && rl < T.th_valid && r < a.Ho)
                    {
                        float *o = out + (size_t)T.n * (a.K / CB) * plane + (size_t)r * a.o_row_stride + (size_t)c * CB;
#pragma unroll
                        for (int kb = 0; kb < ACC / 16; ++kb)
                            if (kb * CB < a.K)
                            {
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                {
                                    float4 x = make_float4(acc[kb * 16 + 4 * j], acc[kb * 16 + 4 * j + 1], acc[kb * 16 + 4 * j + 2],
                                                           acc[kb * 16 + 4 * j + 3]);
                                    float4 *op = reinterpret_cast<float4 *>(o + (size_t)kb * plane) + j;
                                    if (a.accumulate)
                                    {
                                        const float4 s4 = *op;
                                        x.x += s4.x; x.y += s4.y; x.z += s4.z; x.w += s4.w;
                                    }
                                    x.x = apply_act_ns(x.x, act_ns); x.y = apply_act_ns(x.y, act_ns);
                                    x.z = apply_act_ns(x.z, act_ns); x.w = apply_act_ns(x.w, act_ns);
                                    *op = x;
                                }
                            }
                    }
                }
            }
        }
        else
        {
        // ---------------- accumulation + epilogue ----------------
        const int quarter = warp & 3;                    // TMEM lanes [32*quarter, 32*quarter+32)
        const int phalf = (warp - FIRST_ACC_WARP) >> 2;  // which half of the tile's pixels
        const int my_cols = a.NPX / 2;                   // 32, 64, 96 or 128
        const int col0 = phalf * my_cols;
        // 128-channel tile: lane l of quarter q holds channel 32q + l; 64-channel tile: channel
        // 16q + l in lanes 0..15 of each quarter
        const int k_local = (a.MT == 128) ? quarter * 32 + lane : quarter * 16 + lane;
        const bool lane_has_row = (a.MT == 128) || (lane < 16);
        // Output staging rows of MT + 16 floats (free of bank conflicts both for the channel-wise
        // writes and for the float4 reads); a persistent CTA stages 32 pixels of each half at a time.
        const int pitch = a.MT + 16;
        float *stage = reinterpret_cast<float *>(smem + a.stage_off);
        const int psub = lane >> 2, q4 = lane & 3; // 8 pixels x 4 float4 per warp and step
        const size_t plane = (size_t)a.o_kb_stride;
        bool ok = true;
        int gc = 0;
        SB_TILE_LOOP(ok)
        {
            const Tile T = decode_tile(a, t);
            // the bias of this thread's channel seeds its sums (rank 0 only when two CTAs share a tile)
            const float seed = (bias && crank == 0 && lane_has_row && k_local < T.kv) ? __ldg(bias + T.kt * a.MT + k_local) : 0.f;
            float acc[COLS_PER_THREAD];
#pragma unroll
            for (int c = 0; c < COLS_PER_THREAD; ++c)
                acc[c] = seed;
            for (int g = 0; g < groups && ok; ++g, ++gc)
            {
                const int tb = gc & (a.tbufs - 1);
                if (a.tbufs > a.w_stages)
                    ok = mbar_wait(&t_full[tb], (gc >> (a.tbufs == 4 ? 2 : 1)) & 1, status, 15, 1u << 24);
                else
                    ok = mbar_wait(&g_done[gc % a.w_stages], (gc / a.w_stages) & 1, status, 15, 1u << 24);
                if (!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(tb * a.NPX + col0);
#pragma unroll
                for (int piece = 0; piece < COLS_PER_THREAD / 32; ++piece)
                {
                    if (piece * 32 < my_cols)
                    {
                        uint32_t v[32];
                        tmem_ld32(tbase + (uint32_t)(piece * 32), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            acc[piece * 32 + e] += __uint_as_float(v[e]);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&t_empty[tb]);
            }
            // Epilogue (the other roles are already at work on the next tile): a thread owns one
            // channel of up to 128 pixels, the packed output wants 16 channels of one pixel together.
            const int kbs = T.kv / CB; // channel blocks this tile really has
            float *obase = out + ((size_t)T.n * (a.K / CB) + (size_t)T.kt * (a.MT / CB)) * plane + q4 * 4;
            if (!PERSIST)
            {
                // one tile per CTA: every operand buffer is dead, the whole tile is staged at once
                if (ok && lane_has_row)
                {
                    float *srow = stage + (size_t)col0 * pitch + k_local;
                    if (a.MT == 128)
                    {
#pragma unroll
                        for (int e = 0; e < COLS_PER_THREAD; ++e)
                            if (e < my_cols)
                                srow[e * 144] = acc[e];
                    }
                    else
                    {
#pragma unroll
                        for (int e = 0; e < COLS_PER_THREAD; ++e)
                            if (e < my_cols)
                                srow[e * 80] = acc[e];
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory"); // the eight accumulation warps
                uint32_t peer_stage = 0;
                if (split)
                {
                    if (crank == 1)
                    {
                        // hand the staged half-sums to rank 0, then stay until it has read them
                        if (lane == 0)
                        {
                            asm volatile("fence.acq_rel.cluster;" ::: "memory");
                            mbar_arrive_remote(map_to_cta(&peer_staged, 0));
                        }
                        ok = mbar_wait_cluster(&peer_done, 0, status, 21) && false; // rank 1 stores nothing
                    }
                    else
                    {
                        ok = ok && mbar_wait_cluster(&peer_staged, 0, status, 20);
                        peer_stage = map_to_cta(stage, 1);
                    }
                }
                if (ok)
                {
                    for (int pg = warp - FIRST_ACC_WARP; pg < a.NPX / 8; pg += ACC_WARPS)
                    {
                        const int px = pg * 8 + psub;
                        const int ml = T.m_local0 + px;
                        const int rl = a.by_PW.div(ml), cl = ml - rl * a.PW;
                        const int r = T.row_base + rl, c = T.col_base + cl;
                        if (cl < T.tw_valid && rl < T.th_valid && r < a.Ho)
                        {
                            const float *sp = stage + (size_t)px * pitch + q4 * 4;
                            const uint32_t rp = peer_stage + (uint32_t)(((size_t)px * pitch + q4 * 4) * 4);
                            float *o = obase + (size_t)r * a.o_row_stride + (size_t)c * CB;
#pragma unroll
                            for (int kb = 0; kb < 8; ++kb)
                              if (kb < kbs)
                            {
                                float4 x = *reinterpret_cast<const float4 *>(sp + kb * CB);
                                if (split)
                                {
                                    const float4 y = ld_cluster_f4(rp + (uint32_t)(kb * CB * 4)); // rank 1's half
                                    x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
                                }
                                float *ok_ = o + (size_t)kb * plane;
                                if (a.accumulate)
                                {
                                    const float4 s4 = *reinterpret_cast<const float4 *>(ok_);
                                    x.x += s4.x; x.y += s4.y; x.z += s4.z; x.w += s4.w;
                                }
                                x.x = apply_act_ns(x.x, act_ns); x.y = apply_act_ns(x.y, act_ns);
                                x.z = apply_act_ns(x.z, act_ns); x.w = apply_act_ns(x.w, act_ns);
                                *reinterpret_cast<float4 *>(ok_) = x;
                            }
                        }
                    }
                }
                if (split && crank == 0)
                {
                    // rank 1 may leave: its staging rows have been read
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive_remote(map_to_cta(&peer_done, 1));
                }
            }
            else
            {
#pragma unroll
            for (int piece = 0; piece < COLS_PER_THREAD / 32; ++piece)
            {
                if (piece * 32 < my_cols) // uniform over the CTA
                {
                    if (ok && lane_has_row)
                    {
                        float *srow = stage + (size_t)(phalf * 32) * pitch + k_local;
                        if (a.MT == 128)
                        {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                srow[e * 144] = acc[piece * 32 + e];
                        }
                        else
                        {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                srow[e * 80] = acc[piece * 32 + e];
                        }
                    }
                    // The give-up decision is made for the CTA, not per warp: the named barrier below
                    // needs all eight warps at every tile, so a warp whose wait ran out says so before
                    // the barrier and everybody reads it after, and all leave the tile loop together.
                    if (!ok)
                        *reinterpret_cast<volatile int *>(&acc_failed) = 1;
                    asm volatile("bar.sync 1, 256;" ::: "memory"); // the eight accumulation warps
                    if (*reinterpret_cast<volatile int *>(&acc_failed))
                        ok = false;
                    if (ok)
                    {
                        // staged row s holds pixel (s / 32) * my_cols + piece * 32 + s % 32 of the tile
                        const int s_row = (warp - FIRST_ACC_WARP) * 8 + psub;
                        const int px = (s_row >> 5) * my_cols + piece * 32 + (s_row & 31);
                        const int ml = T.m_local0 + px;
                        const int rl = a.by_PW.div(ml), cl = ml - rl * a.PW;
                        const int r = T.row_base + rl, c = T.col_base + cl;
                        if (cl < T.tw_valid && rl < T.th_valid && r < a.Ho)
                        {
                            const float *sp = stage + (size_t)s_row * pitch + q4 * 4;
                            float *o = obase + (size_t)r * a.o_row_stride + (size_t)c * CB;
#pragma unroll
                            for (int kb = 0; kb < 8; ++kb)
                              if (kb < kbs)
                            {
                                float4 x = *reinterpret_cast<const float4 *>(sp + kb * CB);
                                float *ok_ = o + (size_t)kb * plane;
                                if (a.accumulate)
                                {
                                    const float4 s4 = *reinterpret_cast<const float4 *>(ok_);
                                    x.x += s4.x; x.y += s4.y; x.z += s4.z; x.w += s4.w;
                                }
                                x.x = apply_act_ns(x.x, act_ns); x.y = apply_act_ns(x.y, act_ns);
                                x.z = apply_act_ns(x.z, act_ns); x.w = apply_act_ns(x.w, act_ns);
                                *reinterpret_cast<float4 *>(ok_) = x;
                            }
                        }
                    }
                    asm volatile("bar.sync 1, 256;" ::: "memory"); // before the staging rows are reused
                }
            }
            }
        }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0)
        tmem_dealloc(tmem, tmem_cols);
}

// Picks ring depths for the patch / filter sizes already in `a`.  Narrow layers run persistent (one
// CTA per SM walks over the tiles, roles overlap across tiles), which needs the output staging rows
// next to the operand buffers; the others keep the deepest rings and let the staging alias them.  need_two: only accept plans with two patches in flight.
bool fit_rings(TcArgs &a, bool need_two)
{
    a.row_skip = (a.cg == 1 && a.group != a.Fw) ? (a.PW - a.Fw) * 4 : 0;
    const size_t limit = 226 * 1024;
    const int entries = a.PR * a.PW;
    const size_t x_part = ((size_t)entries * 64 * a.cg + 1023) & ~(size_t)1023;
    const size_t w_part = (size_t)a.MT * 64 * a.group;
    const size_t staging = (size_t)64 * (a.MT + 16) * 4; // 32 pixels of each half of the tile
    // {patch slots, filter stages (>= 2: a commit serves both rings)}
    static const int pref[][2] = {{3, 3}, {2, 3}, {2, 2}, {1, 3}, {1, 2}};
    // persistent where it pays and fits: narrow layers (64-channel tiles: small filter stages and
    // staging rows, little work per tile); wide ones need the shared memory for deeper rings
    // Pixel-major persistent tiles whose whole filter fits: one stage per group of a tile, loaded once
    // per CTA.  The filter ring otherwise puts a bulk copy's round trip to L2 into every group's chain
    // of hand-overs (producer waits for the stage, copies, the issuer waits for the copy), and for
    // these layers that chain, not the MMAs, sets the pace (16 -> 32 channels at 208x208: 0.22 ms
    // with no MMA issued at all, 0.30 ms with them).
    a.w_resident = 0;
    // pooled epilogue: exchange rows, one slot of K + 4 floats per pair of columns of every odd row
    const size_t pool_rows = a.pool ? (size_t)(a.TH / 2) * (a.PW / 2) * (a.K + 4) * 4 : 0;
    if (a.pixm && a.k_tiles == 1 && a.cg == 1)
    {
        const int stages = a.cbs * (a.taps / a.group);
        if (stages <= W_STAGES_MAX)
            for (int xs = 3; xs >= 2; --xs)
            {
                const size_t ops = (size_t)xs * 2 * x_part + (size_t)stages * 2 * w_part;
                const size_t smem = ops + pool_rows;
                if (smem <= limit)
                {
                    a.x_slots = xs; a.w_stages = stages; a.smem_bytes = (unsigned)smem; a.tbufs = 4;
                    a.persistent = 1; a.stage_off = (unsigned)ops; a.w_resident = 1;
                    return true;
                }
            }
    }
    for (int persistent = (a.MT == 64 ? 1 : 0); persistent >= (a.pixm ? 1 : 0); --persistent)
        for (const auto &p : pref)
        {
            const int xs = p[0] < a.cbs || persistent ? p[0] : a.cbs;
            if (need_two && xs < 2 && a.cbs >= 2)
                continue;
            const size_t ops = (size_t)xs * 2 * x_part + (size_t)p[1] * 2 * w_part;
            const size_t full = (size_t)a.NPX * (a.MT + 16) * 4; // one tile per CTA stages the whole tile
            const size_t smem = persistent ? ops + (a.pixm ? pool_rows : staging) : (ops > full ? ops : full);
            if (smem <= limit)
            {
                a.x_slots = xs; a.w_stages = p[1]; a.smem_bytes = (unsigned)smem;
                a.tbufs = (a.pixm || 4 * a.NPX <= 512) ? 4 : 2;
                a.persistent = persistent; a.stage_off = persistent ? (unsigned)ops : 0u;
                return true;
            }
        }
    return false;
}

// Wide images: TH x TW pixel tiles.  A tile's patch is (TH + Fh) x (TW + Fw - 1) pixels, so the
// halo stays small (a range of full-width rows of a 208-wide image drags two whole rows of halo
// along for every 256 outputs).  GEMM column j of a tile is patch-linear: row j / PW, column j % PW,
// columns >= TW of each patch row are junk.
bool plan_tiled(const small_b200_layer *L, TcArgs &a)
{
    double best = 0.0;
    int best_tw = 0, best_th = 0;
    const int cap = 256, gran = a.pixm ? 128 : 64;
    for (int tw = 8; tw <= a.Wo && tw + a.Fw - 1 <= cap; tw += (a.pool ? 2 : 1))
    {
        const int pw = tw + a.Fw - 1;
        int th = (cap - tw) / pw + 1;
        if (th > a.Ho)
            th = a.Ho;
        if (a.pool && (th &= ~1) == 0) // pooled epilogue: pairs of rows and of columns stay inside a tile
            continue;
        const int npx = ((th - 1) * pw + tw + gran - 1) / gran * gran;
        const long long tiles = (long long)((a.Wo + tw - 1) / tw) * ((a.Ho + th - 1) / th);
        const double eff = (double)a.Wo * a.Ho / ((double)tiles * npx);
        if (eff > best + 1e-9)
        {
            best = eff; best_tw = tw; best_th = th;
        }
    }
    if (!best_tw)
        return false;
    a.tiled = 1; a.TW = best_tw; a.TH = best_th;
    a.PW = a.TW + a.Fw - 1;
    a.PR = a.TH + a.Fh; // one row more than the taps reach: the junk tail of the last row reads it
    if (a.PR > 256)
        return false;
    a.NPX = ((a.TH - 1) * a.PW + a.TW + gran - 1) / gran * gran;
    a.tiles_x = (a.Wo + a.TW - 1) / a.TW;
    a.px_tiles = a.tiles_x * ((a.Ho + a.TH - 1) / a.TH);
    // the last GEMM column's last tap must stay inside the patch
    if ((a.NPX - 1) + (a.Fh - 1) * a.PW + (a.Fw - 1) >= a.PR * a.PW)
        a.PR = ((a.NPX - 1) + (a.Fh - 1) * a.PW + (a.Fw - 1)) / a.PW + 1;
    return fit_rings(a, false);
}

// Tiling and shared-memory plan of one layer; false when the shape is not covered.
bool plan_as_g(const small_b200_layer *L, TcArgs &a, bool pixm, bool pool, bool whole)
{
    if (!L || L->stride != 1 || row_stride(L) != 1 || L->C % CB != 0 || L->K % CB != 0 || L->C <= 0 || L->K <= 0)
        return false;
    if (L->H <= 0 || L->W <= 0 || L->Fh <= 0 || L->Fw <= 0 || L->Fw > 16 || L->Fh > 16)
        return false;
    a = TcArgs{};
    a.N = L->N; a.C = L->C; a.K = L->K; a.H = L->H; a.W = L->W; a.Fh = L->Fh; a.Fw = L->Fw;
    a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, 1);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, 1);
    a.cbs = L->C / CB; a.taps = L->Fh * L->Fw;
    a.accumulate = L->accumulate; a.act = L->act; a.slope = L->slope;
    a.PW = L->W + (L->pad_l > L->pad_r ? L->pad_l : L->pad_r);
    a.MT = pick_mt(a.K);
    a.k_tiles = (a.K + a.MT - 1) / a.MT;
    a.group = a.Fw; // one kernel row per flush: taps = Fh * Fw is a multiple of it
    a.cg = 1; a.tap_step = 4;
    // few output channels: pixels on the tensor core's M (see the kernel's PIXM paths)
    a.pixm = pixm ? 1 : 0;
    a.merged = (pixm && interleaved_filter(a.K)) ? 1 : 0;
    a.row_skip = 0;
    if (whole)
    {
        // the whole window in one group (TcArgs::row_skip): one channel block, at most 3x3
        if (!a.merged || a.cbs != 1 || a.Fh < 2 || a.taps > 9)
            return false;
        a.group = a.taps;
    }
    a.pool = pool ? 1 : 0;
    if (pool)
    {
        // only the pixel-major tiled plan has the pooled epilogue; even sizes and an even patch width
        if (!pixm || a.accumulate || a.Ho % 2 || a.Wo % 2 || a.Fw % 2 == 0 || a.Ho == 0 || a.Wo == 0 ||
            L->W + (L->pad_l > L->pad_r ? L->pad_l : L->pad_r) <= 64)
            return false;
        return plan_tiled(L, a);
    }
    if (a.Ho == 0 || a.Wo == 0)
        return true;
    if (L->W + (L->pad_l > L->pad_r ? L->pad_l : L->pad_r) > 64)
        return plan_tiled(L, a);
    // 1x1 layer: two channel blocks per patch and per group (see TcArgs::cg)
    if (a.taps == 1 && a.cbs % 2 == 0)
    {
        a.cg = 2; a.cbs /= 2; a.taps = 2; a.group = 2;
    }
    // GEMM columns of one image: the last valid one is (Ho-1)*PW + Wo-1
    const int m_img = (a.Ho - 1) * a.PW + a.Wo;
    const int tiles256 = (m_img + 255) / 256;
    const int gran = a.pixm ? 128 : 64;
    int npx_first = ((m_img + tiles256 - 1) / tiles256 + gran - 1) / gran * gran;
    // First pass: only plans that keep two patches in flight (a layer with few channel blocks
    // per CTA otherwise waits for every patch's load and lo copy), even at a narrower tile;
    // second pass: anything that fits.
    for (int pass = 0; pass < 2; ++pass)
        for (int npx = npx_first; npx >= (pass == 0 ? 128 : gran); npx -= gran)
        {
            a.NPX = npx;
            a.px_tiles = (m_img + npx - 1) / npx;
            const int need = (a.PW - 1) + npx + (a.Fh - 1) * a.PW + (a.Fw - 1);
            a.PR = (need + a.PW - 1) / a.PW;
            if (a.cg > 1)
            {
                // the planes of a patch lie back to back: each must keep the phase of the 64-byte
                // swizzle (a multiple of eight 64-byte rows)
                while ((a.PR * a.PW) % 8)
                    ++a.PR;
                a.tap_step = a.PR * a.PW * 4;
            }
            if (a.PR > 256)
                continue;
            if (fit_rings(a, pass == 0))
                return true;
        }
    return false;
}
bool plan_as(const small_b200_layer *L, TcArgs &a, bool pixm, bool pool = false)
{
    // whole-window groups only where the filter stays resident in shared memory
    if (pixm && plan_as_g(L, a, pixm, pool, true) && (a.w_resident || a.Ho == 0 || a.Wo == 0))
        return true;
    return plan_as_g(L, a, pixm, pool, false);
}
bool plan_shape(const small_b200_layer *L, TcArgs &a)
{
    const bool want_pixm = L && (L->K == 16 || L->K == 32 || L->K == 64);
    if (want_pixm && plan_as(L, a, true))
        return true;
    // the interleaved filter layout is only read by the pixel-major kernel
    if (L && interleaved_filter(L->K))
        return false;
    return plan_as(L, a, false);
}
bool plan(const small_b200_layer *L, TcArgs &a)
{
    if (L && L->Fh == 1 && L->Fw == 1 && L->stride == 1 && !L->pad_t && !L->pad_b && !L->pad_l && !L->pad_r &&
        L->N > 1 && L->H > 0 && L->W > 0 && (long long)L->H * L->W <= 64)
    {
        small_b200_layer V = *L; // the batch as the rows of one image (TcArgs::rows_view)
        V.N = 1; V.H = L->N; V.W = L->H * L->W;
        if (plan_shape(&V, a))
        {
            a.rows_view = 1;
            a.o_kb_stride = (long long)V.W * CB;
            a.o_row_stride = (long long)(L->K / CB) * V.W * CB;
            return true;
        }
    }
    if (!plan_shape(L, a))
        return false;
    a.o_kb_stride = (long long)a.Ho * a.Wo * CB;
    a.o_row_stride = (long long)a.Wo * CB;
    return true;
}
// The convolution with the 2x2 stride-2 max pool `pool` in its epilogue; the strides describe the pooled tensor.
bool plan_pooled(const small_b200_layer *L, const small_b200_layer *pool, TcArgs &a)
{
    if (!L || !pool || !(L->K == 32 || L->K == 64) || L->accumulate)
        return false;
    // the activation is applied after the maximum: it must not decrease (ReLU, or LeakyReLU with a slope >= 0)
    if (L->act == SMALL_B200_ACT_LEAKY && !(L->slope >= 0.f))
        return false;
    if (pool->Fh != 2 || pool->Fw != 2 || pool->stride != 2 || row_stride(pool) != 2 || pool->pad_t || pool->pad_b ||
        pool->pad_l || pool->pad_r)
        return false;
    if (!plan_as(L, a, true, true))
        return false;
    if (pool->H != a.Ho || pool->W != a.Wo || pool->C != L->K || pool->N != L->N)
        return false;
    a.o_kb_stride = (long long)(a.Ho / 2) * (a.Wo / 2) * CB;
    a.o_row_stride = (long long)(a.Wo / 2) * CB;
    return true;
}

int run_tc(const small_b200_layer *L, const small_b200_layer *pool, const float *in, const float *filt_prepared,
           const float *bias, float *out, void *stream);
} // namespace

extern "C"
{
int small_b200_conv2d_f32_tf32x3_supported(const small_b200_layer *L)
{
    TcArgs a;
    return plan(L, a) ? 1 : 0;
}

int small_b200_conv2d_f32_tf32x3_preferred(const small_b200_layer *L)
{
    TcArgs a;
    if (!L || L->C < 16 || !plan(L, a))
        return 0;
    // tiles that run across the images of a batch (1x1 layers on small images, dense heads) are full
    // whatever the image size; otherwise an image must give a tile something to do
    if (a.rows_view)
        return (long long)L->N * L->H * L->W >= 256 ? 1 : 0;
    return (long long)a.Ho * a.Wo >= 9 ? 1 : 0;
}

int small_b200_filter_prepare_tf32x3(const small_b200_layer *L, const float *filt, float *prepared, void *stream)
{
    if (!L || L->C % CB != 0 || L->K % CB != 0 || L->C <= 0 || L->K <= 0 || L->Fh <= 0 || L->Fw <= 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: shape not covered by the tensor-core path.");
    const long long n = (long long)L->K * L->C * L->Fh * L->Fw;
    prepare_filter_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
        n, (L->C / CB) * L->Fh * L->Fw, pick_mt(L->K), L->K, interleaved_filter(L->K) ? 1 : 0, filt, prepared, prepared + n);
    return launched("prepare_filter_kernel");
}

int small_b200_conv2d_f32_tf32x3(const small_b200_layer *L, const float *in, const float *filt_prepared,
                                 const float *bias, float *out, void *stream)
{
    return run_tc(L, nullptr, in, filt_prepared, bias, out, stream);
}

int small_b200_conv2d_maxpool_f32_tf32x3_supported(const small_b200_layer *conv, const small_b200_layer *pool)
{
    TcArgs a;
    return plan_pooled(conv, pool, a) ? 1 : 0;
}

int small_b200_conv2d_maxpool_f32_tf32x3(const small_b200_layer *conv, const small_b200_layer *pool, const float *in,
                                         const float *filt_prepared, const float *bias, float *out, void *stream)
{
    if (!conv || !pool)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D+MaxPool2D<float> (3xTF32) ERROR: null layer.");
    return run_tc(conv, pool, in, filt_prepared, bias, out, stream);
}
} // extern "C"

namespace
{
int run_tc(const small_b200_layer *L, const small_b200_layer *pool, const float *in, const float *filt_prepared,
           const float *bias, float *out, void *stream)
{
    if (int rc = check_window_layer(L, "Conv2D<float>", true, 2))
        return rc;
    TcArgs a;
    if (pool ? !plan_pooled(L, pool, a) : !plan(L, a))
        return fail(SMALL_B200_INVALID_ARGUMENT, pool ? "Conv2D+MaxPool2D<float> (3xTF32) ERROR: shape not covered by the fused tensor-core path."
                                                      : "Conv2D<float> (3xTF32) ERROR: shape not covered by the tensor-core path.");
    if (a.N == 0 || a.Ho == 0 || a.Wo == 0)
        return SMALL_B200_OK;

    CUtensorMap mx;
    {
        // activations [N*cbs][H][W][16 floats]
        const uint64_t dims[4] = {16, (uint64_t)a.W, (uint64_t)a.H, (uint64_t)a.N * a.cbs * a.cg};
        uint64_t strides[3] = {64, (uint64_t)a.W * 64, (uint64_t)a.H * a.W * 64};
        if (a.rows_view) // rows are images (C*P floats apart), planes the channel blocks of one image
        {
            strides[1] = (uint64_t)a.C * a.W * 4;
            strides[2] = (uint64_t)a.W * 64;
        }
        const uint32_t box[4] = {16, (uint32_t)a.PW, (uint32_t)a.PR, (uint32_t)a.cg};
        if (int rc = make_tensor_map(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, in, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
    }
    static PerDeviceOnce configured;
    int dev;
    if (configured.needed(&dev))
    {
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<true, false, true, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        SB_CUDA(cudaFuncSetAttribute(conv_tf32x3_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        configured.mark(dev);
    }
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    const long long tiles = (long long)a.N * a.px_tiles * a.k_tiles;
    if (tiles > 0x7fffffffLL)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<float> (3xTF32) ERROR: too many tiles.");
    a.total_tiles = (int)tiles;
    a.by_px_tiles.set(a.px_tiles); a.by_N.set(a.N); a.by_tiles_x.set(a.tiled ? a.tiles_x : 1); a.by_PW.set(a.PW);
    long long blocks = tiles;
    if (a.persistent && blocks > num_sms())
        blocks = num_sms();
    a.ksplit = 1;
    if (!a.persistent && a.cbs * a.cg >= 64 && a.cbs % 2 == 0)
    {
        // a cluster of two CTAs per tile, each reducing half of the channel blocks, when that
        // shortens the tail: 512 tiles on 148 SMs are 4 rounds, 1024 half tiles are 7 half rounds
        const long long sms = num_sms();
        const long long rounds1 = (tiles + sms - 1) / sms, rounds2 = (2 * tiles + sms - 1) / sms;
        // a 1x1 layer's half tile is too little work to pay for the hand-over between the two CTAs
        // unless the tiles alone leave SMs idle (measured: 512 tiles of 1024->256 at 13x13 0.22 ms
        // whole, 0.25 ms split; 64 tiles of 1024->128 0.050 ms whole, 0.035 ms split)
        if (rounds2 * 100 <= rounds1 * 2 * 93 && (a.cg == 1 || 2 * tiles <= sms))
        {
            a.ksplit = 2;
            blocks = 2 * tiles;
        }
    }
    const float *flo_ = filt_prepared + (size_t)a.K * a.C * a.Fh * a.Fw;
    auto launch_split = [&](const TcArgs &ta, long long nblocks) -> int {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)nblocks); cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = ta.smem_bytes; cfg.stream = as_stream(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        SB_CUDA(cudaLaunchKernelEx(&cfg, conv_tf32x3_kernel<false, true>, mx, filt_prepared, flo_, ta, bias, out, status));
        return SMALL_B200_OK;
    };
    // One tile per CTA and a last wave that fills less than half of the SMs (512 tiles on 148 SMs: three
    // full waves and 68 tiles): that wave runs as clusters of two CTAs that split the reduction, in a
    // launch of its own behind the full waves, and takes a little over half a round instead of a whole
    // one.  (Splitting EVERY tile of such a layer was measured slower: 512 -> 1024 channels at 13x13
    // 0.415 -> 0.425 ms; the exchange between the two CTAs costs about a sixth of a half tile.)
    if (!a.pixm && !a.persistent && a.ksplit == 1 && a.cbs % 2 == 0 && a.cbs >= 8 && a.cg == 1)
    {
        const long long sms = num_sms();
        const long long full = tiles / sms * sms, rem = tiles - full;
        if (full > 0 && rem > 0 && 2 * rem <= sms)
        {
            TcArgs a1 = a;
            a1.tile_base = 0;
            conv_tf32x3_kernel<false, false><<<(unsigned)full, NUM_THREADS, a.smem_bytes, as_stream(stream)>>>(
                mx, filt_prepared, flo_, a1, bias, out, status);
            if (int rc = launched("conv_tf32x3_kernel"))
                return rc;
            TcArgs a2 = a;
            a2.tile_base = (int)full; a2.ksplit = 2;
            if (int rc = launch_split(a2, 2 * rem))
                return rc;
            return launched("conv_tf32x3_kernel");
        }
    }
    const bool whole = a.merged && a.cg == 1 && a.group != a.Fw; // whole-window groups (TcArgs::row_skip)
#define SB_LAUNCH_PIXM(M, P) \
    conv_tf32x3_kernel<true, false, true, M, P><<<(unsigned)blocks, NUM_THREADS, a.smem_bytes, as_stream(stream)>>>( \
        mx, filt_prepared, flo_, a, bias, out, status)
    if (a.pool && whole)
        SB_LAUNCH_PIXM(2, true);
    else if (a.pool && a.merged)
        SB_LAUNCH_PIXM(1, true);
    else if (a.pool)
        SB_LAUNCH_PIXM(0, true);
    else if (whole)
        SB_LAUNCH_PIXM(2, false);
    else if (a.merged)
        SB_LAUNCH_PIXM(1, false);
#undef SB_LAUNCH_PIXM
    else if (a.pixm)
        conv_tf32x3_kernel<true, false, true><<<(unsigned)blocks, NUM_THREADS, a.smem_bytes, as_stream(stream)>>>(
            mx, filt_prepared, filt_prepared + (size_t)a.K * a.C * a.Fh * a.Fw, a, bias, out, status);
    else if (a.persistent)
        conv_tf32x3_kernel<true, false><<<(unsigned)blocks, NUM_THREADS, a.smem_bytes, as_stream(stream)>>>(
            mx, filt_prepared, filt_prepared + (size_t)a.K * a.C * a.Fh * a.Fw, a, bias, out, status);
    else if (a.ksplit == 2)
    {
        if (int rc = launch_split(a, blocks))
            return rc;
    }
    else
        conv_tf32x3_kernel<false, false><<<(unsigned)blocks, NUM_THREADS, a.smem_bytes, as_stream(stream)>>>(
            mx, filt_prepared, filt_prepared + (size_t)a.K * a.C * a.Fh * a.Fw, a, bias, out, status);
    return launched("conv_tf32x3_kernel");
}
} // namespace

// ---------------------------------------------------------------------------------------------
// The same tensor-core convolution for callers that must not allocate device memory.
//
// small_b200_conv2d_f32_tf32x3 needs scratch from its caller: the filter re-laid for the tensor
// core, with its lo copy.  Some callers cannot provide it: code that runs inside
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
    const size_t filt_elems = (size_t)L->K * L->C * L->Fh * L->Fw;
    const size_t need = 2 * filt_elems; // the re-laid filter and its lo copy
    if (need > STATIC_SCRATCH_FLOATS)
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "Conv2D<float> (3xTF32, no-alloc) ERROR: this call needs " + std::to_string(need * 4) +
                        " bytes of scratch (2 x K*C*Fh*Fw filter elements, 4 bytes each) but the "
                        "built-in scratch holds " + std::to_string(STATIC_SCRATCH_FLOATS * 4) +
                        " bytes; use small_b200_conv2d_f32_tf32x3 with caller-provided scratch.");
    float *scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch))
        return rc;
    float *prepared = scratch;
    // Nothing in the scratch has to start from zero: the region this call reads is completely
    // rewritten for the sizes of this call before the convolution reads it.
    if (int rc = small_b200_filter_prepare_tf32x3(L, filt, prepared, stream))
        return rc;
    return small_b200_conv2d_f32_tf32x3(L, in, prepared, bias, out, stream);
}
