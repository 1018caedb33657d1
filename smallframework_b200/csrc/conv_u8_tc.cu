// conv_u8_tc.cu -- uint8 pointwise (1x1) convolution and dense layers on the 5th-generation
// tensor cores: tcgen05.mma kind::i8 with TMA-fed shared-memory tiles and int32 accumulators
// in tensor memory, followed by the zero-point correction, bias, fixed-point requantisation
// and clamp of the reference (include/small/q_abstract_layer.hpp:922-938,
// platforms/reference/intrinsics_quint8.h:191-206, :481-531).
//
// Why the packed layout needs no re-layout for the MMA
//   activations [C/16][pixel][16 B]: one TMA box {16 B, 128 pixels, C/16 planes} lands in
//     shared memory as [plane][pixel][16 B]; 8 pixels x 16 B = 128 contiguous bytes is
//     exactly one core matrix of the K-major no-swizzle canonical layout, with 128 B between
//     8-pixel groups (SBO) and 2048 B between the two 16-byte K chunks of one K=32 MMA (LBO);
//   filter [K/16][C/16][16 c][16 k]: 16 output channels contiguous per input channel is the
//     MN-major canonical layout: a core matrix is 8 c-rows x 16 k-bytes = 128 B, the next
//     8 c-rows follow 128 B later (LBO), the next 16 output channels C/16*256 B later (SBO);
//     the whole tile of a CTA is one contiguous run of global memory -> one bulk copy.
//
// Zero points: sum (a+zI)(w+zF) = sum a*w + zF*sum_c a + zI*sum_c w + C*zI*zF.  The MMA gives
// the first term exactly (u8 x u8 -> s32); the row sums of the activation tile and the column
// sums of the filter tile are taken from the shared-memory tiles by the epilogue threads.
#include "tc_common.cuh"

namespace sb
{
static __device__ int g_device_status = 0;

int *device_status_ptr()
{
    static int *ptrs[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64)
        return nullptr;
    if (!ptrs[dev])
    {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess)
            ptrs[dev] = static_cast<int *>(p);
    }
    return ptrs[dev];
}

encode_tiled_fn get_encode_tiled()
{
    static encode_tiled_fn fn = nullptr;
    if (!fn)
    {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    }
    return fn;
}

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, const void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                    CUtensorMapSwizzle swizzle)
{
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc)
        return fail(SMALL_B200_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i)
    {
        d[i] = dims[i]; b[i] = box[i]; e[i] = 1;
        if (i > 0)
            s[i - 1] = strides_bytes[i - 1];
    }
    CUresult r = enc(map, dt, (cuuint32_t)rank, const_cast<void *>(base), d, s, b, e,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(SMALL_B200_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return SMALL_B200_OK;
}
} // namespace sb

namespace
{
using namespace sb;

struct PwArgs
{
    int P;       // pixels per group (one image, or the whole batch when H = W = 1)
    int groups;  // images (1 when the batch is folded into the pixel axis)
    int cbs;     // input channel blocks (C / 16)
    int K;       // output channels
    int tiles;   // ceil(P / 128)
    int nblocks; // K / NT
    int bulk;    // 1: a channel block of a tile is one contiguous run of pixels (plain bulk copies)
    long long out_pix_stride, out_plane_stride, out_group_stride; // bytes
    int zero_in, zero_filt, lshift, rshift, mult, k_zero;
};

constexpr int TILE_M = 128;

// Persistent: a CTA keeps its slice of the filter (and the per-channel correction terms) and
// walks over pixel tiles; loads, MMAs and the epilogue of consecutive tiles overlap through two
// activation stages in shared memory and two accumulator buffers in tensor memory.
//   warps 0..7  epilogue: a thread owns one pixel of the tile (= TMEM lane 32 * (warp % 4) + lane)
//               and one half of the tile's output channels (warp / 4); the epilogue is a chain of
//               dependent steps (barrier, tensor-memory load, requantisation, store), so twice the
//               warps hide twice the latency
//   warp 8      lane 0 issues the TMA loads (and the warp owns the TMEM allocation)
//   warp 9      lane 0 issues the MMAs
constexpr int PW_EPI_WARPS = 8, PW_THREADS = (PW_EPI_WARPS + 2) * 32;
template <int NT>
__global__ void __launch_bounds__(PW_THREADS)
pw_u8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const PwArgs a, const uint8_t *__restrict__ in,
                const uint8_t *__restrict__ filt,
                const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int *status)
{
    constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[2], mma_bar[2], done_bar[2], b_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ __align__(16) int corr[NT];

    const uint32_t a_bytes = (uint32_t)a.cbs * TILE_M * CB;
    const uint32_t b_bytes = (uint32_t)(NT / CB) * a.cbs * CB * CB;
    uint8_t *sA = smem;                   // [stage][cbs][128][16]
    uint8_t *sB = smem + 2 * (size_t)a_bytes; // [NT/16][cbs][16][16]

    const int nb = blockIdx.y;
    const int total = a.groups * a.tiles;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (warp == PW_EPI_WARPS)
    {
        if (lane == 0)
        {
            for (int i = 0; i < 2; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&mma_bar[i], 1); mbar_init(&done_bar[i], PW_EPI_WARPS); }
            mbar_init(&b_bar, 1);
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == PW_EPI_WARPS && lane == 0)
    {
        mbar_expect_tx(&b_bar, b_bytes);
        tma_load_1d(sB, filt + (size_t)nb * b_bytes, b_bytes, &b_bar);
        bool ok = true;
        int i = 0;
        for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++i)
        {
            const int s = i & 1;
            if (i >= 2)
                ok = mbar_wait(&done_bar[s], ((i >> 1) - 1) & 1, status, 3);
            if (!ok)
                break;
            const int tile = item % a.tiles, g = item / a.tiles;
            if (a.bulk)
            {
                // [cb][pixel][16 B] in memory as in shared memory: one run per channel block (a tiled
                // copy with 16-byte rows moves a row every few cycles and set the pace of this kernel);
                // rows past the image keep stale bytes, their results are never stored
                const int rows = (a.P - tile * TILE_M) < TILE_M ? (a.P - tile * TILE_M) : TILE_M;
                mbar_expect_tx(&full_bar[s], (uint32_t)(a.cbs * rows * CB));
                for (int cb = 0; cb < a.cbs; ++cb)
                    tma_load_1d(sA + (size_t)s * a_bytes + (size_t)cb * TILE_M * CB,
                                in + (((size_t)g * a.cbs + cb) * a.P + (size_t)tile * TILE_M) * CB, (uint32_t)(rows * CB),
                                &full_bar[s]);
            }
            else
            {
                mbar_expect_tx(&full_bar[s], a_bytes);
                tma_load_3d(sA + (size_t)s * a_bytes, &map_a, 0, tile * TILE_M, g * a.cbs, &full_bar[s]);
            }
        }
    }
    else if (warp == PW_EPI_WARPS + 1 && lane == 0)
    {
        bool ok = mbar_wait(&b_bar, 0, status, 4);
        constexpr uint32_t idesc = make_idesc(2 /*s32*/, 0 /*u8*/, 0 /*u8*/, 0 /*A K-major*/, 1 /*B MN-major*/,
                                              TILE_M, NT);
        const uint32_t sb_ = smem_u32(sB);
        int i = 0;
        for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++i)
        {
            const int s = i & 1;
            ok = mbar_wait(&full_bar[s], (i >> 1) & 1, status, 1);
            if (!ok)
                break;
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(sA + (size_t)s * a_bytes);
            for (int j = 0; j < a.cbs / 2; ++j)
            {
                const uint64_t da = make_smem_desc(sa + j * 2 * TILE_M * CB, TILE_M * CB, 8 * CB, 0);
                const uint64_t db = make_smem_desc(sb_ + j * 2 * CB * CB, 8 * CB, a.cbs * CB * CB, 0);
                tc_mma_i8(tmem + (uint32_t)(s * NT), da, db, idesc, j > 0 ? 1u : 0u);
            }
            tc_commit(&mma_bar[s]);
        }
    }
    else if (warp < PW_EPI_WARPS)
    {
        const int px_t = (warp & 3) * 32 + lane;      // this thread's pixel of the tile = its TMEM lane
        constexpr int CPW = NT >= 32 ? NT / 2 : NT;  // output channels per warp group
        const int c_begin = (warp >> 2) * CPW;
        // per-channel constants: k_zero + bias + C*zI*zF + zI * (column sum of the filter)
        bool ok = mbar_wait(&b_bar, 0, status, 5);
        if (tid < NT)
        {
            const int kg = nb * NT + tid;
            int c = a.k_zero + (bias ? bias[kg] : 0) + a.cbs * CB * a.zero_in * a.zero_filt;
            if (ok && a.zero_in != 0)
            {
                int wsum = 0;
                const uint8_t *col = sB + (size_t)(tid / CB) * a.cbs * CB * CB + (tid % CB);
                for (int i = 0; i < a.cbs * CB; ++i)
                    wsum += col[i * CB];
                c += a.zero_in * wsum;
            }
            corr[tid] = c;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        int i = 0;
        for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++i)
        {
            const int s = i & 1;
            const int tile = item % a.tiles, g = item / a.tiles;
            ok = mbar_wait(&full_bar[s], (i >> 1) & 1, status, 6);
            if (!ok)
                break;
            // while the tensor core works: row sum of this thread's pixel
            int asum = 0;
            if (a.zero_filt != 0)
            {
                const uint8_t *arow = sA + (size_t)s * a_bytes + (size_t)px_t * CB;
                for (int cb = 0; cb < a.cbs; ++cb)
                {
                    const uint4 v = *reinterpret_cast<const uint4 *>(arow + (size_t)cb * TILE_M * CB);
                    asum = (int)__dp4a(v.x, 0x01010101u, (unsigned)asum);
                    asum = (int)__dp4a(v.y, 0x01010101u, (unsigned)asum);
                    asum = (int)__dp4a(v.z, 0x01010101u, (unsigned)asum);
                    asum = (int)__dp4a(v.w, 0x01010101u, (unsigned)asum);
                }
            }
            ok = mbar_wait(&mma_bar[s], (i >> 1) & 1, status, 2);
            if (!ok)
                break;
            tc_fence_after_sync();
            const int p = tile * TILE_M + px_t;
            const int base = a.zero_filt * asum;
            uint8_t *orow = out + (size_t)g * a.out_group_stride + (size_t)p * a.out_pix_stride;
#pragma unroll
            for (int cc = 0; cc < CPW; cc += 16)
            {
                const int c0 = c_begin + cc;
                if (c0 >= NT)
                    break; // 16 channels per CTA: the second warp group only keeps the barriers' count
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(s * NT + c0), r);
                tmem_ld_wait();
                int q[16];
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4)
                {
                    const int4 cr = *reinterpret_cast<const int4 *>(corr + c0 + 4 * e4); // c0 is a multiple of 16
                    q[4 * e4 + 0] = (int)r[4 * e4 + 0] + base + cr.x;
                    q[4 * e4 + 1] = (int)r[4 * e4 + 1] + base + cr.y;
                    q[4 * e4 + 2] = (int)r[4 * e4 + 2] + base + cr.z;
                    q[4 * e4 + 3] = (int)r[4 * e4 + 3] + base + cr.w;
                }
                const uint4 o = requant_pack16(q, a.lshift, a.rshift, a.mult);
                if (p < a.P)
                {
                    *reinterpret_cast<uint4 *>(orow + (size_t)((nb * NT + c0) / CB) * a.out_plane_stride) = o;
                }
            }
            // stage s of shared memory and buffer s of tensor memory are free again
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&done_bar[s]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == PW_EPI_WARPS)
        tmem_dealloc(tmem, TMEM_COLS);
}

template <int NT>
int launch_pw(const CUtensorMap &map, const PwArgs &a, size_t smem, const uint8_t *in, const uint8_t *filt, const int32_t *bias,
              uint8_t *out, cudaStream_t st)
{
    auto kern = pw_u8_tc_kernel<NT>;
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
    // as many CTAs as fit at once: tensor memory (2 * NT of 512 columns) and shared memory
    int per_sm = 512 / (2 * NT < 32 ? 32 : 2 * NT);
    const int by_smem = (int)((220 * 1024) / (smem + 2048));
    if (per_sm > by_smem)
        per_sm = by_smem;
    if (per_sm > 8)
        per_sm = 8;
    if (per_sm < 1)
        per_sm = 1;
    const long long total = (long long)a.groups * a.tiles;
    long long gx = (long long)num_sms() * per_sm / a.nblocks;
    if (gx < 1)
        gx = 1;
    if (gx > total)
        gx = total;
    dim3 grid((unsigned)gx, (unsigned)a.nblocks);
    kern<<<grid, PW_THREADS, smem, st>>>(map, a, in, filt, bias, out, status);
    return launched("pw_u8_tc_kernel");
}

// ---------------------------------------------------------------------------------------------
// First layer on a ONE-channel image (the 10x4 stride-2 stem of the keyword-spotting network) as
// an im2col GEMM on the tensor core: a kernel row of the window is Fw <= 4 consecutive image
// bytes = one 32-bit word, so pixel p's row of the A tile is Fh words (K = 4*Fh, padded to 64).
// The epilogue threads build the tile of the NEXT image in shared memory while the MMAs of the
// current one run.  Both operands enter as signed (or the activations as unsigned) bytes already
// shifted by their zero points -- zero_filt = -128, zero_in = -128 or 0 -- and padded taps are
// zero bytes, so the accumulator needs no zero-point correction at all.
struct StemArgs
{
    int N, H, W, Ho, Wo, Fh, Fw, stride, pad_t, pad_l, K;
    int pitch, prow; // padded image in shared memory
    int lshift, rshift, mult, k_zero;
};

template <int NT, bool SIGNED_IN>
__global__ void __launch_bounds__(160)
stem_u8_tc_kernel(const StemArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                  const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int *status)
{
    constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;
    constexpr int KCH = 4; // 16-byte chunks of K = 64
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t built_bar[2], mma_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int seed[NT];

    uint8_t *sA = smem;                                   // [stage][chunk 4][128 px][16 B]
    uint8_t *sB = sA + 2 * KCH * TILE_M * CB;             // [chunk 4][NT][16 B]
    uint8_t *sI = sB + KCH * NT * CB;                     // [stage][prow][pitch] padded image
    const int img_bytes = a.prow * a.pitch;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int px = a.Ho * a.Wo;

    if (warp == 4)
    {
        if (lane == 0)
        {
            for (int i = 0; i < 2; ++i) { mbar_init(&built_bar[i], 128); mbar_init(&mma_bar[i], 1); }
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, TMEM_COLS);
        tmem_relinquish();
    }
    // filter -> K-major canonical [chunk][n][16 B]: byte k = kh*4 + kw of output channel n
    for (int i = tid; i < KCH * NT * CB; i += blockDim.x)
    {
        const int b = i % CB, n = (i / CB) % NT, j = i / (CB * NT);
        const int k = j * CB + b, kh = k >> 2, kw = k & 3;
        uint8_t v = 0;
        if (kh < a.Fh && kw < a.Fw && n < a.K) // filter [K/16][1][Fh][Fw][1][16]
            v = filt[((((size_t)(n / CB)) * a.Fh + kh) * a.Fw + kw) * CB + (n % CB)] ^ 0x80u;
        sB[i] = v;
    }
    for (int i = tid; i < 2 * KCH * TILE_M * CB / 16; i += blockDim.x) // rows of missing pixels / taps stay zero
        reinterpret_cast<uint4 *>(sA)[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int i = tid; i < 2 * img_bytes / 4; i += blockDim.x)
        reinterpret_cast<unsigned *>(sI)[i] = 0u;
    if (tid < NT)
        seed[tid] = a.k_zero + ((bias && tid < a.K) ? bias[tid] : 0);
    fence_proxy_async();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    const int first = blockIdx.x, step = gridDim.x;

    if (warp < 4)
    {
        const int p = tid;                 // this thread's pixel = TMEM lane
        const int oh = p / a.Wo, ow = p - oh * a.Wo;
        auto build = [&](int n, int s) {
            // image n -> padded signed image -> this pixel's row of the A tile in stage s
            uint8_t *img = sI + (size_t)s * img_bytes;
            const uint8_t *src = in + (size_t)n * a.H * a.W;
            for (int i = tid; i < a.H * a.W; i += 128)
            {
                const int h = i / a.W, w = i - h * a.W;
                const uint8_t v = src[i];
                img[(h + a.pad_t) * a.pitch + (w + a.pad_l)] = SIGNED_IN ? (uint8_t)(v ^ 0x80u) : v;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (p < px)
            {
                const uint8_t *row = img + (oh * a.stride) * a.pitch + ow * a.stride;
                uint8_t *arow = sA + (size_t)s * KCH * TILE_M * CB + (size_t)p * CB;
                for (int j = 0; j * 4 < a.Fh; ++j)
                {
                    unsigned wv[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                    {
                        const int kh = j * 4 + t;
                        if (kh < a.Fh)
                        {
                            const uint8_t *pw = row + kh * a.pitch;
                            const unsigned *al = reinterpret_cast<const unsigned *>(pw - ((size_t)pw & 3));
                            wv[t] = __funnelshift_r(al[0], al[1], 8 * (unsigned)((size_t)pw & 3));
                            if (a.Fw < 4)
                                wv[t] &= (1u << (8 * a.Fw)) - 1u;
                        }
                    }
                    *reinterpret_cast<uint4 *>(arow + (size_t)j * TILE_M * CB) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            fence_proxy_async();
            mbar_arrive(&built_bar[s]);
        };
        bool ok = true;
        if (first < a.N)
            build(first, 0);
        int i = 0;
        for (int n = first; n < a.N && ok; n += step, ++i)
        {
            const int s = i & 1;
            if (n + step < a.N)
            {
                // stage s^1 was read by the MMAs of image i-1, whose completion this thread has
                // already waited for in the previous iteration
                asm volatile("bar.sync 1, 128;" ::: "memory"); // everyone is done reading image i-1's padded copy
                build(n + step, s ^ 1);
            }
            ok = mbar_wait(&mma_bar[s], (i >> 1) & 1, status, 7);
            if (!ok)
                break;
            tc_fence_after_sync();
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 16)
            {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(s * NT + c0), r);
                tmem_ld_wait();
                int q[16];
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    q[e] = (int)r[e] + seed[c0 + e];
                const uint4 o = requant_pack16(q, a.lshift, a.rshift, a.mult);
                if (p < px && c0 < a.K)
                    *reinterpret_cast<uint4 *>(out + (((size_t)n * (a.K / CB) + c0 / CB) * px + p) * CB) = o;
            }
            tc_fence_before_sync();
        }
    }
    else if (warp == 4 && lane == 0)
    {
        const uint32_t idesc = make_idesc(2 /*s32*/, SIGNED_IN ? 1u : 0u, 1 /*s8*/, 0 /*A K-major*/, 0 /*B K-major*/,
                                          TILE_M, NT);
        const uint32_t sb_ = smem_u32(sB);
        bool ok = true;
        int i = 0;
        for (int n = first; n < a.N && ok; n += step, ++i)
        {
            const int s = i & 1;
            ok = mbar_wait(&built_bar[s], (i >> 1) & 1, status, 8);
            if (!ok)
                break;
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(sA + (size_t)s * KCH * TILE_M * CB);
            for (int j = 0; j < KCH / 2; ++j) // K = 32 per MMA = two 16-byte chunks
            {
                const uint64_t da = make_smem_desc(sa + j * 2 * TILE_M * CB, TILE_M * CB, 8 * CB, 0);
                const uint64_t db = make_smem_desc(sb_ + j * 2 * NT * CB, NT * CB, 8 * CB, 0);
                tc_mma_i8(tmem + (uint32_t)(s * NT), da, db, idesc, j > 0 ? 1u : 0u);
            }
            tc_commit(&mma_bar[s]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4)
        tmem_dealloc(tmem, TMEM_COLS);
}

template <int NT, bool SIGNED_IN>
int launch_stem(const StemArgs &a, size_t smem, const uint8_t *in, const uint8_t *filt, const int32_t *bias,
                uint8_t *out, cudaStream_t st)
{
    auto kern = stem_u8_tc_kernel<NT, SIGNED_IN>;
    static PerDeviceOnce configured;
    int dev;
    if (configured.needed(&dev))
    {
        SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        configured.mark(dev);
    }
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    int per_sm = 512 / (2 * NT < 32 ? 32 : 2 * NT);
    const int by_smem = (int)((220 * 1024) / (smem + 2048));
    if (per_sm > by_smem) per_sm = by_smem;
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    long long grid = (long long)num_sms() * per_sm;
    if (grid > a.N) grid = a.N;
    kern<<<(unsigned)grid, 160, smem, st>>>(a, in, filt, bias, out, status);
    return launched("stem_u8_tc_kernel");
}
} // namespace

namespace sb
{
// Returns -1 when the shape is not covered by the tensor-core path.
int conv2d_u8_tensor_core(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                          const int32_t *bias, uint8_t *out, cudaStream_t st)
{
    if (L->Fh != 1 || L->Fw != 1 || L->stride != 1 || L->pad_t || L->pad_b || L->pad_l || L->pad_r)
        return -1;
    if (L->C % 32 != 0 || L->C > 256 || L->K % CB != 0)
        return -1;
    const int cbs = L->C / CB;
    const int HW = L->H * L->W;
    if (L->N == 0 || HW == 0)
        return SMALL_B200_OK;
    int nt = (L->K % 128 == 0) ? 128 : (L->K % 64 == 0) ? 64 : (L->K % 32 == 0) ? 32 : 16;
    size_t smem = 2 * (size_t)cbs * TILE_M * CB + (size_t)nt * L->C; // two activation stages + the filter slice
    if (smem > 160 * 1024)
        return -1;

    PwArgs a;
    a.cbs = cbs; a.K = L->K; a.nblocks = L->K / nt;
    a.zero_in = L->zero_in; a.zero_filt = L->zero_filt; a.lshift = L->lshift; a.rshift = L->rshift;
    a.mult = L->multiplier; a.k_zero = L->k_zero;
    uint64_t dims[3], strides[2];
    uint32_t box[3] = {CB, TILE_M, (uint32_t)cbs};
    if (HW == 1)
    {
        // dense layer: the batch is the pixel axis; image n holds its planes contiguously
        a.P = L->N; a.groups = 1; a.bulk = 0;
        dims[0] = CB; dims[1] = (uint64_t)L->N; dims[2] = (uint64_t)cbs;
        strides[0] = (uint64_t)cbs * CB; strides[1] = CB;
        a.out_pix_stride = (long long)(L->K / CB) * CB; a.out_plane_stride = CB; a.out_group_stride = 0;
    }
    else
    {
        a.P = HW; a.groups = L->N;
        a.bulk = (reinterpret_cast<uintptr_t>(in) % 16 == 0) ? 1 : 0;
        dims[0] = CB; dims[1] = (uint64_t)HW; dims[2] = (uint64_t)L->N * cbs;
        strides[0] = CB; strides[1] = (uint64_t)HW * CB;
        a.out_pix_stride = CB; a.out_plane_stride = (long long)HW * CB;
        a.out_group_stride = (long long)(L->K / CB) * HW * CB;
    }
    a.tiles = (a.P + TILE_M - 1) / TILE_M;
    CUtensorMap map;
    if (int rc = make_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, in, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    switch (nt)
    {
    case 128: return launch_pw<128>(map, a, smem, in, filt, bias, out, st);
    case 64: return launch_pw<64>(map, a, smem, in, filt, bias, out, st);
    case 32: return launch_pw<32>(map, a, smem, in, filt, bias, out, st);
    default: return launch_pw<16>(map, a, smem, in, filt, bias, out, st);
    }
}
} // namespace sb

namespace sb
{
// The one-channel first layer on the tensor core; -1 when the shape is not covered.
int conv2d_u8_one_channel_tc(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt, const int32_t *bias,
                             uint8_t *out, cudaStream_t st)
{
    if (L->C != 1 || L->zero_filt != -128 || (L->zero_in != 0 && L->zero_in != -128))
        return -1;
    if (L->Fw > 4 || L->Fh > 16 || L->K % CB != 0 || L->K > 128)
        return -1;
    StemArgs a;
    a.N = L->N; a.H = L->H; a.W = L->W; a.Fh = L->Fh; a.Fw = L->Fw; a.stride = L->stride;
    a.pad_t = L->pad_t; a.pad_l = L->pad_l; a.K = L->K;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, L->stride);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    if (a.Ho * a.Wo > TILE_M || a.Ho * a.Wo <= 0)
        return -1;
    if (a.N == 0)
        return SMALL_B200_OK;
    a.pitch = ((L->W + L->pad_l + L->pad_r + 12) + 3) & ~3; // room for the unaligned window read
    a.prow = L->H + L->pad_t + L->pad_b + 1;
    a.lshift = L->lshift; a.rshift = L->rshift; a.mult = L->multiplier; a.k_zero = L->k_zero;
    const int nt = L->K <= 64 ? 64 : 128;
    const size_t smem = 2 * 4 * TILE_M * CB + (size_t)4 * nt * CB + 2 * (size_t)a.prow * a.pitch;
    if (smem > 96 * 1024)
        return -1;
    const bool sgn = L->zero_in != 0;
    if (nt == 64)
        return sgn ? launch_stem<64, true>(a, smem, in, filt, bias, out, st) : launch_stem<64, false>(a, smem, in, filt, bias, out, st);
    return sgn ? launch_stem<128, true>(a, smem, in, filt, bias, out, st) : launch_stem<128, false>(a, smem, in, filt, bias, out, st);
}
} // namespace sb

extern "C" int small_b200_device_status(int *status)
{
    int v = 0;
    SB_CUDA(cudaDeviceSynchronize());
    int *p = sb::device_status_ptr();
    if (p)
        SB_CUDA(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (status)
        *status = v;
    if (v != 0)
    {
        // reported once: the word is cleared so that later kernels wait with their full limits again
        SB_CUDA(cudaMemset(p, 0, sizeof(int)));
        return sb::fail(SMALL_B200_DEVICE_TIMEOUT,
                        "a bounded device-side wait ran out (code " + std::to_string(v) + ")");
    }
    return SMALL_B200_OK;
}

namespace
{
// One warp: a barrier that nobody ever arrives on, a 32-column tensor-memory allocation as the
// tensor-core kernels hold one, and the same bounded wait they use.  The wait runs out after
// `polls` polls by construction, the status word gets `code`, tensor memory is released and the
// kernel returns.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(uint32_t polls, int code, int *status)
{
    __shared__ __align__(8) uint64_t never;
    __shared__ uint32_t tmem_base_s;
    if (threadIdx.x == 0)
    {
        sb::mbar_init(&never, 1);
        sb::fence_barrier_init();
    }
    __syncwarp();
    sb::tmem_alloc(&tmem_base_s, 32);
    sb::tmem_relinquish();
    sb::tc_fence_before_sync();
    __syncwarp();
    sb::tc_fence_after_sync();
    if (threadIdx.x == 0)
        sb::mbar_wait(&never, 0, status, code, polls);
    __syncwarp();
    sb::tmem_dealloc(tmem_base_s, 32);
}
} // namespace

extern "C" int small_b200_selftest_bounded_wait(uint32_t polls, void *stream)
{
    if (polls == 0 || polls > 4096)
        return sb::fail(SMALL_B200_INVALID_ARGUMENT, "selftest_bounded_wait: polls must be in 1..4096");
    int *status = sb::device_status_ptr();
    if (!status)
        return sb::fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    bounded_wait_selftest_kernel<<<1, 32, 0, sb::as_stream(stream)>>>(polls, 99, status);
    return sb::launched("bounded_wait_selftest_kernel");
}
