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
    long long out_pix_stride, out_plane_stride, out_group_stride; // bytes
    int zero_in, zero_filt, lshift, rshift, mult, k_zero;
};

constexpr int TILE_M = 128;

template <int NT>
__global__ void __launch_bounds__(128)
pw_u8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const PwArgs a, const uint8_t *__restrict__ filt,
                const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int *status)
{
    constexpr uint32_t TMEM_COLS = NT < 32 ? 32 : NT;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar, mma_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int corr[NT];

    uint8_t *sA = smem;                                  // [cbs][128][16]
    uint8_t *sB = smem + (size_t)a.cbs * TILE_M * CB;    // [NT/16][cbs][16][16]
    const uint32_t a_bytes = (uint32_t)a.cbs * TILE_M * CB;
    const uint32_t b_bytes = (uint32_t)(NT / CB) * a.cbs * CB * CB;

    int bid = blockIdx.x;
    const int nb = bid % a.nblocks; bid /= a.nblocks;
    const int tile = bid % a.tiles;
    const int g = bid / a.tiles;
    const int tid = threadIdx.x, warp = tid >> 5;

    if (warp == 0)
    {
        if (tid == 0)
        {
            mbar_init(&full_bar, 1);
            mbar_init(&mma_bar, 1);
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

    if (tid == 0)
    {
        mbar_expect_tx(&full_bar, a_bytes + b_bytes);
        tma_load_3d(sA, &map_a, 0, tile * TILE_M, g * a.cbs, &full_bar);
        tma_load_1d(sB, filt + (size_t)nb * b_bytes, b_bytes, &full_bar);
    }
    bool ok = mbar_wait(&full_bar, 0, status, 1);

    if (tid == 0 && ok)
    {
        tc_fence_after_sync();
        constexpr uint32_t idesc = make_idesc(2 /*s32*/, 0 /*u8*/, 0 /*u8*/, 0 /*A K-major*/, 1 /*B MN-major*/,
                                              TILE_M, NT);
        const uint32_t sa = smem_u32(sA), sb_ = smem_u32(sB);
        for (int j = 0; j < a.cbs / 2; ++j)
        {
            const uint64_t da = make_smem_desc(sa + j * 2 * TILE_M * CB, TILE_M * CB, 8 * CB, 0);
            const uint64_t db = make_smem_desc(sb_ + j * 2 * CB * CB, 8 * CB, a.cbs * CB * CB, 0);
            tc_mma_i8(tmem, da, db, idesc, j > 0 ? 1u : 0u);
        }
        tc_commit(&mma_bar);
    }

    // while the tensor core works: row sum of this thread's pixel, column sums of the filter
    int asum = 0;
    if (ok && a.zero_filt != 0)
    {
        for (int cb = 0; cb < a.cbs; ++cb)
        {
            const uint4 v = *reinterpret_cast<const uint4 *>(sA + ((size_t)cb * TILE_M + tid) * CB);
            asum = (int)__dp4a(v.x, 0x01010101u, (unsigned)asum);
            asum = (int)__dp4a(v.y, 0x01010101u, (unsigned)asum);
            asum = (int)__dp4a(v.z, 0x01010101u, (unsigned)asum);
            asum = (int)__dp4a(v.w, 0x01010101u, (unsigned)asum);
        }
    }
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
    __syncthreads();

    ok = ok && mbar_wait(&mma_bar, 0, status, 2);
    tc_fence_after_sync();
    const int p = tile * TILE_M + tid;
    if (ok)
    {
        const int base = a.zero_filt * asum;
        uint8_t *orow = out + (size_t)g * a.out_group_stride + (size_t)p * a.out_pix_stride;
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 16)
        {
            uint32_t r[16];
            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
            tmem_ld_wait();
            int q[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                q[i] = requant((int)r[i] + base + corr[c0 + i], a.lshift, a.rshift, a.mult);
            if (p < a.P)
            {
                uint4 o;
                o.x = (unsigned)q[0] | ((unsigned)q[1] << 8) | ((unsigned)q[2] << 16) | ((unsigned)q[3] << 24);
                o.y = (unsigned)q[4] | ((unsigned)q[5] << 8) | ((unsigned)q[6] << 16) | ((unsigned)q[7] << 24);
                o.z = (unsigned)q[8] | ((unsigned)q[9] << 8) | ((unsigned)q[10] << 16) | ((unsigned)q[11] << 24);
                o.w = (unsigned)q[12] | ((unsigned)q[13] << 8) | ((unsigned)q[14] << 16) | ((unsigned)q[15] << 24);
                *reinterpret_cast<uint4 *>(orow + (size_t)((nb * NT + c0) / CB) * a.out_plane_stride) = o;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0)
        tmem_dealloc(tmem, TMEM_COLS);
}

template <int NT>
int launch_pw(const CUtensorMap &map, const PwArgs &a, size_t smem, const uint8_t *filt, const int32_t *bias,
              uint8_t *out, cudaStream_t st)
{
    auto kern = pw_u8_tc_kernel<NT>;
    static bool configured = false;
    if (!configured)
    {
        SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        configured = true;
    }
    const long long blocks = (long long)a.groups * a.tiles * a.nblocks;
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    kern<<<(unsigned)blocks, 128, smem, st>>>(map, a, filt, bias, out, status);
    return launched("pw_u8_tc_kernel");
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
    size_t smem = (size_t)cbs * TILE_M * CB + (size_t)nt * L->C;
    if (smem > 96 * 1024)
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
        a.P = L->N; a.groups = 1;
        dims[0] = CB; dims[1] = (uint64_t)L->N; dims[2] = (uint64_t)cbs;
        strides[0] = (uint64_t)cbs * CB; strides[1] = CB;
        a.out_pix_stride = (long long)(L->K / CB) * CB; a.out_plane_stride = CB; a.out_group_stride = 0;
    }
    else
    {
        a.P = HW; a.groups = L->N;
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
    case 128: return launch_pw<128>(map, a, smem, filt, bias, out, st);
    case 64: return launch_pw<64>(map, a, smem, filt, bias, out, st);
    case 32: return launch_pw<32>(map, a, smem, filt, bias, out, st);
    default: return launch_pw<16>(map, a, smem, filt, bias, out, st);
    }
}
} // namespace sb

extern "C" int small_b200_device_status(int *status)
{
    int v = 0;
    SB_CUDA(cudaDeviceSynchronize());
    int *p = sb::device_status_ptr();
    if (p)
        SB_CUDA(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
    *status = v;
    if (v != 0)
        return sb::fail(SMALL_B200_DEVICE_TIMEOUT,
                        "a bounded device-side wait ran out (code " + std::to_string(v) + ")");
    return SMALL_B200_OK;
}
