// peaks.cu -- what the pipes of this GPU deliver when nothing but issue stands in the way: the
// denominators of the per-layer roofline figures.  Three probes, each a loop over operands that
// never leave the SM (registers, shared memory, tensor memory):
//   kind 0  fp32 FMA pipe            independent FFMA chains in registers
//   kind 1  tcgen05 kind::tf32       M = 128, N = 256, K = 8 MMAs on shared-memory operands
//   kind 2  tcgen05 kind::i8         M = 128, N = 256, K = 32
//   kind 3  tcgen05 kind::tf32       M = 128, N = 32: the result is CYCLES PER INSTRUCTION at this GPU's
//   kind 4  tcgen05 kind::i8         M = 128, N = 32  clock, the floor a narrow MMA costs the pipe
// The tensor probes use two issuing threads per CTA, each with its own accumulator in tensor memory
// (one thread alone cannot keep the pipe busy), one CTA per SM.  The reference has no counterpart.
#include "tc_common.cuh"

namespace
{
using namespace sb;

constexpr int FMA_CHAINS = 8;

__global__ void __launch_bounds__(256) ffma_probe_kernel(int iters, float a, float b, float *sink)
{
    float x[FMA_CHAINS];
#pragma unroll
    for (int i = 0; i < FMA_CHAINS; ++i)
        x[i] = (float)(threadIdx.x + i);
    for (int it = 0; it < iters; ++it)
    {
#pragma unroll
        for (int i = 0; i < FMA_CHAINS; ++i)
            x[i] = __fmaf_rn(x[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < FMA_CHAINS; ++i)
        s += x[i];
    if (s == 12345.678f) // never true for the arguments used: keeps the loop alive
        sink[0] = s;
}

template <bool I8, int PROBE_N = 256>
__global__ void __launch_bounds__(128) mma_probe_kernel(int iters, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t done[2];
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // operands: A 128 rows x 32 bytes, B 256 rows x 32 bytes, K-major without swizzle; zeros are as
    // good as any data for the pipe's timing
    for (int i = tid; i < (128 * 32 + PROBE_N * 32 + (PROBE_N < 256 ? 16 * 512 : 0)) / 16; i += 128)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 0)
    {
        if (lane == 0)
        {
            mbar_init(&done[0], 1); mbar_init(&done[1], 1);
            fence_barrier_init();
        }
        __syncwarp();
        tmem_alloc(&tmem_base_s, 512);
        tmem_relinquish();
    }
    fence_proxy_async();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    if ((warp == 1 || warp == 2) && lane == 0)
    {
        const int me = warp - 1;
        const uint32_t idesc = I8 ? make_idesc(2, 0, 0, 0, 0, 128, PROBE_N) : make_idesc(1, 2, 2, 0, 0, 128, PROBE_N);
        // two 16-byte K chunks per operand row: rows 16 bytes apart inside a chunk
        // B first, then the A tile and (narrow probes) the room its 16 positions need
        const uint64_t db = make_smem_desc(smem_u32(smem), PROBE_N * 16, 128, 0);
        const uint64_t da = make_smem_desc(smem_u32(smem + PROBE_N * 32), 128 * 16, 128, 0);
        const uint32_t d = tmem + (uint32_t)(me * PROBE_N);
        for (int it = 0; it < iters; ++it)
        {
            // narrow instructions: a different A tile every time (16 positions 512 bytes apart), as in a
            // kernel that walks over its operands; the wide probes keep one position
            const uint64_t step = PROBE_N < 256 ? (uint64_t)((it & 15) * 32) : 0;
            if (I8)
                tc_mma_i8(d, da + step, db, idesc, it > 0 ? 1u : 0u);
            else
                tc_mma_tf32(d, da + step, db, idesc, it > 0 ? 1u : 0u);
        }
        tc_commit(&done[me]);
        mbar_wait(&done[me], 0, status, 90, 1u << 22);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0)
        tmem_dealloc(tmem, 512);
}
} // namespace

extern "C" int small_b200_peak_probe(int kind, double *tera_ops)
{
    if (!tera_ops || kind < 0 || kind > 4)
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    "peak_probe: kind must be 0 (fp32 FMA), 1 (tf32 MMA), 2 (i8 MMA), 3 or 4 (cycles per narrow tf32 / i8 MMA)");
    int *status = device_status_ptr();
    if (!status)
        return fail(SMALL_B200_CUDA_ERROR, "device status word not available");
    cudaEvent_t e0, e1;
    SB_CUDA(cudaEventCreate(&e0));
    SB_CUDA(cudaEventCreate(&e1));
    const int sms = num_sms();
    double ops = 0.0;
    float best = 1e30f;
    for (int rep = 0; rep < 4; ++rep) // the first run warms up; the best of the others counts
    {
        SB_CUDA(cudaEventRecord(e0, 0));
        if (kind == 0)
        {
            const int iters = 1 << 15, blocks = sms * 8;
            ffma_probe_kernel<<<blocks, 256>>>(iters, 1.0000001f, 1e-7f, nullptr);
            ops = 2.0 * FMA_CHAINS * (double)iters * 256.0 * blocks;
        }
        else
        {
            const int iters = 1 << 14;
            const int n = kind >= 3 ? 32 : 256;
            const size_t smem = 128 * 32 + (size_t)n * 32 + (n < 256 ? 16 * 512 : 0);
            if (kind == 1)
                mma_probe_kernel<false><<<sms, 128, smem>>>(iters, status);
            else if (kind == 2)
                mma_probe_kernel<true><<<sms, 128, smem>>>(iters, status);
            else if (kind == 3)
                mma_probe_kernel<false, 32><<<sms, 128, smem>>>(iters, status);
            else
                mma_probe_kernel<true, 32><<<sms, 128, smem>>>(iters, status);
            ops = 2.0 * 128.0 * n * ((kind == 1 || kind == 3) ? 8.0 : 32.0) * (double)iters * 2.0 * sms;
        }
        if (int rc = launched("peak_probe_kernel"))
            return rc;
        SB_CUDA(cudaEventRecord(e1, 0));
        SB_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        SB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best)
            best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tera_ops = ops / (best * 1e-3) / 1e12;
    if (kind >= 3)
    {
        // two issuing threads per SM, `iters` instructions each: pipe cycles per instruction
        int khz = 0, dev = 0;
        SB_CUDA(cudaGetDevice(&dev));
        SB_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
        *tera_ops = (best * 1e-3) * (khz * 1e3) / (2.0 * (1 << 14));
    }
    return SMALL_B200_OK;
}
