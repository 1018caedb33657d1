// common.cuh -- shared host/device helpers of libsmall_b200.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <string>

#include "small_b200.h"

namespace sb
{
constexpr int CB = SMALL_B200_CB;

extern thread_local std::string g_last_error;
extern std::atomic<uint64_t> g_launches;

inline int fail(int code, const std::string &msg)
{
    g_last_error = msg;
    return code;
}

inline int cuda_fail(cudaError_t e, const char *what)
{
    return fail(e == cudaErrorMemoryAllocation ? SMALL_B200_OUT_OF_MEMORY : SMALL_B200_CUDA_ERROR,
                std::string(what) + ": " + cudaGetErrorString(e));
}

#define SB_CUDA(call)                               \
    do                                              \
    {                                               \
        cudaError_t e_ = (call);                    \
        if (e_ != cudaSuccess)                      \
            return sb::cuda_fail(e_, #call);        \
    } while (0)

// Call after every kernel launch: counts it and turns a launch error into a return code.
inline int launched(const char *name)
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return cuda_fail(e, name);
    return SMALL_B200_OK;
}

inline int out_dim(int in, int pf, int pb, int f, int s)
{
    int o = (in + pf + pb - f) / s + 1; // include/small/utils.hpp:159-165 on the padded extent
    return o > 0 ? o : 0;
}

// Stride along the height (the descriptor's stride_h, 0 = the same as along the width).
inline int row_stride(const small_b200_layer *L) { return L->stride_h > 0 ? L->stride_h : L->stride; }

// Channel block actually used for `channels` input channels (first-layer exception).
inline int eff_block(int channels) { return (channels < CB) ? channels : CB; }

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

inline int num_sms()
{
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64)
        dev = 0;
    if (!sms[dev])
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev] ? sms[dev] : 148;
}

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) belong to a
// device, not to the process: a call site keeps one of these per kernel family and sets its
// attributes the first time each device launches it.
struct PerDeviceOnce
{
    std::atomic<bool> done[64];
    // true when the CURRENT device still needs its set-up; call mark() after it succeeded
    bool needed(int *dev_out)
    {
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64)
            dev = 0;
        *dev_out = dev;
        return !done[dev].load(std::memory_order_acquire);
    }
    void mark(int dev) { done[dev].store(true, std::memory_order_release); }
};

// Shared argument checks of the windowed layers (the reference throws
// std::invalid_argument for these, interface_abstract.hpp:100,218).
int check_window_layer(const small_b200_layer *L, const char *name, bool dense, int max_stride);

// Fixed-point tail of the uint8 path; bit-exact restatement of QUINT8_QUANTIZE_TILE_C
// (include/small/platforms/reference/intrinsics_quint8.h:481-531).
__host__ __device__ inline int32_t requant(int32_t acc, int32_t lshift, int32_t rshift, int32_t mult)
{
    const long long a = (long long)(int32_t)((uint32_t)acc << lshift);
    const long long b = (long long)mult;
    const bool overflow = (a == b) && (a == -2147483648LL);
    const long long prod = a * b;
    const long long nudge = prod >= 0 ? (1LL << 30) : (1LL - (1LL << 30));
    const long long q = (prod + nudge) / (1LL << 31); // C division truncates toward zero
    int32_t v = overflow ? 2147483647 : (int32_t)q;
    const int32_t mask = (int32_t)((1LL << rshift) - 1);
    const int32_t mod = v & mask;
    const int32_t thr = (mask >> 1) + (v < 0 ? -1 : 0);
    v = (v >> rshift) + (mod > thr ? -1 : 0); // the reference's "one" is ~0
    return v > 0 ? (v < 255 ? v : 255) : 0;
}

#ifdef __CUDACC__
// The same tail for a positive multiplier (every quantiser in practice), in 32-bit arithmetic:
// a non-positive input ends at 0 after the clamp, and for a positive one the nudge is 2^30, the
// truncating division a plain shift and the rounding threshold mask >> 1.  About a third of the
// instructions of the general form; bit-identical to it (the uint8 GPU tests compare every layer
// with the oracle, which is pinned to the reference).
static __device__ __noinline__ int32_t requant_general(int32_t acc, int32_t lshift, int32_t rshift, int32_t mult)
{
    return requant(acc, lshift, rshift, mult);
}
// Unclamped result of the tail for a positive multiplier: with t = v * mult + 2^30 the reference's
// two steps (t >> 31, then the rounding shift "floor minus one when the remainder exceeds half")
// collapse into u = t >> (30 + rshift), r = (u >> 1) - (u & 1) for rshift >= 1 (the remainder
// exceeds mask >> 1 exactly when bit rshift-1 of t >> 31 is set) and r = t >> 31 for rshift = 0.
__device__ __forceinline__ int32_t requant_raw(int32_t acc, int32_t lshift, int32_t rshift, int32_t mult)
{
    int32_t v = (int32_t)((uint32_t)acc << lshift);
    v = v > 0 ? v : 0;
    // one wide multiply-add (a 32-bit multiply-high would go to the slow special-function pipe)
    const unsigned long long t = (unsigned long long)(uint32_t)v * (uint32_t)mult + (1ull << 30);
    const uint32_t u = (uint32_t)(t >> (30 + rshift));
    return (int32_t)(u >> 1) - (int32_t)(u & (rshift > 0 ? 1u : 0u));
}
__device__ __forceinline__ int32_t requant_dev(int32_t acc, int32_t lshift, int32_t rshift, int32_t mult)
{
    if (mult <= 0)
        return requant_general(acc, lshift, rshift, mult);
    const int32_t r = requant_raw(acc, lshift, rshift, mult);
    return r < 0 ? 0 : (r > 255 ? 255 : r);
}
// Four results clamped to 0..255 and packed, lowest byte first, by two saturating pack-converts.
__device__ __forceinline__ uint32_t pack4_sat(int32_t r0, int32_t r1, int32_t r2, int32_t r3)
{
    uint32_t hi, d;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(r3), "r"(r2), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(r1), "r"(r0), "r"(hi));
    return d;
}
// Four accumulators -> four output bytes.  The inlined path covers a positive multiplier with
// rshift >= 2 (every quantiser in practice): the shift by 30 + rshift then only needs the high word
// of the product.  Everything else goes through one out-of-line routine so that the unrolled
// epilogues carry a single copy of the arithmetic.
static __device__ __noinline__ uint32_t requant_pack4_general(int32_t a0, int32_t a1, int32_t a2, int32_t a3,
                                                              int32_t lshift, int32_t rshift, int32_t mult)
{
    return pack4_sat(requant(a0, lshift, rshift, mult), requant(a1, lshift, rshift, mult),
                     requant(a2, lshift, rshift, mult), requant(a3, lshift, rshift, mult));
}
// The common quantiser (no left shift, positive multiplier, rshift >= 2): clamp at zero first (a
// non-positive accumulator ends at 0), then one unsigned wide multiply-add t = acc * mult + 2^30,
// u = (t >> 32) >> (rshift - 2) and r = (u >> 1) - (u & 1) as in requant_raw.  (A signed multiply
// without the clamp gives the same bytes after the saturating pack but measured a third slower.)
__device__ __forceinline__ int32_t requant_fast_raw(int32_t acc, int32_t sh /* rshift - 2 */, int32_t mult)
{
    const int32_t v = acc > 0 ? acc : 0;
    const unsigned long long t = (unsigned long long)(uint32_t)v * (uint32_t)mult + (1ull << 30);
    const uint32_t u = (uint32_t)(t >> 32) >> sh;
    return (int32_t)(u >> 1) - (int32_t)(u & 1u);
}
__device__ __forceinline__ bool requant_is_fast(int32_t lshift, int32_t rshift, int32_t mult)
{
    return lshift == 0 && mult > 0 && rshift >= 2;
}
__device__ __forceinline__ uint32_t requant_pack4(int32_t a0, int32_t a1, int32_t a2, int32_t a3, int32_t lshift,
                                                  int32_t rshift, int32_t mult)
{
    if (!requant_is_fast(lshift, rshift, mult))
        return requant_pack4_general(a0, a1, a2, a3, lshift, rshift, mult);
    const int32_t sh = rshift - 2;
    return pack4_sat(requant_fast_raw(a0, sh, mult), requant_fast_raw(a1, sh, mult), requant_fast_raw(a2, sh, mult),
                     requant_fast_raw(a3, sh, mult));
}
// Seeded form of the common quantiser.  Whatever is added to every accumulator of a channel before
// requantisation (bias, zero-point terms, k_zero) is a per-channel constant c, so it can ride in the
// addend of the wide multiply: seed = c * mult + 2^30 and t = acc * mult + seed, ONE instruction on the
// multiplier pipe for "add the constant, multiply, add the nudge".  The clamp at zero is dropped: a
// negative acc + c gives t < 2^30, hence w = t >> 32 <= 0 and a result <= 0, which the saturating pack
// turns into 0 exactly like the clamped form.  With w in hand, u = w >> (rshift - 2) and
// r = (u >> 1) - (u & 1) become r = (w - 2 * (w & bit)) >> (rshift - 1), bit = 1 << (rshift - 2): one
// logic op, one multiply-add, one shift.  Five instructions per output instead of eight, and only
// 2.5 of them on the half-rate integer ALU pipe.
__device__ __forceinline__ long long requant_seed(int32_t c, int32_t mult)
{
    return (long long)c * (long long)mult + (1ll << 30);
}
__device__ __forceinline__ int32_t requant_seeded_raw(int32_t acc, int32_t mult, long long seed, int32_t bit, int32_t sh1)
{
    const long long t = (long long)acc * (long long)mult + seed;
    const int32_t w = (int32_t)(t >> 32);
    return (w - 2 * (w & bit)) >> sh1;
}

// 16 accumulators -> 16 output bytes (one decision for all of them)
__device__ __forceinline__ uint4 requant_pack16(const int32_t *acc, int32_t lshift, int32_t rshift, int32_t mult)
{
    uint4 o;
    if (requant_is_fast(lshift, rshift, mult))
    {
        const int32_t sh = rshift - 2;
        int32_t r[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            r[k] = requant_fast_raw(acc[k], sh, mult);
        o.x = pack4_sat(r[0], r[1], r[2], r[3]);
        o.y = pack4_sat(r[4], r[5], r[6], r[7]);
        o.z = pack4_sat(r[8], r[9], r[10], r[11]);
        o.w = pack4_sat(r[12], r[13], r[14], r[15]);
    }
    else
    {
        o.x = requant_pack4_general(acc[0], acc[1], acc[2], acc[3], lshift, rshift, mult);
        o.y = requant_pack4_general(acc[4], acc[5], acc[6], acc[7], lshift, rshift, mult);
        o.z = requant_pack4_general(acc[8], acc[9], acc[10], acc[11], lshift, rshift, mult);
        o.w = requant_pack4_general(acc[12], acc[13], acc[14], acc[15], lshift, rshift, mult);
    }
    return o;
}
#endif

__device__ __forceinline__ float apply_act(float v, int act, float slope)
{
    if (act == SMALL_B200_ACT_RELU)
        return v > 0.f ? v : 0.f;
    if (act == SMALL_B200_ACT_LEAKY)
        return v > 0.f ? v : v * slope;
    return v;
}
// The three activations as one branch-free form: v > 0 ? v : v * ns, with ns = 1 (none), 0 (ReLU) or the
// slope (LeakyReLU); the product goes through an fma with +0 so that ReLU of a negative value is +0
// like the plain form's.  Bit-identical to apply_act() for every finite v.  For ReLU of -inf or NaN it
// gives NaN (their product with 0) where the plain form gives 0: a form that selects 0 explicitly was
// measured and cost the 3-channel first layer of the 416x416 network 0.10 ms of its 0.27 (the extra
// select changes the register allocation of the whole kernel), so the convolution epilogues keep
// this one and the stand-alone activation kernels use apply_act().
__device__ __forceinline__ float act_neg_scale(int act, float slope)
{
    return act == SMALL_B200_ACT_RELU ? 0.f : (act == SMALL_B200_ACT_LEAKY ? slope : 1.f);
}
__device__ __forceinline__ float apply_act_ns(float v, float ns)
{
    return v > 0.f ? v : __fmaf_rn(v, ns, 0.f);
}
} // namespace sb
