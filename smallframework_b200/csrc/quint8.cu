// quint8.cu -- the uint8 layers on the CUDA cores: dense convolution (general shapes),
// depthwise convolution, max / average pooling and ReLU, each followed by the
// reference's fixed-point requantisation.  Replaces
// small::quint8_detail::abstract_layer (include/small/q_abstract_layer.hpp:884-1571) and the
// QUINT8_{CONV,DW,MAX}_TILE_C / QUINT8_QUANTIZE_TILE_C microkernels
// (platforms/reference/intrinsics_quint8.h:191-289, :481-531).
//
// Arithmetic (bit-exact with the reference): zero points are ADDED, padded taps are
// SKIPPED (they contribute nothing, not even zero_in * w), accumulation is int32 and stays
// in registers for the whole reduction -- the reference parks partial sums in the output
// buffer between input-channel blocks (q_abstract_layer.hpp:1144), which is why its
// callers over-allocate outputs four times; nothing of that is needed here.
#include "common.cuh"

namespace
{
using namespace sb;

struct QArgs
{
    int N, C, K, H, W, Ho, Wo, Fh, Fw, stride, pad_t, pad_l;
    int cib, cbs;
    int zero_in, zero_filt, lshift, rshift, mult, k_zero;
};

__device__ __forceinline__ int byte_of(const uint4 &v, int i)
{
    const unsigned w = (i < 4) ? v.x : (i < 8) ? v.y : (i < 12) ? v.z : v.w;
    return (int)((w >> (8 * (i & 3))) & 0xffu);
}

__device__ __forceinline__ uint4 pack16(const int *v)
{
    uint4 o;
    o.x = (unsigned)v[0] | ((unsigned)v[1] << 8) | ((unsigned)v[2] << 16) | ((unsigned)v[3] << 24);
    o.y = (unsigned)v[4] | ((unsigned)v[5] << 8) | ((unsigned)v[6] << 16) | ((unsigned)v[7] << 24);
    o.z = (unsigned)v[8] | ((unsigned)v[9] << 8) | ((unsigned)v[10] << 16) | ((unsigned)v[11] << 24);
    o.w = (unsigned)v[12] | ((unsigned)v[13] << 8) | ((unsigned)v[14] << 16) | ((unsigned)v[15] << 24);
    return o;
}

// Dense convolution, one thread per output pixel and block of 16 output channels.
// All threads of a CTA share the output-channel block, so filter reads are warp-uniform
// 16-byte loads served by L1.
// PARTIAL (the reference's int32 partial-sum form, one image and one block of output channels): the
// accumulators start from the int32 values the output buffer holds, [pixel][16], and go back there as
// int32; requant_in_place_kernel turns them into bytes afterwards.
template <bool PARTIAL>
__global__ void __launch_bounds__(128)
conv2d_u8_direct_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                        const int32_t *__restrict__ bias, uint8_t *out)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    const int kb = blockIdx.y, n = blockIdx.z;
    if (p >= a.Ho * a.Wo)
        return;
    const int oh = p / a.Wo, ow = p - oh * a.Wo;
    int acc[CB];
    if (PARTIAL)
    {
        const int4 *seed = reinterpret_cast<const int4 *>(out) + (size_t)p * 4;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
        {
            const int4 v = seed[k4];
            acc[4 * k4] = v.x; acc[4 * k4 + 1] = v.y; acc[4 * k4 + 2] = v.z; acc[4 * k4 + 3] = v.w;
        }
    }
    else
    {
#pragma unroll
        for (int k = 0; k < CB; ++k)
            acc[k] = a.k_zero + (bias ? bias[kb * CB + k] : 0);
    }
    const int taps = a.Fh * a.Fw;
    const uint8_t *img = in + (size_t)n * a.C * a.H * a.W;
    const uint8_t *fk = filt + (size_t)kb * a.cbs * taps * a.cib * CB;
    for (int cb = 0; cb < a.cbs; ++cb)
    {
        const uint8_t *plane = img + (size_t)cb * a.H * a.W * a.cib;
        const uint8_t *fcb = fk + (size_t)cb * taps * a.cib * CB;
        for (int kh = 0; kh < a.Fh; ++kh)
        {
            const int ih = oh * a.stride - a.pad_t + kh;
            if (ih < 0 || ih >= a.H)
                continue;
            for (int kw = 0; kw < a.Fw; ++kw)
            {
                const int iw = ow * a.stride - a.pad_l + kw;
                if (iw < 0 || iw >= a.W)
                    continue;
                const uint8_t *px = plane + ((size_t)ih * a.W + iw) * a.cib;
                const uint4 *fw = reinterpret_cast<const uint4 *>(fcb + (size_t)(kh * a.Fw + kw) * a.cib * CB);
                if (a.cib == CB)
                {
                    const uint4 av = *reinterpret_cast<const uint4 *>(px);
#pragma unroll
                    for (int c = 0; c < CB; ++c)
                    {
                        const int x = byte_of(av, c) + a.zero_in;
                        const uint4 wv = __ldg(fw + c);
#pragma unroll
                        for (int k = 0; k < CB; ++k)
                            acc[k] += x * (byte_of(wv, k) + a.zero_filt);
                    }
                }
                else
                {
                    for (int c = 0; c < a.cib; ++c)
                    {
                        const int x = (int)px[c] + a.zero_in;
                        const uint4 wv = __ldg(fw + c);
#pragma unroll
                        for (int k = 0; k < CB; ++k)
                            acc[k] += x * (byte_of(wv, k) + a.zero_filt);
                    }
                }
            }
        }
    }
    if (PARTIAL)
    {
        int4 *dst = reinterpret_cast<int4 *>(out) + (size_t)p * 4;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
            dst[k4] = make_int4(acc[4 * k4], acc[4 * k4 + 1], acc[4 * k4 + 2], acc[4 * k4 + 3]);
        return;
    }
    *reinterpret_cast<uint4 *>(out + (((size_t)n * (a.K / CB) + kb) * a.Ho * a.Wo + p) * CB) =
        requant_pack16(acc, a.lshift, a.rshift, a.mult);
}

// The int32 accumulators [pixels][16] at the start of a buffer become the bytes [pixels][16] at the start
// of the same buffer.  Pixel p's bytes land on the accumulators of pixel p / 4, so the pass runs as ONE
// CTA that walks the pixels in order, a block of 1024 at a time: read, barrier, write, barrier -- every
// accumulator is read before anything is written over it, as in the reference's sequential loop nest.
__global__ void __launch_bounds__(1024) requant_in_place_kernel(int pixels, const QArgs a, uint8_t *buf)
{
    for (int base = 0; base < pixels; base += 1024)
    {
        const int p = base + (int)threadIdx.x;
        int acc[CB];
        if (p < pixels)
        {
            const int4 *src = reinterpret_cast<const int4 *>(buf) + (size_t)p * 4;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
            {
                const int4 v = src[k4];
                acc[4 * k4] = v.x; acc[4 * k4 + 1] = v.y; acc[4 * k4 + 2] = v.z; acc[4 * k4 + 3] = v.w;
            }
        }
        __syncthreads();
        if (p < pixels)
            *reinterpret_cast<uint4 *>(buf + (size_t)p * CB) = requant_pack16(acc, a.lshift, a.rshift, a.mult);
        __syncthreads();
    }
}

// OP: 0 depthwise conv, 1 max pool, 2 average pool; one thread per output pixel and block
// of 16 channels (one 128-bit load per tap, one 128-bit store).
template <int OP, bool PARTIAL = false>
__global__ void __launch_bounds__(256)
window_u8_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                 const int32_t *__restrict__ bias, uint8_t *out)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * (a.C / CB) * a.Ho * a.Wo;
    if (i >= total)
        return;
    const long long o = i;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n*(C/16)+cb
    const int cb = (int)(i % (a.C / CB));
    const uint8_t *plane = in + (size_t)i * a.H * a.W * CB;
    const int h0 = oh * a.stride - a.pad_t, w0 = ow * a.stride - a.pad_l;
    int acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = a.k_zero + ((OP == 0 && bias) ? bias[cb * CB + k] : 0);
    if (PARTIAL) // one image, one channel block: o is the pixel
    {
        const int4 *seed = reinterpret_cast<const int4 *>(out) + (size_t)o * 4;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
        {
            const int4 v = seed[k4];
            acc[4 * k4] = v.x; acc[4 * k4 + 1] = v.y; acc[4 * k4 + 2] = v.z; acc[4 * k4 + 3] = v.w;
        }
    }
    if (OP == 1)
    {
        // q_abstract_layer.hpp:277-288: interior tiles are seeded with the RAW first tap
        const bool interior = h0 >= 0 && w0 >= 0 && h0 + a.Fh <= a.H && w0 + a.Fw <= a.W;
        if (interior)
        {
            const uint4 v = *reinterpret_cast<const uint4 *>(plane + ((size_t)h0 * a.W + w0) * CB);
#pragma unroll
            for (int k = 0; k < CB; ++k)
                acc[k] = byte_of(v, k);
        }
    }
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
            const uint4 v = *reinterpret_cast<const uint4 *>(plane + ((size_t)ih * a.W + iw) * CB);
            if (OP == 0)
            {
                const uint4 f = __ldg(reinterpret_cast<const uint4 *>(
                    filt + (((size_t)cb * a.Fh + kh) * a.Fw + kw) * CB));
#pragma unroll
                for (int k = 0; k < CB; ++k)
                    acc[k] += (byte_of(v, k) + a.zero_in) * (byte_of(f, k) + a.zero_filt);
            }
            else if (OP == 1)
            {
#pragma unroll
                for (int k = 0; k < CB; ++k)
                {
                    const int x = byte_of(v, k) + a.zero_in;
                    acc[k] = x > acc[k] ? x : acc[k];
                }
            }
            else
            {
#pragma unroll
                for (int k = 0; k < CB; ++k)
                    acc[k] += byte_of(v, k) + a.zero_in;
            }
        }
    }
    if (PARTIAL)
    {
        int4 *dst = reinterpret_cast<int4 *>(out) + (size_t)o * 4;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
            dst[k4] = make_int4(acc[4 * k4], acc[4 * k4 + 1], acc[4 * k4 + 2], acc[4 * k4 + 3]);
        return;
    }
    *reinterpret_cast<uint4 *>(out + o * CB) = requant_pack16(acc, a.lshift, a.rshift, a.mult);
}


// ---------------------------------------------------------------------------------------------
// Fast paths for the quantisation every configuration here uses: filter zero point -128 (the
// reference ADDS offsets, so w + zero_filt is a signed byte) and input zero point 0 or -128
// (a + zero_in is an unsigned or a signed byte).  The products then fit dp4a, four per
// instruction.  Padded taps must contribute nothing: their shifted activation is 0.
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b, int c) // unsigned a bytes x signed b bytes
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
template <bool SIGNED_IN>
__device__ __forceinline__ int dp4a_in(unsigned a, unsigned b, int c)
{
    return SIGNED_IN ? __dp4a((int)a, (int)b, c) : dp4a_us(a, b, c);
}

// 4 x 4 byte transpose: r[t] holds 4 channels of tap t; c[j] gets the 4 taps of channel j
__device__ __forceinline__ void transpose4x4(const unsigned r0, const unsigned r1, const unsigned r2,
                                             const unsigned r3, unsigned *c)
{
    const unsigned t0 = __byte_perm(r0, r1, 0x5140), t1 = __byte_perm(r2, r3, 0x5140);
    const unsigned t2 = __byte_perm(r0, r1, 0x7362), t3 = __byte_perm(r2, r3, 0x7362);
    c[0] = __byte_perm(t0, t1, 0x5410); c[1] = __byte_perm(t0, t1, 0x7632);
    c[2] = __byte_perm(t2, t3, 0x5410); c[3] = __byte_perm(t2, t3, 0x7632);
}

// Depthwise convolution: one thread per output pixel and block of 16 channels.  A depthwise sum
// runs over TAPS of one channel while the packed layout keeps CHANNELS of one pixel together, so
// the taps are taken four at a time and byte-transposed (8 PRMT per 4 x 4) into dp4a operands;
// the filter is transposed once per CTA into shared memory as signed bytes.
// QUADS > 0: the number of tap groups is known at compile time and every tap is loaded before
// the arithmetic starts (one round trip to memory instead of one per group).
template <bool SIGNED_IN, int QUADS>
__global__ void __launch_bounds__(256)
dwconv_u8_dp4a_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                      const int32_t *__restrict__ bias, uint8_t *__restrict__ out)
{
    extern __shared__ __align__(16) unsigned sw[]; // [cb][quad][16 ch]: (w ^ 0x80) of 4 taps; then tap -> (kh, kw)
    const int taps = a.Fh * a.Fw, quads = QUADS > 0 ? QUADS : (taps + 3) / 4, cbs = a.C / CB;
    short2 *tap_pos = reinterpret_cast<short2 *>(sw + cbs * quads * CB);
    for (int i = threadIdx.x; i < cbs * quads * CB; i += blockDim.x)
    {
        const int ch = i % CB, q = (i / CB) % quads, cb = i / (CB * quads);
        unsigned wv = 0;
        for (int t = 0; t < 4; ++t)
        {
            const int tap = 4 * q + t;
            if (tap < taps)
                wv |= (unsigned)(filt[((size_t)cb * taps + tap) * CB + ch] ^ 0x80u) << (8 * t);
        }
        sw[i] = wv; // a missing tap keeps weight 0
    }
    for (int i = threadIdx.x; i < quads * 4; i += blockDim.x)
        tap_pos[i] = i < taps ? make_short2((short)(i / a.Fw), (short)(i % a.Fw)) : make_short2(-30000, -30000);
    __syncthreads();

    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * cbs * a.Ho * a.Wo;
    if (i >= total)
        return;
    const long long o = i;
    const int ow = (int)(i % a.Wo); i /= a.Wo;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n*(C/16)+cb
    const int cb = (int)(i % cbs);
    const uint8_t *plane = in + (size_t)i * a.H * a.W * CB;
    const int h0 = oh * a.stride - a.pad_t, w0 = ow * a.stride - a.pad_l;
    int acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = a.k_zero + (bias ? bias[cb * CB + k] : 0);
    const uint4 *wq = reinterpret_cast<const uint4 *>(sw + (size_t)cb * quads * CB);
    if (QUADS > 0)
    {
        uint4 v[QUADS > 0 ? QUADS * 4 : 1];
#pragma unroll
        for (int t = 0; t < QUADS * 4; ++t)
        {
            const short2 pos = tap_pos[t];
            const int ih = h0 + pos.x, iw = w0 + pos.y;
            v[t] = make_uint4(0u, 0u, 0u, 0u);
            if (pos.x >= 0 && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
            {
                v[t] = *reinterpret_cast<const uint4 *>(plane + ((size_t)ih * a.W + iw) * CB);
                if (SIGNED_IN)
                {
                    v[t].x ^= 0x80808080u; v[t].y ^= 0x80808080u; v[t].z ^= 0x80808080u; v[t].w ^= 0x80808080u;
                }
            }
        }
#pragma unroll
        for (int q = 0; q < QUADS; ++q)
        {
#pragma unroll
            for (int g = 0; g < 4; ++g)
            {
                unsigned c[4];
                const unsigned r0 = g == 0 ? v[4 * q].x : g == 1 ? v[4 * q].y : g == 2 ? v[4 * q].z : v[4 * q].w;
                const unsigned r1 = g == 0 ? v[4 * q + 1].x : g == 1 ? v[4 * q + 1].y : g == 2 ? v[4 * q + 1].z : v[4 * q + 1].w;
                const unsigned r2 = g == 0 ? v[4 * q + 2].x : g == 1 ? v[4 * q + 2].y : g == 2 ? v[4 * q + 2].z : v[4 * q + 2].w;
                const unsigned r3 = g == 0 ? v[4 * q + 3].x : g == 1 ? v[4 * q + 3].y : g == 2 ? v[4 * q + 3].z : v[4 * q + 3].w;
                transpose4x4(r0, r1, r2, r3, c);
                const uint4 w4 = wq[q * 4 + g];
                acc[4 * g + 0] = dp4a_in<SIGNED_IN>(c[0], w4.x, acc[4 * g + 0]);
                acc[4 * g + 1] = dp4a_in<SIGNED_IN>(c[1], w4.y, acc[4 * g + 1]);
                acc[4 * g + 2] = dp4a_in<SIGNED_IN>(c[2], w4.z, acc[4 * g + 2]);
                acc[4 * g + 3] = dp4a_in<SIGNED_IN>(c[3], w4.w, acc[4 * g + 3]);
            }
        }
    }
    else
    for (int q = 0; q < quads; ++q)
    {
        unsigned r[4][4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
        {
            const short2 pos = tap_pos[4 * q + t];
            const int ih = h0 + pos.x, iw = w0 + pos.y;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (pos.x >= 0 && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
            {
                v = *reinterpret_cast<const uint4 *>(plane + ((size_t)ih * a.W + iw) * CB);
                if (SIGNED_IN)
                {
                    v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u;
                }
            }
            r[t][0] = v.x; r[t][1] = v.y; r[t][2] = v.z; r[t][3] = v.w;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
        {
            unsigned c[4];
            transpose4x4(r[0][g], r[1][g], r[2][g], r[3][g], c);
            const uint4 w4 = wq[q * 4 + g];
            acc[4 * g + 0] = dp4a_in<SIGNED_IN>(c[0], w4.x, acc[4 * g + 0]);
            acc[4 * g + 1] = dp4a_in<SIGNED_IN>(c[1], w4.y, acc[4 * g + 1]);
            acc[4 * g + 2] = dp4a_in<SIGNED_IN>(c[2], w4.z, acc[4 * g + 2]);
            acc[4 * g + 3] = dp4a_in<SIGNED_IN>(c[3], w4.w, acc[4 * g + 3]);
        }
    }
    *reinterpret_cast<uint4 *>(out + o * CB) = requant_pack16(acc, a.lshift, a.rshift, a.mult);
}

// Depthwise 3x3, stride 1, a row strip per thread: TW neighbouring outputs of one row x 8
// channels.  The three taps of a kernel COLUMN of one input pixel are transposed once and serve
// the (up to) three outputs that see this input column through kw = 0, 1, 2, so a strip of TW
// outputs costs TW + 2 transposes instead of 3 * TW, and the index arithmetic is paid once per
// strip.  Filter words in shared memory: [cb][half][kw][8 ch] = (w[0][kw], w[1][kw], w[2][kw], 0)
// as signed bytes.
template <bool SIGNED_IN, int TW>
__global__ void __launch_bounds__(256, 3)
dwconv3x3_u8_rows_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                         const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int strips, int pad_t, int pad_l)
{
    extern __shared__ __align__(16) unsigned sw[]; // [cb][half][kw][8]
    const int cbs = a.C / CB;
    for (int i = threadIdx.x; i < cbs * 48; i += blockDim.x)
    {
        const int j = i % 8, kw = (i / 8) % 3, half = (i / 24) % 2, cb = i / 48;
        const int ch = half * 8 + j;
        unsigned wv = 0;
        for (int kh = 0; kh < 3; ++kh)
            wv |= (unsigned)(filt[(((size_t)cb * 3 + kh) * 3 + kw) * CB + ch] ^ 0x80u) << (8 * kh);
        sw[i] = wv;
    }
    __syncthreads();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.N * cbs * a.Ho * strips * 2;
    if (i >= total)
        return;
    const int half = (int)(i & 1); i >>= 1;
    const int strip = (int)(i % strips); i /= strips;
    const int oh = (int)(i % a.Ho); i /= a.Ho; // i = n * cbs + cb
    const int cb = (int)(i % cbs);
    const uint8_t *plane = in + (size_t)i * a.H * a.W * CB + half * 8;
    const int ow0 = strip * TW;
    unsigned wreg[3][8];
    {
        const uint4 *wp = reinterpret_cast<const uint4 *>(sw + ((size_t)cb * 2 + half) * 24);
#pragma unroll
        for (int kw = 0; kw < 3; ++kw)
        {
            const uint4 w0 = wp[kw * 2], w1 = wp[kw * 2 + 1];
            wreg[kw][0] = w0.x; wreg[kw][1] = w0.y; wreg[kw][2] = w0.z; wreg[kw][3] = w0.w;
            wreg[kw][4] = w1.x; wreg[kw][5] = w1.y; wreg[kw][6] = w1.z; wreg[kw][7] = w1.w;
        }
    }
    int acc[TW][8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const int s0 = a.k_zero + (bias ? bias[cb * CB + half * 8 + j] : 0);
#pragma unroll
        for (int o = 0; o < TW; ++o)
            acc[o][j] = s0;
    }
    const int ih0 = oh - pad_t;
    const bool rok0 = ih0 >= 0 && ih0 < a.H, rok1 = ih0 + 1 >= 0 && ih0 + 1 < a.H, rok2 = ih0 + 2 >= 0 && ih0 + 2 < a.H;
    const uint8_t *row0 = plane + (size_t)ih0 * a.W * CB, *row1 = row0 + (size_t)a.W * CB, *row2 = row1 + (size_t)a.W * CB;
#pragma unroll
    for (int x = 0; x < TW + 2; ++x)
    {
        const int xi = ow0 - pad_l + x;
        if (xi < 0 || xi >= a.W)
            continue; // a padded column adds nothing
        uint2 r0 = make_uint2(0u, 0u), r1 = make_uint2(0u, 0u), r2 = make_uint2(0u, 0u);
        if (rok0) r0 = *reinterpret_cast<const uint2 *>(row0 + (size_t)xi * CB);
        if (rok1) r1 = *reinterpret_cast<const uint2 *>(row1 + (size_t)xi * CB);
        if (rok2) r2 = *reinterpret_cast<const uint2 *>(row2 + (size_t)xi * CB);
        if (SIGNED_IN)
        {
            if (rok0) { r0.x ^= 0x80808080u; r0.y ^= 0x80808080u; }
            if (rok1) { r1.x ^= 0x80808080u; r1.y ^= 0x80808080u; }
            if (rok2) { r2.x ^= 0x80808080u; r2.y ^= 0x80808080u; }
        }
        unsigned c[8];
        transpose4x4(r0.x, r1.x, r2.x, 0u, c);
        transpose4x4(r0.y, r1.y, r2.y, 0u, c + 4);
#pragma unroll
        for (int kw = 0; kw < 3; ++kw)
        {
            const int o = x - kw; // output o of the strip sees input column x through tap column kw
            if (o >= 0 && o < TW)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    acc[o][j] = dp4a_in<SIGNED_IN>(c[j], wreg[kw][j], acc[o][j]);
            }
        }
    }
    uint8_t *orow = out + (((size_t)i * a.Ho + oh) * a.Wo) * CB + half * 8;
#pragma unroll
    for (int o = 0; o < TW; ++o)
    {
        if (ow0 + o < a.Wo)
        {
            uint2 v;
            v.x = requant_pack4(acc[o][0], acc[o][1], acc[o][2], acc[o][3], a.lshift, a.rshift, a.mult);
            v.y = requant_pack4(acc[o][4], acc[o][5], acc[o][6], acc[o][7], a.lshift, a.rshift, a.mult);
            *reinterpret_cast<uint2 *>(orow + (size_t)(ow0 + o) * CB) = v;
        }
    }
}

// Dense convolution whose whole reduction is at most 32 bytes: a 1x1 layer on 16 channels, or a first
// layer (1..3 channels, [H][W][C] image) whose window holds at most 32 values, e.g. 3x3 on 3 channels.
// These are streaming layers -- one 16-byte load (or a few byte loads) and one 16-byte store per pixel
// and block of output channels -- with too little arithmetic for the tensor core to matter.  A thread
// makes one output pixel: its reduction row sits in up to eight registers of four bytes, the filter in
// shared memory as words of four reduction bytes, [word][output channel], so one 128-bit broadcast
// fetch feeds four dp4a.  Filter zero point -128, input zero point 0 or -128 (operands enter shifted);
// taps outside the image are zero bytes, i.e. skipped, as in the reference.
// FIX333: the 3x3 window on 3 channels.  A kernel row of the window is 9 contiguous bytes of the
// [H][W][3] image: three aligned 32-bit loads and two funnel shifts instead of nine byte loads; rows at
// the left border, or whose aligned reads would pass the end of the buffer, take the byte path.
template <bool SIGNED_IN, bool FIRST, bool FIX333 = false>
__global__ void __launch_bounds__(256)
conv2d_u8_onestep_kernel(const QArgs a, int words, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                         const int32_t *__restrict__ bias, uint8_t *__restrict__ out)
{
    extern __shared__ __align__(16) unsigned smem_u[]; // [K/16][words][16 k]
    const int R = a.Fh * a.Fw * a.C; // reduction length in bytes (<= 32)
    const int kbs = a.K / CB;
    for (int i = threadIdx.x; i < kbs * words * CB; i += blockDim.x)
    {
        const int k = i % CB, j = (i / CB) % words, kb = i / (CB * words);
        unsigned wv = 0;
        for (int t = 0; t < 4; ++t)
        {
            const int r = 4 * j + t;
            if (r < R) // filter [K/16][R rows][16 k] for both layouts
                wv |= (unsigned)(filt[((size_t)kb * R + r) * CB + k] ^ 0x80u) << (8 * t);
        }
        smem_u[i] = wv;
    }
    __syncthreads();
    const long long total = (long long)a.N * a.Ho * a.Wo;
    const int hw = a.Ho * a.Wo;
    // a CTA keeps its copy of the filter for many pixels
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x)
    {
    const int n = (int)(g / hw), p = (int)(g - (long long)n * hw);
    const int oh = p / a.Wo, ow = p - oh * a.Wo;
    const int ih0 = oh * a.stride - a.pad_t, iw0 = ow * a.stride - a.pad_l;
    unsigned x[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    bool gathered = false;
    if (FIRST && FIX333)
    {
        const uint8_t *img = in + (size_t)n * 3 * a.H * a.W;
        const uint8_t *in_end = in + (size_t)a.N * 3 * a.H * a.W;
        const uint8_t *last = img + ((size_t)(ih0 + 2 < a.H ? ih0 + 2 : a.H - 1) * a.W + iw0) * 3;
        if (iw0 >= 0 && ih0 + 2 >= 0 && (reinterpret_cast<uintptr_t>(last) & ~(uintptr_t)3) + 12 <= reinterpret_cast<uintptr_t>(in_end))
        {
            const int vb = (a.W - iw0) >= 3 ? 9 : (a.W - iw0) * 3; // bytes of a row's run inside the image
            const unsigned f = SIGNED_IN ? 0x80808080u : 0u;
            unsigned r0[3], r1[3], r2[3];
#pragma unroll
            for (int kh = 0; kh < 3; ++kh)
            {
                const int ih = ih0 + kh;
                r0[kh] = r1[kh] = r2[kh] = 0u;
                if (ih >= 0 && ih < a.H)
                {
                    const uintptr_t addr = reinterpret_cast<uintptr_t>(img + ((size_t)ih * a.W + iw0) * 3);
                    const unsigned *wp = reinterpret_cast<const unsigned *>(addr & ~(uintptr_t)3);
                    const unsigned sh = (unsigned)(addr & 3) * 8;
                    const unsigned w0 = wp[0], w1 = wp[1], w2 = wp[2];
                    r0[kh] = __funnelshift_r(w0, w1, sh) ^ f;
                    r1[kh] = __funnelshift_r(w1, w2, sh) ^ f;
                    r2[kh] = ((w2 >> sh) ^ f) & 0xffu;
                    if (vb <= 6) { r2[kh] = 0u; r1[kh] &= 0x0000ffffu; }
                    if (vb <= 3) { r1[kh] = 0u; r0[kh] &= 0x00ffffffu; }
                }
            }
            x[0] = r0[0]; x[1] = r1[0];
            x[2] = r2[0] | (r0[1] << 8);
            x[3] = (r0[1] >> 24) | (r1[1] << 8);
            x[4] = (r1[1] >> 24) | (r2[1] << 8) | (r0[2] << 16);
            x[5] = (r0[2] >> 16) | (r1[2] << 16);
            x[6] = (r1[2] >> 16) | (r2[2] << 16);
            gathered = true;
        }
    }
    if (FIRST && !gathered)
    {
        const uint8_t *img = in + (size_t)n * a.C * a.H * a.W;
        int kh = 0, kw = 0, c = 0;
#pragma unroll
        for (int r = 0; r < 32; ++r) // unrolled: x[] stays in registers
        {
            const int ih = ih0 + kh, iw = iw0 + kw;
            if (r < R && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W)
            {
                const unsigned v = (unsigned)img[((size_t)ih * a.W + iw) * a.C + c] ^ (SIGNED_IN ? 0x80u : 0u);
                x[r >> 2] |= v << (8 * (r & 3));
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
    if (!FIRST && ih0 >= 0 && ih0 < a.H && iw0 >= 0 && iw0 < a.W) // 1x1 window on one block of 16 channels
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(in + (((size_t)n * a.H + ih0) * a.W + iw0) * CB);
        const unsigned f = SIGNED_IN ? 0x80808080u : 0u;
        x[0] = v.x ^ f; x[1] = v.y ^ f; x[2] = v.z ^ f; x[3] = v.w ^ f;
    }
    uint8_t *o = out + ((size_t)n * kbs * hw + p) * CB;
    for (int kb = 0; kb < kbs; ++kb)
    {
        int acc[CB];
#pragma unroll
        for (int k = 0; k < CB; ++k)
            acc[k] = a.k_zero + (bias ? bias[kb * CB + k] : 0);
        const uint4 *w4 = reinterpret_cast<const uint4 *>(smem_u + (size_t)kb * words * CB);
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            if (j >= words)
                break;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
            {
                const uint4 wv = w4[j * 4 + k4];
                acc[4 * k4 + 0] = dp4a_in<SIGNED_IN>(x[j], wv.x, acc[4 * k4 + 0]);
                acc[4 * k4 + 1] = dp4a_in<SIGNED_IN>(x[j], wv.y, acc[4 * k4 + 1]);
                acc[4 * k4 + 2] = dp4a_in<SIGNED_IN>(x[j], wv.z, acc[4 * k4 + 2]);
                acc[4 * k4 + 3] = dp4a_in<SIGNED_IN>(x[j], wv.w, acc[4 * k4 + 3]);
            }
        }
        *reinterpret_cast<uint4 *>(o + (size_t)kb * hw * CB) = requant_pack16(acc, a.lshift, a.rshift, a.mult);
    }
    }
}

// Dense convolution of a ONE-channel image (the first layer of the keyword-spotting network):
// the Fw taps of a kernel row are consecutive bytes of the image, so a row of the window is one
// (unaligned) 32-bit word per 4 taps and feeds dp4a directly.  A CTA takes IMGS images: it
// keeps them zero-padded in shared memory (shifted to signed bytes when zero_in = -128) next to
// the filter as [kb][kh][quad][16 k] words of 4 kw-bytes; a thread makes one pixel x 16 channels.
constexpr int C1_IMGS = 2;
template <bool SIGNED_IN>
__global__ void __launch_bounds__(256)
conv2d_u8_c1_dp4a_kernel(const QArgs a, const uint8_t *__restrict__ in, const uint8_t *__restrict__ filt,
                         const int32_t *__restrict__ bias, uint8_t *__restrict__ out, int pitch, int prow)
{
    extern __shared__ __align__(16) unsigned smem_u[];
    const int quads = (a.Fw + 3) / 4, kbs = a.K / CB;
    unsigned *sw = smem_u;                                    // [kb][kh][quad][16]
    uint8_t *simg = reinterpret_cast<uint8_t *>(sw + (size_t)kbs * a.Fh * quads * CB); // [img][prow][pitch]
    const int n0 = blockIdx.x * C1_IMGS;
    const int imgs = (a.N - n0) < C1_IMGS ? (a.N - n0) : C1_IMGS;
    for (int i = threadIdx.x; i < kbs * a.Fh * quads * CB; i += blockDim.x)
    {
        const int k = i % CB, q = (i / CB) % quads, kh = (i / (CB * quads)) % a.Fh, kb = i / (CB * quads * a.Fh);
        unsigned wv = 0;
        for (int t = 0; t < 4; ++t)
        {
            const int kw = 4 * q + t;
            if (kw < a.Fw) // filter [K/16][1][Fh][Fw][1][16]
                wv |= (unsigned)(filt[(((size_t)kb * a.Fh + kh) * a.Fw + kw) * CB + k] ^ 0x80u) << (8 * t);
        }
        sw[i] = wv;
    }
    const int img_bytes = prow * pitch;
    for (int i = threadIdx.x; i < C1_IMGS * img_bytes / 4; i += blockDim.x)
        reinterpret_cast<unsigned *>(simg)[i] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < imgs * a.H * a.W; i += blockDim.x)
    {
        const int im = i / (a.H * a.W), p = i - im * a.H * a.W;
        const int h = p / a.W, w = p - h * a.W;
        const uint8_t v = in[(size_t)(n0 + im) * a.H * a.W + p];
        simg[(size_t)im * img_bytes + (h + a.pad_t) * pitch + (w + a.pad_l)] = SIGNED_IN ? (uint8_t)(v ^ 0x80u) : v;
    }
    __syncthreads();
    const int px = a.Ho * a.Wo;
    const int items = imgs * kbs * px;
    for (int it = threadIdx.x; it < items; it += blockDim.x)
    {
        const int p = it % px, kb = (it / px) % kbs, im = it / (px * kbs);
        const int oh = p / a.Wo, ow = p - oh * a.Wo;
        int acc[CB];
#pragma unroll
        for (int k = 0; k < CB; ++k)
            acc[k] = a.k_zero + (bias ? bias[kb * CB + k] : 0);
        const uint8_t *row = simg + (size_t)im * img_bytes + (oh * a.stride) * pitch + ow * a.stride;
        const uint4 *wk = reinterpret_cast<const uint4 *>(sw + (size_t)kb * a.Fh * quads * CB);
        for (int kh = 0; kh < a.Fh; ++kh, row += pitch)
        {
            for (int q = 0; q < quads; ++q)
            {
                const uint8_t *pw = row + 4 * q;
                const unsigned *al = reinterpret_cast<const unsigned *>(pw - ((size_t)pw & 3));
                const unsigned aw = __funnelshift_r(al[0], al[1], 8 * (unsigned)((size_t)pw & 3));
                const uint4 *w4 = wk + (kh * quads + q) * 4;
#pragma unroll
                for (int g = 0; g < 4; ++g)
                {
                    const uint4 wv = w4[g];
                    acc[4 * g + 0] = dp4a_in<SIGNED_IN>(aw, wv.x, acc[4 * g + 0]);
                    acc[4 * g + 1] = dp4a_in<SIGNED_IN>(aw, wv.y, acc[4 * g + 1]);
                    acc[4 * g + 2] = dp4a_in<SIGNED_IN>(aw, wv.z, acc[4 * g + 2]);
                    acc[4 * g + 3] = dp4a_in<SIGNED_IN>(aw, wv.w, acc[4 * g + 3]);
                }
            }
        }
        *reinterpret_cast<uint4 *>(out + (((size_t)(n0 + im) * kbs + kb) * px + p) * CB) =
            requant_pack16(acc, a.lshift, a.rshift, a.mult);
    }
}

// Global average pool (window = whole image, no padding): one warp per image and 16-channel
// block; lanes stride over the pixels, then a shuffle tree adds the 16 channel sums.
__global__ void __launch_bounds__(256)
global_avgpool_u8_kernel(const QArgs a, const uint8_t *__restrict__ in, uint8_t *__restrict__ out)
{
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long planes = (long long)a.N * (a.C / CB);
    if (warp >= planes)
        return;
    const int px = a.H * a.W;
    const uint4 *plane = reinterpret_cast<const uint4 *>(in + (size_t)warp * px * CB);
    int acc[CB];
#pragma unroll
    for (int k = 0; k < CB; ++k)
        acc[k] = 0;
    for (int p = lane; p < px; p += 32)
    {
        const uint4 v = plane[p];
#pragma unroll
        for (int k = 0; k < CB; ++k)
            acc[k] += byte_of(v, k);
    }
#pragma unroll
    for (int k = 0; k < CB; ++k)
    {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], off);
        acc[k] = requant_dev(acc[k] + px * a.zero_in + a.k_zero, a.lshift, a.rshift, a.mult);
    }
    if (lane == 0)
        *reinterpret_cast<uint4 *>(out + (size_t)warp * CB) = pack16(acc);
}

__global__ void __launch_bounds__(256)
relu_u8_kernel(long long n16, const QArgs a, const uint8_t *in, uint8_t *out) // in may alias out
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride)
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(in + i * 16);
        int r[CB];
#pragma unroll
        for (int k = 0; k < CB; ++k)
        {
            const int x = byte_of(v, k) + a.zero_in;
            r[k] = requant_dev(x > a.k_zero ? x : a.k_zero, a.lshift, a.rshift, a.mult);
        }
        *reinterpret_cast<uint4 *>(out + i * 16) = pack16(r);
    }
}

void fill(const small_b200_layer *L, QArgs &a, bool dense)
{
    a.N = L->N; a.C = L->C; a.K = dense ? L->K : L->C; a.H = L->H; a.W = L->W;
    a.Fh = L->Fh; a.Fw = L->Fw; a.stride = L->stride; a.pad_t = L->pad_t; a.pad_l = L->pad_l;
    a.Ho = out_dim(L->H, L->pad_t, L->pad_b, L->Fh, L->stride);
    a.Wo = out_dim(L->W, L->pad_l, L->pad_r, L->Fw, L->stride);
    a.cib = dense ? eff_block(L->C) : CB;
    a.cbs = L->C / a.cib;
    a.zero_in = L->zero_in; a.zero_filt = L->zero_filt; a.lshift = L->lshift;
    a.rshift = L->rshift; a.mult = L->multiplier; a.k_zero = L->k_zero;
}

int check_quant(const small_b200_layer *L, const char *name)
{
    if (L->lshift < 0 || L->lshift > 31 || L->rshift < 0 || L->rshift > 31)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: shift out of range.");
    if (row_stride(L) != L->stride)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: stride unsupported (a row stride of its own "
                                                                      "is provided for the fp32 layers only).");
    return SMALL_B200_OK;
}

// The reference's quint8 Partial forms (interface_abstract.hpp:595-767 PartialConv2D, :1194
// PartialDepthwiseConv2D) reuse the uint8 output buffer as int32 storage: the accumulators of output
// channel block k start at BYTE k * Ho*Wo*block and are four times as long as the block's bytes
// (q_abstract_layer.hpp:1135-1144), so the accumulators of one block lie over those of the next three and
// the form has a defined meaning for ONE block of output channels only -- 16 channels on this platform --
// and one image.  There: out holds int32 [Ho*Wo][16] on entry and the bytes [Ho*Wo][16] of
// requantise(entry + convolution) at its start on return.  Anything else is refused.
int check_partial_u8(const small_b200_layer *L, const char *name, int channels, const int32_t *bias)
{
    if (channels != CB || L->N != 1)
        return fail(SMALL_B200_INVALID_ARGUMENT,
                    std::string(name) + " ERROR: the int32 partial sums of different blocks of output channels (and of "
                                        "different images) overlap inside the output buffer; only 16 output channels "
                                        "and one image have a defined result.");
    if (bias)
        return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: the partial-sum form takes no bias.");
    return SMALL_B200_OK;
}

template <int OP>
int launch_window(const small_b200_layer *L, const char *name, int max_stride, const uint8_t *in,
                  const uint8_t *filt, const int32_t *bias, uint8_t *out, void *stream)
{
    if (int rc = check_window_layer(L, name, false, max_stride))
        return rc;
    if (int rc = check_quant(L, name))
        return rc;
    QArgs a; fill(L, a, false);
    const long long items = (long long)a.N * (a.C / CB) * a.Ho * a.Wo;
    if (L->accumulate)
    {
        if (OP != 0)
            return fail(SMALL_B200_INVALID_ARGUMENT, std::string(name) + " ERROR: no partial form.");
        if (int rc = check_partial_u8(L, "PartialDepthwiseConv2D<quint8>", L->C, bias))
            return rc;
        if (items == 0)
            return SMALL_B200_OK;
        window_u8_kernel<OP, true><<<(unsigned)((items + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, filt, nullptr, out);
        if (int rc = launched(name))
            return rc;
        requant_in_place_kernel<<<1, 1024, 0, as_stream(stream)>>>(a.Ho * a.Wo, a, out);
        return launched("requant_in_place_kernel");
    }
    if (items == 0)
        return SMALL_B200_OK;
    if (OP == 0 && a.zero_filt == -128 && (a.zero_in == 0 || a.zero_in == -128) && a.Fh == 3 && a.Fw == 3 &&
        a.stride == 1 && a.C <= 2048 && a.Wo >= 3)
    {
        // 3x3 stride 1: row strips of 4, 5 or 6 outputs per thread, whichever tiles the width best
        const bool sgn = a.zero_in != 0;
        cudaStream_t st = as_stream(stream);
        int tw = 6, waste = 1 << 30;
        for (int t = 6; t >= 4; --t)
        {
            const int w_ = (a.Wo + t - 1) / t * t - a.Wo;
            if (w_ < waste) { waste = w_; tw = t; }
        }
        const int strips = (a.Wo + tw - 1) / tw;
        const long long threads = (long long)a.N * (a.C / CB) * a.Ho * strips * 2;
        const unsigned blocks = (unsigned)((threads + 255) / 256);
        const size_t smem = (size_t)(a.C / CB) * 48 * 4;
#define SB_DW_ROWS(S, T) dwconv3x3_u8_rows_kernel<S, T><<<blocks, 256, smem, st>>>(a, in, filt, bias, out, strips, L->pad_t, L->pad_l)
        if (tw == 6) { if (sgn) SB_DW_ROWS(true, 6); else SB_DW_ROWS(false, 6); }
        else if (tw == 5) { if (sgn) SB_DW_ROWS(true, 5); else SB_DW_ROWS(false, 5); }
        else { if (sgn) SB_DW_ROWS(true, 4); else SB_DW_ROWS(false, 4); }
#undef SB_DW_ROWS
        return launched("dwconv3x3_u8_rows_kernel");
    }
    if (OP == 0 && a.zero_filt == -128 && (a.zero_in == 0 || a.zero_in == -128) && a.Fh * a.Fw <= 64 && a.C <= 2048)
    {
        const int quads = (a.Fh * a.Fw + 3) / 4;
        const size_t smem = (size_t)(a.C / CB) * quads * CB * 4 + (size_t)quads * 4 * sizeof(short2);
        const unsigned blocks = (unsigned)((items + 255) / 256);
        const bool sgn = a.zero_in != 0;
        cudaStream_t st = as_stream(stream);
        if (quads == 3) // 3x3
            sgn ? dwconv_u8_dp4a_kernel<true, 3><<<blocks, 256, smem, st>>>(a, in, filt, bias, out)
                : dwconv_u8_dp4a_kernel<false, 3><<<blocks, 256, smem, st>>>(a, in, filt, bias, out);
        else if (quads == 1)
            sgn ? dwconv_u8_dp4a_kernel<true, 1><<<blocks, 256, smem, st>>>(a, in, filt, bias, out)
                : dwconv_u8_dp4a_kernel<false, 1><<<blocks, 256, smem, st>>>(a, in, filt, bias, out);
        else
            sgn ? dwconv_u8_dp4a_kernel<true, 0><<<blocks, 256, smem, st>>>(a, in, filt, bias, out)
                : dwconv_u8_dp4a_kernel<false, 0><<<blocks, 256, smem, st>>>(a, in, filt, bias, out);
        return launched("dwconv_u8_dp4a_kernel");
    }
    if (OP == 2 && a.Fh == a.H && a.Fw == a.W && !L->pad_t && !L->pad_b && !L->pad_l && !L->pad_r)
    {
        const long long warps = (long long)a.N * (a.C / CB);
        global_avgpool_u8_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, out);
        return launched("global_avgpool_u8_kernel");
    }
    window_u8_kernel<OP><<<(unsigned)((items + 255) / 256), 256, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched(name);
}
} // namespace

namespace sb
{
// Defined in conv_u8_tc.cu: the tensor-core path for shapes it supports.  Returns -1 when
// the shape is not covered, otherwise a SMALL_B200_* code.
int conv2d_u8_tensor_core(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                          const int32_t *bias, uint8_t *out, cudaStream_t st);
int conv2d_u8_one_channel_tc(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                             const int32_t *bias, uint8_t *out, cudaStream_t st);
// Defined in conv_u8_ring.cu: every other window / stride / channel count as an implicit GEMM on the
// tensor core, for the zero points it covers; -1 otherwise.
int conv2d_u8_ring(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt, const int32_t *bias,
                   uint8_t *out, cudaStream_t st);
}

namespace
{
// path: 0 = the faster kernel for the shape, 1 = CUDA cores only, 2 = tensor cores or an error
int conv2d_u8_dispatch(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt, const int32_t *bias,
                       uint8_t *out, void *stream, int path)
{
    const bool tensor_core = path != 1;
    if (int rc = check_window_layer(L, "Conv2D<quint8>", true, 2))
        return rc;
    if (int rc = check_quant(L, "Conv2D<quint8>"))
        return rc;
    if (L->accumulate)
    {
        if (int rc = check_partial_u8(L, "PartialConv2D<quint8>", L->K, bias))
            return rc;
        if (path == 2)
            return fail(SMALL_B200_INVALID_ARGUMENT, "PartialConv2D<quint8> ERROR: runs on the CUDA cores only.");
        QArgs a; fill(L, a, true);
        if (a.Ho <= 0 || a.Wo <= 0)
            return SMALL_B200_OK;
        dim3 grid((a.Ho * a.Wo + 127) / 128, 1, 1);
        conv2d_u8_direct_kernel<true><<<grid, 128, 0, as_stream(stream)>>>(a, in, filt, nullptr, out);
        if (int rc = launched("conv2d_u8_direct_kernel"))
            return rc;
        requant_in_place_kernel<<<1, 1024, 0, as_stream(stream)>>>(a.Ho * a.Wo, a, out);
        return launched("requant_in_place_kernel");
    }
    const int tc = tensor_core ? conv2d_u8_tensor_core(L, in, filt, bias, out, as_stream(stream)) : -1;
    if (tc >= 0)
        return tc;
    QArgs a; fill(L, a, true);
    if (a.N == 0 || a.Ho == 0 || a.Wo == 0)
        return SMALL_B200_OK;
    if (tensor_core)
    {
        const int tc1 = conv2d_u8_one_channel_tc(L, in, filt, bias, out, as_stream(stream));
        if (tc1 >= 0)
            return tc1;
    }
    // A reduction of one 32-byte step (a 1x1 layer on 16 channels, a 3x3 first layer on 3) is a streaming
    // layer with nothing for the tensor core to do: measured on MobileNet-v1 0.25 uint8 at batch 2048, the
    // implicit GEMM takes 0.43 ms for the 3x3x3 first layer and 0.188 ms for 16 -> 16 channels (the direct
    // kernel 0.35 and 0.185), and wins from 16 -> 32 channels on (0.052 against 0.097 ms).  Those layers
    // run the one-step dp4a kernel when the zero points let the operands enter shifted.
    const long long red = (long long)L->C * L->Fh * L->Fw;
    const bool ring_first = red > 32 || (L->C >= CB && L->K >= 32);
    if (path != 2 && !(tensor_core && ring_first) && red <= 32 && (L->C < CB || (L->Fh == 1 && L->Fw == 1)) &&
        a.zero_filt == -128 && (a.zero_in == 0 || a.zero_in == -128) && a.K <= 1024 &&
        reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0)
    {
        const int words = (int)((red + 3) / 4);
        const size_t smem = (size_t)(a.K / CB) * words * CB * sizeof(unsigned);
        const long long total = (long long)a.N * a.Ho * a.Wo;
        long long nb = (total + 255) / 256;
        if (nb > (long long)num_sms() * 16)
            nb = (long long)num_sms() * 16;
        const unsigned blocks = (unsigned)nb;
        const bool sgn = a.zero_in != 0, first = L->C < CB;
        cudaStream_t st = as_stream(stream);
        if (first && a.C == 3 && a.Fh == 3 && a.Fw == 3)
            sgn ? conv2d_u8_onestep_kernel<true, true, true><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out)
                : conv2d_u8_onestep_kernel<false, true, true><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out);
        else if (first)
            sgn ? conv2d_u8_onestep_kernel<true, true><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out)
                : conv2d_u8_onestep_kernel<false, true><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out);
        else
            sgn ? conv2d_u8_onestep_kernel<true, false><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out)
                : conv2d_u8_onestep_kernel<false, false><<<blocks, 256, smem, st>>>(a, words, in, filt, bias, out);
        return launched("conv2d_u8_onestep_kernel");
    }
    if (path == 2 || (tensor_core && ring_first))
    {
        const int tc2 = conv2d_u8_ring(L, in, filt, bias, out, as_stream(stream));
        if (tc2 >= 0)
            return tc2;
    }
    if (path == 2)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2D<quint8> ERROR: layer not covered by the tensor-core kernels.");
    if (a.C == 1 && a.zero_filt == -128 && (a.zero_in == 0 || a.zero_in == -128))
    {
        // one-channel image: rows of the window are words of the (zero-padded) image
        const int quads = (a.Fw + 3) / 4;
        const int pitch = ((a.W + L->pad_l + L->pad_r + 4 * quads + 8) + 3) & ~3; // room for the unaligned read
        const int prow = a.H + L->pad_t + L->pad_b + 1;
        const size_t smem = (size_t)(a.K / CB) * a.Fh * quads * CB * 4 + (size_t)C1_IMGS * prow * pitch;
        if (smem <= 160 * 1024)
        {
            static PerDeviceOnce configured;
            int dev;
            if (configured.needed(&dev))
            {
                SB_CUDA(cudaFuncSetAttribute(conv2d_u8_c1_dp4a_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
                SB_CUDA(cudaFuncSetAttribute(conv2d_u8_c1_dp4a_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
                configured.mark(dev);
            }
            const unsigned blocks = (unsigned)((a.N + C1_IMGS - 1) / C1_IMGS);
            if (a.zero_in == 0)
                conv2d_u8_c1_dp4a_kernel<false><<<blocks, 256, smem, as_stream(stream)>>>(a, in, filt, bias, out, pitch, prow);
            else
                conv2d_u8_c1_dp4a_kernel<true><<<blocks, 256, smem, as_stream(stream)>>>(a, in, filt, bias, out, pitch, prow);
            return launched("conv2d_u8_c1_dp4a_kernel");
        }
    }
    dim3 grid((a.Ho * a.Wo + 127) / 128, a.K / CB, a.N);
    conv2d_u8_direct_kernel<false><<<grid, 128, 0, as_stream(stream)>>>(a, in, filt, bias, out);
    return launched("conv2d_u8_direct_kernel");
}
} // namespace

extern "C"
{
int small_b200_conv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                         const int32_t *bias, uint8_t *out, void *stream)
{
    return conv2d_u8_dispatch(L, in, filt, bias, out, stream, 0);
}

int small_b200_conv2d_u8_cuda_cores(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                                    const int32_t *bias, uint8_t *out, void *stream)
{
    return conv2d_u8_dispatch(L, in, filt, bias, out, stream, 1);
}

int small_b200_conv2d_u8_tensor_core(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                                     const int32_t *bias, uint8_t *out, void *stream)
{
    return conv2d_u8_dispatch(L, in, filt, bias, out, stream, 2);
}

int small_b200_dwconv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                           const int32_t *bias, uint8_t *out, void *stream)
{
    return launch_window<0>(L, "DepthwiseConv2D<quint8>", 2, in, filt, bias, out, stream);
}

int small_b200_maxpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    return launch_window<1>(L, "MaxPool2D<quint8>", 2, in, nullptr, nullptr, out, stream);
}

int small_b200_avgpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    return launch_window<2>(L, "AveragePool2D<quint8>", 3, in, nullptr, nullptr, out, stream);
}

int small_b200_relu_u8(int64_t n, const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream)
{
    if (n < 0 || n % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "ReLUActivation<quint8> ERROR: in_channels unsupported.");
    if (int rc = check_quant(L, "ReLUActivation<quint8>"))
        return rc;
    if (n == 0)
        return SMALL_B200_OK;
    QArgs a{};
    a.zero_in = L->zero_in; a.lshift = L->lshift; a.rshift = L->rshift; a.mult = L->multiplier;
    a.k_zero = L->k_zero;
    const long long n16 = n / 16;
    long long blocks = (n16 + 255) / 256;
    const long long cap = (long long)num_sms() * 16;
    if (blocks > cap)
        blocks = cap;
    relu_u8_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(n16, a, in, out);
    return launched("relu_u8");
}
} // extern "C"
