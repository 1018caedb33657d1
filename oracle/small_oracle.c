/*
 * small_oracle.c -- CPU restatement of SMaLL's layer semantics (TEST INFRASTRUCTURE,
 * see small_oracle.h).  Compile with -ffp-contract=off so that a*b+c is a separate
 * multiply and add, as in the reference's REF build (CMakeLists.txt:57-58,104-108: no
 * -mfma on the REF platform).
 *
 * The reference expresses every layer as one loop nest
 * (include/small/abstract_layer.hpp:1368-1823) with separate edge kernels for output
 * pixels whose window touches padding.  The restatement below computes each output
 * element directly; what it keeps from the loop nest is
 *   - the order in which terms are added: input-channel block, kernel row, kernel
 *     column, channel inside the block (abstract_layer.hpp:1630, :542-563);
 *   - padded taps are skipped, never multiplied by zero (compute_with_padding,
 *     abstract_layer.hpp:205-239);
 *   - a pixel is a "border" pixel when its window leaves the image; border pixels of
 *     a max pool start from 0, interior ones from their first tap
 *     (abstract_layer.hpp:515-523, :333, :720, :887).
 */
#include "small_oracle.h"

#include <math.h>
#include <stddef.h>
#include <stdlib.h>

int32_t so_out_dim(int32_t in, int32_t pad_front, int32_t pad_back, int32_t f, int32_t stride)
{
    /* include/small/utils.hpp:159-165 on the padded extent (abstract_layer.hpp:1449-1452) */
    int32_t o = (in + pad_front + pad_back - f) / stride + 1;
    return o > 0 ? o : 0;
}

void so_calc_padding(int32_t in, int32_t f, int32_t stride, int32_t *front, int32_t *back)
{
    /* include/small/utils.hpp:43-64 */
    int32_t p;
    if (in % stride == 0)
        p = (f > stride) ? f - stride : 0;
    else
        p = (f > (in % stride)) ? f - (in % stride) : 0;
    *front = p / 2;
    *back  = p - *front;
}

/* First-layer exception: buffers.hpp:52-57, interface_abstract.hpp:106-214. */
static int32_t eff_cib(int32_t C, int32_t cib)
{
    return (C < cib && (C == 1 || C == 2 || C == 3)) ? C : cib;
}

static inline size_t act_idx(int32_t H, int32_t W, int32_t cb, int32_t c, int32_t h, int32_t w)
{
    /* buffers.hpp:115-119 */
    return (size_t)(c / cb) * H * W * cb + (size_t)h * W * cb + (size_t)w * cb + (c % cb);
}

static inline float apply_act(float v, int act, float slope)
{
    if (act == 1)
        return v > 0.f ? v : 0.f; /* FLOAT_MAX_TILE_C against a zeroed tile */
    if (act == 2)
        return v > 0.f ? v : v * slope; /* FLOAT_COND_SCALE_TILE_C, intrinsics_float.h:423-439 */
    return v;
}

/* ---------------------------------------------------------------- float conv */
/* Every output element is an independent sum, so the outputs of one channel block (cob
 * accumulators side by side, which the compiler may keep in vector registers) and the rows of
 * the image (OpenMP) are computed in parallel; the order of additions INSIDE each sum is the
 * sequential one of the loop nest, so the result does not depend on the thread count. */
#define SO_MAX_COB 64
void so_conv2d_f32(const so_shape *s, const float *in, const float *filt,
                   const float *bias, int act, float slope, int accumulate, float *out)
{
    const int32_t cib = eff_cib(s->C, s->cib), cob = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    const int32_t ncb = s->C / cib;
    const int32_t kbs = (s->K + cob - 1) / cob;
    if (cob > SO_MAX_COB)
        return;
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t kb = 0; kb < kbs; ++kb)
        for (int32_t oh = 0; oh < Ho; ++oh)
        {
            const int32_t kv = (s->K - kb * cob) < cob ? (s->K - kb * cob) : cob;
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                float acc[SO_MAX_COB];
                float *o = out + act_idx(Ho, Wo, cob, kb * cob, oh, ow);
                for (int32_t j = 0; j < kv; ++j)
                {
                    acc[j] = accumulate ? o[j] : 0.f;
                    if (bias)
                        acc[j] = acc[j] + bias[kb * cob + j];
                }
                for (int32_t b = 0; b < ncb; ++b)
                    for (int32_t kh = 0; kh < s->Fh; ++kh)
                    {
                        const int32_t ih = oh * s->stride - s->pad_t + kh;
                        if (ih < 0 || ih >= s->H)
                            continue;
                        for (int32_t kw = 0; kw < s->Fw; ++kw)
                        {
                            const int32_t iw = ow * s->stride - s->pad_l + kw;
                            if (iw < 0 || iw >= s->W)
                                continue;
                            const float *a = in + ((size_t)b * s->H * s->W + (size_t)ih * s->W + iw) * cib;
                            /* packed_weight_index, buffers.hpp:69-78 */
                            const float *f = filt + ((((size_t)kb * ncb + b) * s->Fh + kh) * s->Fw + kw) * cib * cob;
                            for (int32_t c = 0; c < cib; ++c)
                            {
                                const float av = a[c];
                                const float *fc = f + (size_t)c * cob;
                                for (int32_t j = 0; j < kv; ++j)
                                    acc[j] = acc[j] + av * fc[j];
                            }
                        }
                    }
                for (int32_t j = 0; j < kv; ++j)
                    o[j] = apply_act(acc[j], act, slope);
            }
        }
}

void so_dwconv2d_f32(const so_shape *s, const float *in, const float *filt,
                     const float *bias, int act, float slope, int accumulate, float *out)
{
    /* interface_abstract.hpp:994-1057: G_b = C_ob, K_b = F_cb = 1, op_class 1 */
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                const size_t oi = act_idx(Ho, Wo, cb, c, oh, ow);
                float acc = accumulate ? out[oi] : 0.f;
                if (bias)
                    acc = acc + bias[c];
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                {
                    const int32_t ih = oh * s->stride - s->pad_t + kh;
                    if (ih < 0 || ih >= s->H)
                        continue;
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t iw = ow * s->stride - s->pad_l + kw;
                        if (iw < 0 || iw >= s->W)
                            continue;
                        const float a = in[act_idx(s->H, s->W, cb, c, ih, iw)];
                        const float f = filt[(((size_t)(c / cb) * s->Fh + kh) * s->Fw + kw) * cb + (c % cb)];
                        acc = acc + a * f;
                    }
                }
                out[oi] = apply_act(acc, act, slope);
            }
}

/* Grouped convolution (interface_abstract.hpp:1265-1330 float, :1332-1400 quint8): the loop
 * nest with G_b = gb, K_b = F_cb = 1, whose layouts (abstract_layer.hpp:1419-1432) are
 *   I [G/gb][C][H][W][gb]   F [G/gb][K][C][Fh][Fw][gb]   O [G/gb][K][Ho][Wo][gb]
 * s->C / s->K are the channels of ONE group, s->cob is gb.  Reduction order of the nest:
 * input channel, kernel row, kernel column; padded taps skipped.  With gb = 1 the float
 * result is bit-identical to the reference's REF platform (tests/test_oracle_reference.py);
 * for larger blocks the reference's float instantiation is not a grouped convolution (it
 * uses the dense microkernel, op_class 2), so there the layout above is the definition. */
static inline size_t grp_idx(int32_t planes, int32_t H, int32_t W, int32_t gb, int32_t g, int32_t p,
                             int32_t h, int32_t w)
{
    return ((((size_t)(g / gb) * planes + p) * H + h) * W + w) * gb + (g % gb);
}

void so_groupconv2d_f32(const so_shape *s, int32_t groups, const float *in, const float *filt,
                        const float *bias, int act, float slope, int accumulate, float *out)
{
    const int32_t gb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t g = 0; g < groups; ++g)
        for (int32_t k = 0; k < s->K; ++k)
            for (int32_t oh = 0; oh < Ho; ++oh)
                for (int32_t ow = 0; ow < Wo; ++ow)
                {
                    const size_t oi = grp_idx(s->K, Ho, Wo, gb, g, k, oh, ow);
                    float acc = accumulate ? out[oi] : 0.f;
                    if (bias)
                        acc = acc + bias[((size_t)(g / gb) * s->K + k) * gb + (g % gb)];
                    for (int32_t c = 0; c < s->C; ++c)
                        for (int32_t kh = 0; kh < s->Fh; ++kh)
                        {
                            const int32_t ih = oh * s->stride - s->pad_t + kh;
                            if (ih < 0 || ih >= s->H)
                                continue;
                            for (int32_t kw = 0; kw < s->Fw; ++kw)
                            {
                                const int32_t iw = ow * s->stride - s->pad_l + kw;
                                if (iw < 0 || iw >= s->W)
                                    continue;
                                const float a = in[grp_idx(s->C, s->H, s->W, gb, g, c, ih, iw)];
                                const float f = filt[grp_idx(s->K * s->C, s->Fh, s->Fw, gb, g,
                                                             k * s->C + c, kh, kw)];
                                acc = acc + a * f;
                            }
                        }
                    out[oi] = apply_act(acc, act, slope);
                }
}

/* ---------------------------------------------------------------- float pools */
static int window_is_interior(const so_shape *s, int32_t oh, int32_t ow)
{
    const int32_t h0 = oh * s->stride - s->pad_t, w0 = ow * s->stride - s->pad_l;
    return h0 >= 0 && w0 >= 0 && h0 + s->Fh <= s->H && w0 + s->Fw <= s->W;
}

void so_maxpool2d_f32(const so_shape *s, const float *in, float *out)
{
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                const int32_t h0 = oh * s->stride - s->pad_t, w0 = ow * s->stride - s->pad_l;
                float m = 0.f; /* border pixels: the tile is zeroed first */
                if (window_is_interior(s, oh, ow))
                    m = in[act_idx(s->H, s->W, cb, c, h0, w0)]; /* FLOAT_LOAD_TILE_C_strided */
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t ih = h0 + kh, iw = w0 + kw;
                        if (ih < 0 || ih >= s->H || iw < 0 || iw >= s->W)
                            continue;
                        const float a = in[act_idx(s->H, s->W, cb, c, ih, iw)];
                        m = (a > m) ? a : m; /* FLOAT_MAX_TILE_C, intrinsics_float.h:306-321 */
                    }
                out[act_idx(Ho, Wo, cb, c, oh, ow)] = m;
            }
}

void so_avgpool2d_f32(const so_shape *s, const float *in, float *out)
{
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    /* abstract_layer.hpp:565-569: always 1/(Fh*Fw), padded taps included in the count */
    const float norm = (float)(1.0 / (1.0 * s->Fh * s->Fw));
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                const int32_t h0 = oh * s->stride - s->pad_t, w0 = ow * s->stride - s->pad_l;
                float acc = 0.f;
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t ih = h0 + kh, iw = w0 + kw;
                        if (ih < 0 || ih >= s->H || iw < 0 || iw >= s->W)
                            continue;
                        acc = acc + in[act_idx(s->H, s->W, cb, c, ih, iw)];
                    }
                out[act_idx(Ho, Wo, cb, c, oh, ow)] = acc * norm;
            }
}

/* ---------------------------------------------------------------- float elementwise */
void so_relu_f32(int64_t n, const float *in, float *out)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = in[i] > 0.f ? in[i] : 0.f;
}

void so_leaky_relu_f32(int64_t n, const float *in, float slope, float *out)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = in[i] > 0.f ? in[i] : in[i] * slope;
}

void so_accum_f32(int64_t n, const float *in, float *out)
{
    /* interface_abstract.hpp:1950-1980: OP_ADD with rewrite_output = 0 */
    for (int64_t i = 0; i < n; ++i)
        out[i] = out[i] + in[i];
}

void so_bias_f32(int32_t C, int32_t H, int32_t W, int32_t cb, const float *bias,
                 int accumulate, float *out)
{
    /* interface_abstract.hpp:1992-2060: OP_UPSAMPLE with an "infinite" stride, i.e. the
     * per-channel value is broadcast to every pixel. */
    for (int32_t c = 0; c < C; ++c)
        for (int32_t h = 0; h < H; ++h)
            for (int32_t w = 0; w < W; ++w)
            {
                const size_t i = act_idx(H, W, cb, c, h, w);
                out[i] = accumulate ? out[i] + bias[c] : bias[c];
            }
}

void so_upsample2d_f32(int32_t C, int32_t H, int32_t W, int32_t cb, int32_t scale,
                       const float *in, float *out)
{
    /* interface_abstract.hpp:1845-1888; out[h][w] = in[h/scale][w/scale] */
    const int32_t Ho = H * scale, Wo = W * scale;
    for (int32_t c = 0; c < C; ++c)
        for (int32_t h = 0; h < Ho; ++h)
            for (int32_t w = 0; w < Wo; ++w)
                out[act_idx(Ho, Wo, cb, c, h, w)] = in[act_idx(H, W, cb, c, h / scale, w / scale)];
}

void so_softmax_f32(int32_t C, int32_t H, int32_t W, int32_t cb, const float *in, float *out)
{
    /* interface_abstract.hpp:1778-1833: exp pass, one global sum over C*H*W, scale pass.
     * No max subtraction.  The sum runs in buffer order. */
    const int64_t n = (int64_t)C * H * W;
    (void)cb;
    for (int64_t i = 0; i < n; ++i)
        out[i] = expf(in[i]);
    float sum = 0.f;
    for (int64_t i = 0; i < n; ++i)
        sum = sum + out[i];
    const float inv = (float)(1.0 / sum);
    for (int64_t i = 0; i < n; ++i)
        out[i] = out[i] * inv;
}

/* ---------------------------------------------------------------- uint8 */
int32_t so_requant(int32_t acc, int32_t lshift, int32_t rshift, int32_t multiplier)
{
    /* QUINT8_QUANTIZE_TILE_C + VQRDMULH + RNDRSHIFT,
     * include/small/platforms/reference/intrinsics_quint8.h:481-531.
     * The clamp to [0,255] uses the template defaults, not the buffer's fields
     * (q_abstract_layer.hpp:160-161). */
    const int64_t a = (int64_t)(int32_t)((uint32_t)acc * (uint32_t)(1u << lshift));
    const int64_t b = (int64_t)multiplier;
    const int overflow = (a == b) && (a == -2147483648LL);
    const int64_t prod = a * b;
    const int32_t nudge = prod >= 0 ? (1 << 30) : (1 - (1 << 30));
    const int32_t hi = (int32_t)((prod + nudge) / (1LL << 31)); /* truncating division */
    int32_t v = overflow ? 2147483647 : hi;
    const int32_t mask = (int32_t)((1LL << rshift) - 1);
    const int32_t mod = v & mask;
    const int32_t threshold = (mask >> 1) + ((v < 0) ? -1 : 0);
    v = (v >> rshift) + ((mod > threshold) ? -1 : 0); /* "one" is ~0 in the reference */
    return v > 0 ? (v < 255 ? v : 255) : 0;
}

static void conv2d_u8_impl(const so_shape *s, const so_quant *q, const uint8_t *in,
                           const uint8_t *filt, const int32_t *bias, const int32_t *partial, uint8_t *out)
{
    const int32_t cib = eff_cib(s->C, s->cib), cob = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    const int32_t ncb = s->C / cib;
    for (int32_t k = 0; k < s->K; ++k)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                /* Partial form: the tile is loaded from the int32 values kept in the output buffer
                 * instead of being set to k_zero (q_abstract_layer.hpp:1151, first = false) */
                int32_t acc = partial ? partial[act_idx(Ho, Wo, cob, k, oh, ow)] : q->k_zero + (bias ? bias[k] : 0);
                for (int32_t b = 0; b < ncb; ++b)
                    for (int32_t kh = 0; kh < s->Fh; ++kh)
                    {
                        const int32_t ih = oh * s->stride - s->pad_t + kh;
                        if (ih < 0 || ih >= s->H)
                            continue;
                        for (int32_t kw = 0; kw < s->Fw; ++kw)
                        {
                            const int32_t iw = ow * s->stride - s->pad_l + kw;
                            if (iw < 0 || iw >= s->W)
                                continue;
                            const uint8_t *a = in + ((size_t)b * s->H * s->W + (size_t)ih * s->W + iw) * cib;
                            const uint8_t *f = filt + ((((size_t)(k / cob) * ncb + b) * s->Fh + kh) * s->Fw + kw) * cib * cob + (k % cob);
                            for (int32_t c = 0; c < cib; ++c) /* QUINT8_CONV_TILE_C :191-206 */
                                acc += ((int32_t)a[c] + q->zero_in) * ((int32_t)f[(size_t)c * cob] + q->zero_filt);
                        }
                    }
                out[act_idx(Ho, Wo, cob, k, oh, ow)] =
                    (uint8_t)so_requant(acc, q->lshift, q->rshift, q->multiplier);
            }
}

void so_conv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                  const uint8_t *filt, const int32_t *bias, uint8_t *out)
{
    conv2d_u8_impl(s, q, in, filt, bias, NULL, out);
}

void so_partial_conv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                          const uint8_t *filt, const int32_t *partial, uint8_t *out)
{
    conv2d_u8_impl(s, q, in, filt, NULL, partial, out);
}

static void dwconv2d_u8_impl(const so_shape *s, const so_quant *q, const uint8_t *in,
                             const uint8_t *filt, const int32_t *bias, const int32_t *partial, uint8_t *out)
{
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                int32_t acc = partial ? partial[act_idx(Ho, Wo, cb, c, oh, ow)] : q->k_zero + (bias ? bias[c] : 0);
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                {
                    const int32_t ih = oh * s->stride - s->pad_t + kh;
                    if (ih < 0 || ih >= s->H)
                        continue;
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t iw = ow * s->stride - s->pad_l + kw;
                        if (iw < 0 || iw >= s->W)
                            continue;
                        const int32_t a = in[act_idx(s->H, s->W, cb, c, ih, iw)];
                        const int32_t f = filt[(((size_t)(c / cb) * s->Fh + kh) * s->Fw + kw) * cb + (c % cb)];
                        acc += (a + q->zero_in) * (f + q->zero_filt); /* QUINT8_DW_TILE_C :270-289 */
                    }
                }
                out[act_idx(Ho, Wo, cb, c, oh, ow)] =
                    (uint8_t)so_requant(acc, q->lshift, q->rshift, q->multiplier);
            }
}

void so_dwconv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                    const uint8_t *filt, const int32_t *bias, uint8_t *out)
{
    dwconv2d_u8_impl(s, q, in, filt, bias, NULL, out);
}

void so_partial_dwconv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                            const uint8_t *filt, const int32_t *partial, uint8_t *out)
{
    dwconv2d_u8_impl(s, q, in, filt, NULL, partial, out);
}

void so_groupconv2d_u8(const so_shape *s, const so_quant *q, int32_t groups, const uint8_t *in,
                       const uint8_t *filt, const int32_t *bias, uint8_t *out)
{
    /* q_abstract_layer.hpp:894 with op_class 1 (interface_abstract.hpp:1358): lane-wise
     * QUINT8_DW_TILE_C per input channel of the group */
    const int32_t gb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t g = 0; g < groups; ++g)
        for (int32_t k = 0; k < s->K; ++k)
            for (int32_t oh = 0; oh < Ho; ++oh)
                for (int32_t ow = 0; ow < Wo; ++ow)
                {
                    int32_t acc = q->k_zero +
                                  (bias ? bias[((size_t)(g / gb) * s->K + k) * gb + (g % gb)] : 0);
                    for (int32_t c = 0; c < s->C; ++c)
                        for (int32_t kh = 0; kh < s->Fh; ++kh)
                        {
                            const int32_t ih = oh * s->stride - s->pad_t + kh;
                            if (ih < 0 || ih >= s->H)
                                continue;
                            for (int32_t kw = 0; kw < s->Fw; ++kw)
                            {
                                const int32_t iw = ow * s->stride - s->pad_l + kw;
                                if (iw < 0 || iw >= s->W)
                                    continue;
                                const int32_t a = in[grp_idx(s->C, s->H, s->W, gb, g, c, ih, iw)];
                                const int32_t f = filt[grp_idx(s->K * s->C, s->Fh, s->Fw, gb, g,
                                                               k * s->C + c, kh, kw)];
                                acc += (a + q->zero_in) * (f + q->zero_filt);
                            }
                        }
                    out[grp_idx(s->K, Ho, Wo, gb, g, k, oh, ow)] =
                        (uint8_t)so_requant(acc, q->lshift, q->rshift, q->multiplier);
                }
}

void so_maxpool2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in, uint8_t *out)
{
    /* q_abstract_layer.hpp:277-288: interior tiles start from the RAW first tap (no zero
     * point), border tiles from k_zero; every tap then enters as a + zero_in
     * (QUINT8_MAX_TILE_C, intrinsics_quint8.h:231-246); the maximum is requantised. */
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                const int32_t h0 = oh * s->stride - s->pad_t, w0 = ow * s->stride - s->pad_l;
                int32_t m = q->k_zero;
                if (window_is_interior(s, oh, ow))
                    m = in[act_idx(s->H, s->W, cb, c, h0, w0)];
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t ih = h0 + kh, iw = w0 + kw;
                        if (ih < 0 || ih >= s->H || iw < 0 || iw >= s->W)
                            continue;
                        const int32_t a = (int32_t)in[act_idx(s->H, s->W, cb, c, ih, iw)] + q->zero_in;
                        m = a > m ? a : m;
                    }
                out[act_idx(Ho, Wo, cb, c, oh, ow)] =
                    (uint8_t)so_requant(m, q->lshift, q->rshift, q->multiplier);
            }
}

void so_relu_u8(int64_t n, const so_quant *q, const uint8_t *in, uint8_t *out)
{
    /* interface_abstract.hpp:1577-1607: OP_RELU, tile seeded with k_zero = 0 */
    for (int64_t i = 0; i < n; ++i)
    {
        int32_t m = q->k_zero;
        const int32_t a = (int32_t)in[i] + q->zero_in;
        m = a > m ? a : m;
        out[i] = (uint8_t)so_requant(m, q->lshift, q->rshift, q->multiplier);
    }
}

void so_avgpool2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in, uint8_t *out)
{
    const int32_t cb = s->cob;
    const int32_t Ho = so_out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride);
    const int32_t Wo = so_out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    for (int32_t c = 0; c < s->C; ++c)
        for (int32_t oh = 0; oh < Ho; ++oh)
            for (int32_t ow = 0; ow < Wo; ++ow)
            {
                const int32_t h0 = oh * s->stride - s->pad_t, w0 = ow * s->stride - s->pad_l;
                int32_t acc = q->k_zero;
                for (int32_t kh = 0; kh < s->Fh; ++kh)
                    for (int32_t kw = 0; kw < s->Fw; ++kw)
                    {
                        const int32_t ih = h0 + kh, iw = w0 + kw;
                        if (ih < 0 || ih >= s->H || iw < 0 || iw >= s->W)
                            continue;
                        acc += (int32_t)in[act_idx(s->H, s->W, cb, c, ih, iw)] + q->zero_in;
                    }
                out[act_idx(Ho, Wo, cb, c, oh, ow)] =
                    (uint8_t)so_requant(acc, q->lshift, q->rshift, q->multiplier);
            }
}

/* ---------------------------------------------------------------- detection head */
static float so_sigmoid(float v)
{
    /* include/small/YOLOLayer.hpp:22-24: 1.0 / (1.0 + std::exp(-v)) in double, result back to float */
    return (float)(1.0 / (1.0 + (double)expf(-v)));
}

void so_yolo_decode_f32(int32_t Cp, int32_t H, int32_t W, int32_t cb, int32_t num_anchors, int32_t num_classes,
                        float stride, const float *anchor_wh, const float *in, float *out)
{
    /* include/small/YOLOLayer.hpp:168-222 on the packed input (the reference unpacks first) */
    const int32_t rec = num_classes + 5;
    size_t pred = 0;
    for (int32_t a = 0; a < num_anchors; ++a)
        for (int32_t h = 0; h < H; ++h)
            for (int32_t w = 0; w < W; ++w, ++pred)
                for (int32_t j = 0; j < rec; ++j)
                {
                    const float v = in[act_idx(H, W, cb, a * rec + j, h, w)];
                    float r;
                    if (j == 0)
                        r = stride * (so_sigmoid(v) + (float)w);
                    else if (j == 1)
                        r = stride * (so_sigmoid(v) + (float)h);
                    else if (j == 2)
                        r = expf(v) * anchor_wh[2 * a];
                    else if (j == 3)
                        r = expf(v) * anchor_wh[2 * a + 1];
                    else
                        r = so_sigmoid(v);
                    out[pred * rec + j] = r;
                }
    (void)Cp;
}

typedef struct
{
    float x, y, w, h, obj, score;
    int32_t cls;
} so_det;

static float so_overlap(float x1, float w1, float x2, float w2)
{
    /* include/small/non_max_suppression.hpp:33-42 */
    const float l1 = x1 - w1 / 2, l2 = x2 - w2 / 2;
    const float left = l1 > l2 ? l1 : l2;
    const float r1 = x1 + w1 / 2, r2 = x2 + w2 / 2;
    const float right = r1 < r2 ? r1 : r2;
    return right - left;
}

static float so_iou(const so_det *a, const so_det *b)
{
    /* include/small/non_max_suppression.hpp:45-59 */
    const float area_a = a->w * a->h, area_b = b->w * b->h;
    const float wo = so_overlap(a->x, a->w, b->x, b->w), ho = so_overlap(a->y, a->h, b->y, b->h);
    const float inter = (wo < 0.f || ho < 0.f) ? 0.f : wo * ho;
    const float uni = area_a + area_b - inter;
    return inter / uni;
}

int32_t so_nms_f32(const float *pred, int32_t num_pred, int32_t num_classes, float conf_thr, float iou_thr,
                   int32_t max_det, float *out, int32_t *candidates)
{
    /* Darknet.hpp:85-122 (collection, in prediction-then-class order) and non_max_suppression.hpp:98-155.
     * std::sort leaves the order of equal objectness values open; here ties keep the collection order
     * (an insertion sort is stable). */
    const int32_t rec = num_classes + 5;
    int32_t n = 0, cap = 1024;
    so_det *d = (so_det *)malloc((size_t)cap * sizeof(so_det));
    for (int32_t p = 0; p < num_pred; ++p)
    {
        const float *r = pred + (size_t)p * rec;
        if (!(r[4] > conf_thr))
            continue;
        for (int32_t c = 0; c < num_classes; ++c)
            if (r[5 + c] > conf_thr)
            {
                if (n == cap)
                    d = (so_det *)realloc(d, (size_t)(cap *= 2) * sizeof(so_det));
                const so_det v = {r[0], r[1], r[2], r[3], r[4], r[5 + c], c};
                d[n++] = v;
            }
    }
    *candidates = n;
    for (int32_t i = 1; i < n; ++i)
    {
        const so_det v = d[i];
        int32_t j = i - 1;
        while (j >= 0 && d[j].obj < v.obj)
        {
            d[j + 1] = d[j];
            --j;
        }
        d[j + 1] = v;
    }
    char *alive = (char *)malloc((size_t)(n > 0 ? n : 1));
    for (int32_t i = 0; i < n; ++i)
        alive[i] = 1;
    int32_t kept = 0;
    for (int32_t i = 0; i < n; ++i)
    {
        if (!alive[i])
            continue;
        if (kept < max_det)
        {
            float *o = out + (size_t)kept * 7;
            o[0] = d[i].x; o[1] = d[i].y; o[2] = d[i].w; o[3] = d[i].h; o[4] = d[i].obj; o[5] = d[i].score;
            o[6] = (float)d[i].cls;
        }
        ++kept;
        for (int32_t j = i + 1; j < n; ++j)
            if (alive[j] && d[j].cls == d[i].cls && !(so_iou(&d[i], &d[j]) < iou_thr))
                alive[j] = 0;
    }
    free(alive);
    free(d);
    return kept;
}

/* ---------------------------------------------------------------- weight preparation */
void so_conv_weights_prepare_f32(int32_t K, int32_t Keff, int32_t C, int32_t Fh, int32_t Fw, int32_t cb,
                                 const float *filt, const float *bias, const float *gamma, const float *beta,
                                 const float *mean, const float *var, float eps, float *packed, float *packed_bias)
{
    /* detail::initialize_conv2d_buffers, include/small/Conv2DLayer.hpp:135-341: zero-padded packing
     * (:179-209, packed_weight_index buffers.hpp:33-79), padded bias (:225-240), BN folding (:284-331) */
    const int32_t cib = eff_cib(C, cb);
    const size_t total = (size_t)K * C * Fh * Fw;
    for (size_t i = 0; i < total; ++i)
        packed[i] = 0.f;
    for (int32_t k = 0; k < Keff; ++k)
        for (int32_t c = 0; c < C; ++c)
            for (int32_t h = 0; h < Fh; ++h)
                for (int32_t w = 0; w < Fw; ++w)
                    packed[((((size_t)(k / cb) * (C / cib) + c / cib) * Fh + h) * Fw + w) * cib * cb +
                           (size_t)(c % cib) * cb + (k % cb)] = filt[(((size_t)k * C + c) * Fh + h) * Fw + w];
    if (packed_bias)
        for (int32_t k = 0; k < K; ++k)
            packed_bias[k] = (bias && k < Keff) ? bias[k] : 0.f;
    if (!gamma)
        return;
    for (int32_t k = 0; k < Keff; ++k)
    {
        const float rsq = 1.0f / sqrtf(var[k] + eps);
        const float scale = gamma[k] * rsq;
        if (!bias)
            packed_bias[k] = beta[k] - mean[k] * scale;
        else
            packed_bias[k] = beta[k] + scale * (packed_bias[k] - mean[k]);
        for (int32_t c = 0; c < C; ++c)
            for (int32_t h = 0; h < Fh; ++h)
                for (int32_t w = 0; w < Fw; ++w)
                    packed[((((size_t)(k / cb) * (C / cib) + c / cib) * Fh + h) * Fw + w) * cib * cb +
                           (size_t)(c % cib) * cb + (k % cb)] *= scale;
    }
}
