// ref_shim.cpp -- C-ABI wrapper around the UNMODIFIED reference (TEST INFRASTRUCTURE).
//
// Compiled by oracle/Makefile against the reference's own headers, once per CPU
// platform of the reference:
//   REF   (include/small/platforms/reference: scalar C, float + quint8)  -> _ref/libsmall_ref.so
//   ZEN2  (include/small/platforms/zen2: AVX2+FMA, float only)           -> _ref/libsmall_zen2.so
// Nothing of the reference is copied: this file only calls the public small::
// functions (include/small/interface.hpp:49-497) on the reference's Buffer classes.
// It serves as the second opinion for oracle/small_oracle.c and as the timed CPU
// baseline.  The shipped CUDA library never loads it.
#include <small.h>
#include <small/Conv2DLayer.hpp>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <string>
#include <vector>

#include "small_oracle.h" // so_shape / so_quant PODs only

namespace
{
thread_local std::string g_err;

template <class B>
B make(const void *src, size_t n, size_t alloc = 0)
{
    B b(alloc > n ? alloc : n);
    if (src)
        std::memcpy(b.data(), src, n * sizeof(typename B::value_type));
    return b;
}

int out_dim(int in, int pf, int pb, int f, int s)
{
    int o = (in + pf + pb - f) / s + 1;
    return o > 0 ? o : 0;
}

#define GUARD(...)                       \
    try                                  \
    {                                    \
        __VA_ARGS__;                     \
        return 0;                        \
    }                                    \
    catch (std::invalid_argument & e)    \
    {                                    \
        g_err = e.what();                \
        return 1;                        \
    }                                    \
    catch (std::exception & e)           \
    {                                    \
        g_err = e.what();                \
        return 2;                        \
    }

double now_s()
{
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return t.tv_sec + 1e-9 * t.tv_nsec;
}
} // namespace

extern "C"
{
const char *ref_last_error() { return g_err.c_str(); }
int ref_float_cb() { return FLOAT_C_ob; }
int ref_has_quint8()
{
#if defined(SMALL_HAS_QUINT8_SUPPORT)
    return 1;
#else
    return 0;
#endif
}
#if defined(SMALL_HAS_QUINT8_SUPPORT)
int ref_quint8_cb() { return QUINT8_C_ob; }
#else
int ref_quint8_cb() { return 0; }
#endif

// The reference reads OMP_NUM_THREADS on every call (abstract_layer.hpp:1535-1556).
void ref_set_threads(int n)
{
    setenv("OMP_NUM_THREADS", std::to_string(n).c_str(), 1);
}

// detail::initialize_conv2d_buffers (include/small/Conv2DLayer.hpp:135): what a Conv2DLayer does to its
// weights when it is built.  n_bias / n_bn = 0 mean "no bias" / "no batch normalisation".
int ref_init_conv2d_buffers(int K, int Keff, int C, int Fh, int Fw, const float *filt, const float *bias, int n_bias,
                            const float *gamma, const float *beta, const float *mean, const float *var, int n_bn,
                            float eps, float *packed, float *packed_bias)
{
    GUARD({
        auto F = make<small::FloatBuffer>(filt, (size_t)Keff * C * Fh * Fw);
        auto B = make<small::FloatBuffer>(bias, (size_t)n_bias);
        auto G = make<small::FloatBuffer>(gamma, (size_t)n_bn);
        auto Be = make<small::FloatBuffer>(beta, (size_t)n_bn);
        auto M = make<small::FloatBuffer>(mean, (size_t)n_bn);
        auto V = make<small::FloatBuffer>(var, (size_t)n_bn);
        small::FloatBuffer PF, PB;
        small::detail::initialize_conv2d_buffers(K, Keff, C, Fh, Fw, F, B, G, Be, M, V, eps, false, PF, PB);
        std::memcpy(packed, PF.data(), PF.size() * sizeof(float));
        if (PB.size())
            std::memcpy(packed_bias, PB.data(), PB.size() * sizeof(float));
    })
}

// ------------------------------------------------------------------ float ops
int ref_conv2d_f32(const so_shape *s, const float *in, const float *filt, int partial, float *out)
{
    const size_t ni = (size_t)s->C * s->H * s->W, nf = (size_t)s->K * s->C * s->Fh * s->Fw;
    const size_t no = (size_t)s->K * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        auto I = make<small::FloatBuffer>(in, ni);
        auto F = make<small::FloatBuffer>(filt, nf);
        auto O = make<small::FloatBuffer>(out, no);
        if (partial)
            small::PartialConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                                 s->K, s->C, s->H, s->W, I, F, O);
        else
            small::Conv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                          s->K, s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no * sizeof(float));
    })
}

int ref_dwconv2d_f32(const so_shape *s, const float *in, const float *filt, int partial, float *out)
{
    const size_t ni = (size_t)s->C * s->H * s->W, nf = (size_t)s->C * s->Fh * s->Fw;
    const size_t no = (size_t)s->C * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        auto I = make<small::FloatBuffer>(in, ni);
        auto F = make<small::FloatBuffer>(filt, nf);
        auto O = make<small::FloatBuffer>(out, no);
        if (partial)
            small::PartialDepthwiseConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l,
                                          s->pad_r, s->C, s->H, s->W, I, F, O);
        else
            small::DepthwiseConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                                   s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no * sizeof(float));
    })
}

// small::GroupConv2D / PartialGroupConv2D<FloatBuffer> (interface_abstract.hpp:1265, :1402):
// `groups` groups of s->C channels each (the interface has one argument for the input and the
// output channels of a group).
int ref_groupconv2d_f32(const so_shape *s, int groups, const float *in, const float *filt, int partial,
                        float *out)
{
    const size_t ni = (size_t)groups * s->C * s->H * s->W;
    const size_t nf = (size_t)groups * s->C * s->C * s->Fh * s->Fw;
    const size_t no = (size_t)groups * s->C * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        auto I = make<small::FloatBuffer>(in, ni);
        auto F = make<small::FloatBuffer>(filt, nf);
        auto O = make<small::FloatBuffer>(out, no);
        if (partial)
            small::PartialGroupConv2D(s->Fh, s->Fw, s->stride, groups, s->pad_t, s->pad_b, s->pad_l,
                                      s->pad_r, s->C, s->H, s->W, I, F, O);
        else
            small::GroupConv2D(s->Fh, s->Fw, s->stride, groups, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                               s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no * sizeof(float));
    })
}

int ref_pool2d_f32(const so_shape *s, int average, const float *in, float *out)
{
    const size_t ni = (size_t)s->C * s->H * s->W;
    const size_t no = (size_t)s->C * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        auto I = make<small::FloatBuffer>(in, ni);
        auto O = make<small::FloatBuffer>(nullptr, no);
        if (average)
            small::AveragePool2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                                 s->C, s->H, s->W, I, O);
        else
            small::MaxPool2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                             s->C, s->H, s->W, I, O);
        std::memcpy(out, O.data(), no * sizeof(float));
    })
}

// op: 0 ReLU, 1 LeakyReLU(slope), 2 Accum (out += in), 3 SoftMax, 4 UpSample2D x2
int ref_eltwise_f32(int op, int C, int H, int W, float slope, const float *in, float *out)
{
    const size_t n = (size_t)C * H * W;
    GUARD({
        auto I = make<small::FloatBuffer>(in, n);
        auto O = make<small::FloatBuffer>(op == 2 ? out : nullptr, op == 4 ? 4 * n : n);
        if (op == 0)
            small::ReLUActivation(C, H, W, I, O);
        else if (op == 1)
        {
            small::FloatBuffer S(1);
            S.data()[0] = slope;
            small::LeakyReLUActivation(C, H, W, I, S, O);
        }
        else if (op == 2)
            small::Accum(C, H, W, I, O);
        else if (op == 3)
            small::SoftMax(C, H, W, I, O);
        else if (op == 4)
            small::UpSample2D(2, C, H, W, I, O);
        else
            throw std::invalid_argument("ref_eltwise_f32: bad op");
        std::memcpy(out, O.data(), O.size() * sizeof(float));
    })
}

int ref_bias_f32(int C, int H, int W, const float *bias, int partial, float *out)
{
    const size_t n = (size_t)C * H * W;
    GUARD({
        auto B = make<small::FloatBuffer>(bias, C);
        auto O = make<small::FloatBuffer>(out, n);
        if (partial)
            small::PartialBias(C, H, W, B, O);
        else
            small::Bias(C, H, W, B, O);
        std::memcpy(out, O.data(), n * sizeof(float));
    })
}

// ------------------------------------------------------------------ quint8 ops
#if defined(SMALL_HAS_QUINT8_SUPPORT)
namespace
{
void set_q(small::QUInt8Buffer &I, small::QUInt8Buffer *F, small::QUInt8Buffer &O, const so_quant *q)
{
    I.m_zero = q->zero_in;
    if (F)
        F->m_zero = q->zero_filt;
    O.lshift = q->lshift;
    O.rshift = q->rshift;
    O.multiplier = q->multiplier;
}
} // namespace

// The quint8 loop nest keeps int32 partial sums inside the uint8 output buffer
// (q_abstract_layer.hpp:1144), so callers allocate it four times too large
// (test/test_conv2d.cpp:302); different output-channel blocks alias there, hence one
// thread only.
int ref_conv2d_u8(const so_shape *s, const so_quant *q, int depthwise, const uint8_t *in,
                  const uint8_t *filt, uint8_t *out)
{
    const int K = depthwise ? s->C : s->K;
    const size_t ni = (size_t)s->C * s->H * s->W;
    const size_t nf = depthwise ? (size_t)s->C * s->Fh * s->Fw : (size_t)s->K * s->C * s->Fh * s->Fw;
    const size_t no = (size_t)K * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        ref_set_threads(1);
        auto I = make<small::QUInt8Buffer>(in, ni);
        auto F = make<small::QUInt8Buffer>(filt, nf);
        auto O = make<small::QUInt8Buffer>(nullptr, no, 4 * no + 64);
        set_q(I, &F, O, q);
        if (depthwise)
            small::DepthwiseConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                                   s->C, s->H, s->W, I, F, O);
        else
            small::Conv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r, s->K,
                          s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no);
    })
}

// small::PartialConv2D / PartialDepthwiseConv2D<QUInt8Buffer> (interface_abstract.hpp:595, :1194): the
// loop nest reads its starting accumulators as int32 from the output buffer (block k at BYTE offset
// k * Ho*Wo*block, q_abstract_layer.hpp:1135-1144) and leaves the bytes at the start.  Meaningful for
// one block of output channels; the caller passes such a shape.
int ref_partial_conv2d_u8(const so_shape *s, const so_quant *q, int depthwise, const uint8_t *in,
                          const uint8_t *filt, const int32_t *partial, uint8_t *out)
{
    const int K = depthwise ? s->C : s->K;
    const size_t ni = (size_t)s->C * s->H * s->W;
    const size_t nf = depthwise ? (size_t)s->C * s->Fh * s->Fw : (size_t)s->K * s->C * s->Fh * s->Fw;
    const size_t no = (size_t)K * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        ref_set_threads(1);
        auto I = make<small::QUInt8Buffer>(in, ni);
        auto F = make<small::QUInt8Buffer>(filt, nf);
        auto O = make<small::QUInt8Buffer>(nullptr, no, 4 * no + 64);
        set_q(I, &F, O, q);
        std::memcpy(O.data(), partial, no * sizeof(int32_t));
        if (depthwise)
            small::PartialDepthwiseConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                                          s->C, s->H, s->W, I, F, O);
        else
            small::PartialConv2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r, s->K,
                                 s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no);
    })
}

// small::GroupConv2D<QUInt8Buffer> (interface_abstract.hpp:1332)
int ref_groupconv2d_u8(const so_shape *s, const so_quant *q, int groups, const uint8_t *in,
                       const uint8_t *filt, uint8_t *out)
{
    const size_t ni = (size_t)groups * s->C * s->H * s->W;
    const size_t nf = (size_t)groups * s->C * s->C * s->Fh * s->Fw;
    const size_t no = (size_t)groups * s->C * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        ref_set_threads(1);
        auto I = make<small::QUInt8Buffer>(in, ni);
        auto F = make<small::QUInt8Buffer>(filt, nf);
        auto O = make<small::QUInt8Buffer>(nullptr, no, 4 * no + 64);
        set_q(I, &F, O, q);
        small::GroupConv2D(s->Fh, s->Fw, s->stride, groups, s->pad_t, s->pad_b, s->pad_l, s->pad_r,
                           s->C, s->H, s->W, I, F, O);
        std::memcpy(out, O.data(), no);
    })
}

int ref_maxpool2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in, uint8_t *out)
{
    const size_t ni = (size_t)s->C * s->H * s->W;
    const size_t no = (size_t)s->C * out_dim(s->H, s->pad_t, s->pad_b, s->Fh, s->stride) *
                      out_dim(s->W, s->pad_l, s->pad_r, s->Fw, s->stride);
    GUARD({
        ref_set_threads(1);
        auto I = make<small::QUInt8Buffer>(in, ni);
        auto O = make<small::QUInt8Buffer>(nullptr, no, 4 * no + 64);
        set_q(I, nullptr, O, q);
        small::MaxPool2D(s->Fh, s->Fw, s->stride, s->pad_t, s->pad_b, s->pad_l, s->pad_r, s->C,
                         s->H, s->W, I, O);
        std::memcpy(out, O.data(), no);
    })
}

int ref_relu_u8(int C, int H, int W, const so_quant *q, const uint8_t *in, uint8_t *out)
{
    const size_t n = (size_t)C * H * W;
    GUARD({
        ref_set_threads(1);
        auto I = make<small::QUInt8Buffer>(in, n);
        auto O = make<small::QUInt8Buffer>(nullptr, n, 4 * n + 64);
        set_q(I, nullptr, O, q);
        small::ReLUActivation(C, H, W, I, O);
        std::memcpy(out, O.data(), n);
    })
}
#endif // SMALL_HAS_QUINT8_SUPPORT

// ------------------------------------------------------------------ timed layer chains
// One image at a time through a chain of layers, the way the reference's layer
// classes drive the functional interface (Conv2DLayer.hpp:807-879: Bias ->
// PartialConv2D -> separate activation pass).  Weights arrive already packed for this
// platform's blocking.  Returns wall seconds for `images` images in *seconds and the
// last image's output in `out`.
struct ref_layer
{
    int32_t op; // 0 conv, 1 dwconv, 2 maxpool, 3 avgpool
    so_shape s;
    int32_t act; // 0 none, 1 ReLU, 2 LeakyReLU
    float slope;
    const void *filt;
    const void *bias;
    so_quant q;
};

int ref_run_chain_f32(const ref_layer *layers, int n_layers, const float *in, size_t in_elems,
                      int images, int threads, float *out, size_t out_elems, double *seconds)
{
    GUARD({
        ref_set_threads(threads);
        std::vector<small::FloatBuffer> filt, bias;
        size_t max_act = in_elems;
        for (int l = 0; l < n_layers; ++l)
        {
            const ref_layer &L = layers[l];
            const so_shape &s = L.s;
            const int K = (L.op == 0) ? s.K : s.C;
            size_t nf = (L.op == 0) ? (size_t)s.K * s.C * s.Fh * s.Fw
                                    : (L.op == 1 ? (size_t)s.C * s.Fh * s.Fw : 0);
            filt.push_back(make<small::FloatBuffer>(L.filt, nf ? nf : 1));
            bias.push_back(make<small::FloatBuffer>(L.bias, L.bias ? K : 1));
            size_t no = (size_t)K * out_dim(s.H, s.pad_t, s.pad_b, s.Fh, s.stride) *
                        out_dim(s.W, s.pad_l, s.pad_r, s.Fw, s.stride);
            if (no > max_act)
                max_act = no;
        }
        small::FloatBuffer a(max_act), b(max_act), slope(1), input(in_elems);
        std::memcpy(input.data(), in, in_elems * sizeof(float));
        small::FloatBuffer *cur = nullptr;
        const double t0 = now_s();
        for (int img = 0; img < images; ++img)
        {
            small::FloatBuffer const *src = &input;
            small::FloatBuffer *dst = &a;
            for (int l = 0; l < n_layers; ++l)
            {
                const ref_layer &L = layers[l];
                const so_shape &s = L.s;
                const int Ho = out_dim(s.H, s.pad_t, s.pad_b, s.Fh, s.stride);
                const int Wo = out_dim(s.W, s.pad_l, s.pad_r, s.Fw, s.stride);
                if (L.op == 0 || L.op == 1)
                {
                    const int K = (L.op == 0) ? s.K : s.C;
                    if (L.bias)
                        small::Bias(K, Ho, Wo, bias[l], *dst);
                    if (L.op == 0)
                    {
                        if (L.bias)
                            small::PartialConv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l,
                                                 s.pad_r, s.K, s.C, s.H, s.W, *src, filt[l], *dst);
                        else
                            small::Conv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l, s.pad_r,
                                          s.K, s.C, s.H, s.W, *src, filt[l], *dst);
                    }
                    else
                    {
                        if (L.bias)
                            small::PartialDepthwiseConv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b,
                                                          s.pad_l, s.pad_r, s.C, s.H, s.W, *src,
                                                          filt[l], *dst);
                        else
                            small::DepthwiseConv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l,
                                                   s.pad_r, s.C, s.H, s.W, *src, filt[l], *dst);
                    }
                    if (L.act == 1)
                        small::ReLUActivation(K, Ho, Wo, *dst, *dst);
                    else if (L.act == 2)
                    {
                        slope.data()[0] = L.slope;
                        small::LeakyReLUActivation(K, Ho, Wo, *dst, slope, *dst);
                    }
                }
                else if (L.op == 2)
                    small::MaxPool2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l, s.pad_r, s.C,
                                     s.H, s.W, *src, *dst);
                else if (L.op == 3)
                    small::AveragePool2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l, s.pad_r,
                                         s.C, s.H, s.W, *src, *dst);
                else
                    throw std::invalid_argument("ref_run_chain_f32: bad op");
                cur = dst;
                src = dst;
                dst = (dst == &a) ? &b : &a;
            }
        }
        *seconds = now_s() - t0;
        if (out && cur)
            std::memcpy(out, cur->data(), out_elems * sizeof(float));
    })
}

#if defined(SMALL_HAS_QUINT8_SUPPORT)
// uint8 chain: conv / dwconv / maxpool only (the reference has no quint8 average pool
// and no per-channel bias), one thread per image because of the aliasing noted above;
// `threads` images run side by side, each on private buffers.
static void chain_u8_impl(const ref_layer *layers, int n_layers, const uint8_t *in, size_t in_elems,
                          int images, int threads, uint8_t *out, size_t out_elems, double *seconds)
{
        ref_set_threads(1);
        size_t max_act = in_elems;
        for (int l = 0; l < n_layers; ++l)
        {
            const so_shape &s = layers[l].s;
            const int K = (layers[l].op == 0) ? s.K : s.C;
            size_t no = (size_t)K * out_dim(s.H, s.pad_t, s.pad_b, s.Fh, s.stride) *
                        out_dim(s.W, s.pad_l, s.pad_r, s.Fw, s.stride);
            if (no > max_act)
                max_act = no;
        }
        const double t0 = now_s();
        std::string err;
#pragma omp parallel for num_threads(threads) schedule(static)
        for (int img = 0; img < images; ++img)
        {
            try
            {
                small::QUInt8Buffer a(4 * max_act + 64), b(4 * max_act + 64), input(in_elems);
                std::memcpy(input.data(), in, in_elems);
                small::QUInt8Buffer const *src = &input;
                small::QUInt8Buffer *dst = &a;
                for (int l = 0; l < n_layers; ++l)
                {
                    const ref_layer &L = layers[l];
                    const so_shape &s = L.s;
                    const size_t nf = (L.op == 0) ? (size_t)s.K * s.C * s.Fh * s.Fw
                                                  : (size_t)s.C * s.Fh * s.Fw;
                    const_cast<small::QUInt8Buffer *>(src)->m_zero = L.q.zero_in;
                    dst->lshift = L.q.lshift;
                    dst->rshift = L.q.rshift;
                    dst->multiplier = L.q.multiplier;
                    if (L.op == 0 || L.op == 1)
                    {
                        auto F = make<small::QUInt8Buffer>(L.filt, nf);
                        F.m_zero = L.q.zero_filt;
                        if (L.op == 0)
                            small::Conv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l, s.pad_r,
                                          s.K, s.C, s.H, s.W, *src, F, *dst);
                        else
                            small::DepthwiseConv2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l,
                                                   s.pad_r, s.C, s.H, s.W, *src, F, *dst);
                    }
                    else if (L.op == 2)
                        small::MaxPool2D(s.Fh, s.Fw, s.stride, s.pad_t, s.pad_b, s.pad_l, s.pad_r,
                                         s.C, s.H, s.W, *src, *dst);
                    else
                        throw std::invalid_argument("ref_run_chain_u8: op has no quint8 reference");
                    src = dst;
                    dst = (dst == &a) ? &b : &a;
                }
                if (img == images - 1 && out)
                    std::memcpy(out, src->data(), out_elems);
            }
            catch (std::exception &e)
            {
#pragma omp critical
                err = e.what();
            }
        }
        *seconds = now_s() - t0;
        if (!err.empty())
            throw std::invalid_argument(err);
}

int ref_run_chain_u8(const ref_layer *layers, int n_layers, const uint8_t *in, size_t in_elems,
                     int images, int threads, uint8_t *out, size_t out_elems, double *seconds)
{
    GUARD(chain_u8_impl(layers, n_layers, in, in_elems, images, threads, out, out_elems, seconds))
}
#endif
} // extern "C"
