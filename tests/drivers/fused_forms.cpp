// fused_forms.cpp -- every function of the reference's fused interface (include/small/
// fused_interface_abstract.hpp:55-3667 and the 1-D file beside it) through the small:: boundary of
// the B200 platform, each against the composition of the unfused small:: functions that defines it
// (the way the reference's demo/fused_block_driver.cpp checks its two variants), plus the 1-D family
// with stride 2 against a direct loop, Dropout, and the quint8 Partial forms.  The unfused functions themselves are what the
// reference's own test drivers and the oracle tests pin.  Exit code 0 = all checks passed.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <stdexcept>
#include <vector>

#include <small.h>

using Buf = small::FloatBuffer;

static int failures = 0;
static std::mt19937 rng(11);

static void fill(Buf &b, float lo, float hi)
{
    std::uniform_real_distribution<float> d(lo, hi);
    float *p = b.data();
    for (size_t i = 0; i < b.size(); ++i)
        p[i] = d(rng);
}

static void expect_close(const char *what, Buf &got, Buf &want, size_t n)
{
    const float *g = got.data(), *w = want.data();
    double worst = 0, top = 0;
    for (size_t i = 0; i < n; ++i)
    {
        worst = std::fmax(worst, std::fabs((double)g[i] - w[i]));
        top = std::fmax(top, std::fabs((double)w[i]));
    }
    const bool ok = worst <= 1e-5 * (top > 0 ? top : 1);
    std::printf("%-46s max|diff| %.3g of %.3g  %s\n", what, worst, top, ok ? "ok" : "FAIL");
    failures += !ok;
}

int main()
{
    const int C = 32, K = 64, H = 12, W = 14;
    const uint8_t p = 1;
    const int Hc = H, Wc = W;                      // 3x3 'same'
    Buf in((size_t)C * H * W), f((size_t)K * C * 9), bias(K), mid((size_t)K * Hc * Wc), tile(16);
    fill(in, -1, 1); fill(f, -0.1f, 0.1f); fill(bias, -0.5f, 0.5f);

    // ---- one-op forms
    {
        Buf a((size_t)K * Hc * Wc), b((size_t)K * Hc * Wc);
        small::Conv2D_ReLU(3, 3, 1, p, p, p, p, K, C, H, W, in, f, a);
        small::Conv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("Conv2D_ReLU", a, b, a.size());
        small::Conv2D_Bias_ReLU(3, 3, 1, p, p, p, p, K, C, H, W, in, f, bias, a);
        small::Bias(K, Hc, Wc, bias, b);
        small::PartialConv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("Conv2D_Bias_ReLU", a, b, a.size());
    }
    Buf dwf((size_t)K * 9), dwb(K);
    fill(dwf, -0.3f, 0.3f); fill(dwb, -0.5f, 0.5f);
    {
        Buf x((size_t)K * Hc * Wc), a((size_t)K * Hc * Wc), b((size_t)K * Hc * Wc);
        fill(x, -1, 1);
        small::DepthwiseConv2D_ReLU(3, 3, 1, p, p, p, p, K, Hc, Wc, x, dwf, a);
        small::DepthwiseConv2D(3, 3, 1, p, p, p, p, K, Hc, Wc, x, dwf, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("DepthwiseConv2D_ReLU", a, b, a.size());
        small::DepthwiseConv2D_Bias_ReLU(3, 3, 1, p, p, p, p, K, Hc, Wc, x, dwf, dwb, a);
        small::Bias(K, Hc, Wc, dwb, b);
        small::PartialDepthwiseConv2D(3, 3, 1, p, p, p, p, K, Hc, Wc, x, dwf, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("DepthwiseConv2D_Bias_ReLU", a, b, a.size());
    }
    // ---- conv -> max pool (2x2/2: one kernel; 3x3/2: two kernels), with a small and a full-size
    //      inter_output_buf
    for (int pk = 2; pk <= 3; ++pk)
    {
        const int Hp = (Hc - pk) / 2 + 1, Wp = (Wc - pk) / 2 + 1;
        Buf a((size_t)K * Hp * Wp), b((size_t)K * Hp * Wp), c((size_t)K * Hc * Wc);
        auto unfused = [&](bool with_bias, bool relu) {
            if (with_bias)
            {
                small::Bias(K, Hc, Wc, bias, c);
                small::PartialConv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
            }
            else
                small::Conv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
            if (relu)
                small::ReLUActivation(K, Hc, Wc, c, c);
            small::MaxPool2D(pk, pk, 2, 0, 0, 0, 0, K, Hc, Wc, c, b);
        };
        small::Conv2D_Maxpool2D(3, 3, 1, p, p, p, p, pk, pk, 2, 0, 0, 0, 0, K, C, H, W, in, f, tile, a);
        unfused(false, false);
        expect_close(pk == 2 ? "Conv2D_Maxpool2D 2x2" : "Conv2D_Maxpool2D 3x3", a, b, a.size());
        small::Conv2D_ReLU_Maxpool2D(3, 3, 1, p, p, p, p, pk, pk, 2, 0, 0, 0, 0, K, C, H, W, in, f, mid, a);
        unfused(false, true);
        expect_close(pk == 2 ? "Conv2D_ReLU_Maxpool2D 2x2" : "Conv2D_ReLU_Maxpool2D 3x3", a, b, a.size());
        small::Conv2D_Bias_ReLU_Maxpool2D(3, 3, 1, p, p, p, p, pk, pk, 2, 0, 0, 0, 0, K, C, H, W, in, f, bias, tile, a);
        unfused(true, true);
        expect_close(pk == 2 ? "Conv2D_Bias_ReLU_Maxpool2D 2x2" : "Conv2D_Bias_ReLU_Maxpool2D 3x3", a, b, a.size());
    }
    // ---- conv -> max pool on an image wider than 64 pixels with 32 output channels: the tensor-core
    //      kernel takes the pool in its epilogue
    {
        const int C2 = 16, K2 = 32, H2 = 20, W2 = 100;
        Buf in2((size_t)C2 * H2 * W2), f2((size_t)K2 * C2 * 9), bias2(K2);
        Buf a((size_t)K2 * (H2 / 2) * (W2 / 2)), b((size_t)K2 * (H2 / 2) * (W2 / 2)), c((size_t)K2 * H2 * W2);
        fill(in2, -1, 1); fill(f2, -0.1f, 0.1f); fill(bias2, -0.5f, 0.5f);
        small::Conv2D_Bias_ReLU_Maxpool2D(3, 3, 1, p, p, p, p, 2, 2, 2, 0, 0, 0, 0, K2, C2, H2, W2, in2, f2, bias2, tile, a);
        small::Bias(K2, H2, W2, bias2, c);
        small::PartialConv2D(3, 3, 1, p, p, p, p, K2, C2, H2, W2, in2, f2, c);
        small::ReLUActivation(K2, H2, W2, c, c);
        small::MaxPool2D(2, 2, 2, 0, 0, 0, 0, K2, H2, W2, c, b);
        expect_close("Conv2D_Bias_ReLU_Maxpool2D wide image", a, b, a.size());
        small::Conv2D_Maxpool2D(3, 3, 1, p, p, p, p, 2, 2, 2, 0, 0, 0, 0, K2, C2, H2, W2, in2, f2, tile, a);
        small::Conv2D(3, 3, 1, p, p, p, p, K2, C2, H2, W2, in2, f2, c);
        small::MaxPool2D(2, 2, 2, 0, 0, 0, 0, K2, H2, W2, c, b);
        expect_close("Conv2D_Maxpool2D wide image", a, b, a.size());
    }
    // ---- conv -> depthwise conv
    {
        Buf a((size_t)K * Hc * Wc), b((size_t)K * Hc * Wc), c((size_t)K * Hc * Wc);
        small::Conv2D_DepthwiseConv2D(3, 3, 1, p, p, p, p, 3, 3, 1, p, p, p, p, K, C, H, W, in, f, tile, dwf, a);
        small::Conv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
        small::DepthwiseConv2D(3, 3, 1, p, p, p, p, K, Hc, Wc, c, dwf, b);
        expect_close("Conv2D_DepthwiseConv2D", a, b, a.size());
        small::Conv2D_ReLU_DepthwiseConv2D_ReLU(3, 3, 1, p, p, p, p, 3, 3, 1, p, p, p, p, K, C, H, W, in, f, mid, dwf, a);
        small::ReLUActivation(K, Hc, Wc, c, c);
        small::DepthwiseConv2D(3, 3, 1, p, p, p, p, K, Hc, Wc, c, dwf, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("Conv2D_ReLU_DepthwiseConv2D_ReLU", a, b, a.size());
        small::Conv2D_Bias_ReLU_DepthwiseConv2D_Bias_ReLU(3, 3, 1, p, p, p, p, 3, 3, 1, p, p, p, p, K, C, H, W, in, f,
                                                          bias, tile, dwf, dwb, a);
        small::Bias(K, Hc, Wc, bias, c);
        small::PartialConv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
        small::ReLUActivation(K, Hc, Wc, c, c);
        small::Bias(K, Hc, Wc, dwb, b);
        small::PartialDepthwiseConv2D(3, 3, 1, p, p, p, p, K, Hc, Wc, c, dwf, b);
        small::ReLUActivation(K, Hc, Wc, b, b);
        expect_close("Conv2D_Bias_ReLU_DepthwiseConv2D_Bias_ReLU", a, b, a.size());
    }
    // ---- grouped forms: group g = the dense 16 -> 16 convolution Conv2D computes on channel block g
    {
        const int G = K / 16;
        Buf gf((size_t)G * 9 * 256), gb(K), x((size_t)K * Hc * Wc), a((size_t)K * Hc * Wc), b((size_t)K * Hc * Wc);
        fill(gf, -0.2f, 0.2f); fill(gb, -0.5f, 0.5f); fill(x, -1, 1);
        auto blockwise = [&](Buf &src, Buf &dst, bool with_bias, bool relu) {
            for (int g = 0; g < G; ++g)
            {
                Buf xi((size_t)16 * Hc * Wc), fi(9 * 256), oi((size_t)16 * Hc * Wc), bi(16);
                std::copy(src.data() + (size_t)g * 16 * Hc * Wc, src.data() + (size_t)(g + 1) * 16 * Hc * Wc, xi.data());
                std::copy(gf.data() + (size_t)g * 9 * 256, gf.data() + (size_t)(g + 1) * 9 * 256, fi.data());
                std::copy(gb.data() + g * 16, gb.data() + (g + 1) * 16, bi.data());
                if (with_bias)
                {
                    small::Bias(16, Hc, Wc, bi, oi);
                    small::PartialConv2D(3, 3, 1, p, p, p, p, 16, 16, Hc, Wc, xi, fi, oi);
                }
                else
                    small::Conv2D(3, 3, 1, p, p, p, p, 16, 16, Hc, Wc, xi, fi, oi);
                if (relu)
                    small::ReLUActivation(16, Hc, Wc, oi, oi);
                std::copy(oi.data(), oi.data() + oi.size(), dst.data() + (size_t)g * 16 * Hc * Wc);
            }
        };
        small::GroupConv2D_ReLU(3, 3, 1, G, p, p, p, p, K, Hc, Wc, x, gf, a);
        blockwise(x, b, false, true);
        expect_close("GroupConv2D_ReLU", a, b, a.size());
        small::GroupConv2D_Bias_ReLU(3, 3, 1, G, p, p, p, p, K, Hc, Wc, x, gf, gb, a);
        blockwise(x, b, true, true);
        expect_close("GroupConv2D_Bias_ReLU", a, b, a.size());
        Buf c((size_t)K * Hc * Wc);
        small::Conv2D_GroupConv(3, 3, 1, p, p, p, p, 3, 3, 1, G, p, p, p, p, K, C, H, W, in, f, tile, gf, a);
        small::Conv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
        blockwise(c, b, false, false);
        expect_close("Conv2D_GroupConv", a, b, a.size());
        small::Conv2D_ReLU_GroupConv2D_ReLU(3, 3, 1, p, p, p, p, 3, 3, 1, G, p, p, p, p, K, C, H, W, in, f, mid, gf, a);
        small::ReLUActivation(K, Hc, Wc, c, c);
        blockwise(c, b, false, true);
        expect_close("Conv2D_ReLU_GroupConv2D_ReLU", a, b, a.size());
        small::Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU(3, 3, 1, p, p, p, p, 3, 3, 1, G, p, p, p, p, K, C, H, W, in, f, bias,
                                                      tile, gf, gb, a);
        small::Bias(K, Hc, Wc, bias, c);
        small::PartialConv2D(3, 3, 1, p, p, p, p, K, C, H, W, in, f, c);
        small::ReLUActivation(K, Hc, Wc, c, c);
        blockwise(c, b, true, true);
        expect_close("Conv2D_Bias_ReLU_GroupConv2D_Bias_ReLU", a, b, a.size());
    }
    // ---- 1-D family with stride 2 against a direct loop: layout [C/16][batch][W][16]
    {
        const int B = 5, Wi = 37, k = 5, s = 2, lp = 2, rp = 2, Wo = (Wi + lp + rp - k) / s + 1, K1 = 32, C1 = 16;
        Buf x((size_t)C1 * B * Wi), w((size_t)K1 * C1 * k), a((size_t)K1 * B * Wo), want((size_t)K1 * B * Wo);
        fill(x, -1, 1); fill(w, -0.2f, 0.2f);
        small::Conv1D(k, s, lp, rp, K1, C1, B, Wi, x, w, a);
        const float *xp = x.data(), *wp = w.data();
        float *o = want.data();
        for (int kk = 0; kk < K1; ++kk)
            for (int b = 0; b < B; ++b)
                for (int ow = 0; ow < Wo; ++ow)
                {
                    float acc = 0.f;
                    for (int t = 0; t < k; ++t)
                    {
                        const int iw = ow * s - lp + t;
                        if (iw < 0 || iw >= Wi)
                            continue;
                        for (int c = 0; c < C1; ++c) // filter [K/16][C/16][1][k][16 c][16 k]
                            acc += xp[((size_t)b * Wi + iw) * 16 + c] * wp[(((size_t)(kk / 16) * k + t) * 16 + c) * 16 + kk % 16];
                    }
                    o[(((size_t)(kk / 16) * B + b) * Wo + ow) * 16 + kk % 16] = acc;
                }
        expect_close("Conv1D stride 2", a, want, a.size());
        Buf r1((size_t)K1 * B * Wo);
        small::Conv1D_ReLU(k, s, lp, rp, K1, C1, B, Wi, x, w, r1);
        small::ReLUActivation1D(K1, B, Wo, want, want);
        expect_close("Conv1D_ReLU stride 2", r1, want, r1.size());
        // pool of that output, stride 2, and the fused pair
        const int Wp = (Wo - 2) / 2 + 1;
        Buf pa((size_t)K1 * B * Wp), pb((size_t)K1 * B * Wp), scratch(16);
        small::MaxPool1D(2, 2, 0, 0, K1, B, Wo, want, pb);
        small::Conv1D_ReLU_Maxpool1D(k, s, lp, rp, 2, 2, 0, 0, K1, C1, B, Wi, x, w, scratch, pa);
        expect_close("Conv1D_ReLU_Maxpool1D stride 2", pa, pb, pa.size());
        Buf up((size_t)K1 * B * Wo * 2);
        small::UpSample1D(2, K1, B, Wo, want, up);
        bool same = true;
        for (int cb = 0; cb < K1 / 16 && same; ++cb)
            for (int b = 0; b < B && same; ++b)
                for (int q = 0; q < 2 * Wo * 16; ++q)
                    same = same && up.data()[((size_t)(cb * B + b) * 2 * Wo) * 16 + q] ==
                                       want.data()[((size_t)(cb * B + b) * Wo + (q / 16) / 2) * 16 + q % 16];
        std::printf("%-46s %s\n", "UpSample1D", same ? "ok" : "FAIL");
        failures += !same;
    }
    // ---- Dropout: output = input * rate
    {
        Buf x((size_t)32 * 6 * 6), rate(1), o(x.size());
        fill(x, -1, 1);
        rate.data()[0] = 0.75f;
        small::Dropout(32, 6, 6, x, rate, o);
        bool same = true;
        for (size_t i = 0; i < x.size(); ++i)
            same = same && o.data()[i] == x.data()[i] * 0.75f;
        std::printf("%-46s %s\n", "Dropout", same ? "ok" : "FAIL");
        failures += !same;
    }
    // ---- quint8 Partial forms: with zero partial sums waiting in the output buffer they equal the plain
    // forms (one block of 16 output channels, where the reference's in-buffer int32 storage is defined);
    // more than one block is refused with std::invalid_argument
    {
        const int C1 = 32, H = 9, W = 7, K1 = 16;
        small::QUInt8Buffer x((size_t)C1 * H * W), w((size_t)K1 * C1 * 9), wd((size_t)K1 * 9);
        std::uniform_int_distribution<int> d(0, 255);
        for (size_t i = 0; i < x.size(); ++i) x.data()[i] = (uint8_t)d(rng);
        for (size_t i = 0; i < w.size(); ++i) w.data()[i] = (uint8_t)d(rng);
        for (size_t i = 0; i < wd.size(); ++i) wd.data()[i] = (uint8_t)d(rng);
        const size_t n = (size_t)K1 * H * W;
        small::QUInt8Buffer plain(n), part(4 * n), x16(n), dplain(n), dpart(4 * n);
        plain.multiplier = part.multiplier = 1 << 30; plain.rshift = part.rshift = 14; plain.lshift = part.lshift = 0;
        dplain.multiplier = dpart.multiplier = 1 << 30; dplain.rshift = dpart.rshift = 9; dplain.lshift = dpart.lshift = 0;
        small::Conv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, plain);
        for (size_t i = 0; i < 4 * n; ++i) part.data()[i] = 0;
        small::PartialConv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, part);
        bool same = true;
        for (size_t i = 0; i < n; ++i) same = same && plain.data()[i] == part.data()[i];
        std::printf("%-46s %s\n", "PartialConv2D<quint8> from zero partial sums", same ? "ok" : "FAIL");
        failures += !same;
        for (size_t i = 0; i < n; ++i) x16.data()[i] = x.data()[i];
        small::DepthwiseConv2D(3, 3, 1, 1, 1, 1, 1, K1, H, W, x16, wd, dplain);
        for (size_t i = 0; i < 4 * n; ++i) dpart.data()[i] = 0;
        small::PartialDepthwiseConv2D(3, 3, 1, 1, 1, 1, 1, K1, H, W, x16, wd, dpart);
        same = true;
        for (size_t i = 0; i < n; ++i) same = same && dplain.data()[i] == dpart.data()[i];
        std::printf("%-46s %s\n", "PartialDepthwiseConv2D<quint8>", same ? "ok" : "FAIL");
        failures += !same;
        bool refused = false;
        small::QUInt8Buffer w32((size_t)32 * C1 * 9), o32((size_t)4 * 32 * H * W);
        try { small::PartialConv2D(3, 3, 1, 1, 1, 1, 1, 32, C1, H, W, x, w32, o32); }
        catch (std::invalid_argument const &) { refused = true; }
        std::printf("%-46s %s\n", "PartialConv2D<quint8>, two blocks: refused", refused ? "ok" : "FAIL");
        failures += !refused;
    }
    // ---- a convolution call waits for the next call (an in-place activation joins it): what the buffers
    // hold must not depend on that
    {
        const int C1 = 32, K1 = 64, H = 13, W = 13;
        Buf x((size_t)C1 * H * W), w((size_t)K1 * C1 * 9), bias(K1), slope(1);
        fill(x, -1, 1); fill(w, -0.1f, 0.1f); fill(bias, -0.5f, 0.5f);
        slope.data()[0] = 0.1f;
        const size_t n = (size_t)K1 * H * W;
        Buf fused(n), a(n), b(n), c(n);
        small::Conv2D_ReLU(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, fused);
        small::Conv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, a);
        small::ReLUActivation(K1, H, W, a, a);                       // joins the convolution
        expect_close("Conv2D, then ReLU in place", a, fused, n);
        small::Conv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, b);
        bool neg = false;
        for (size_t i = 0; i < n; ++i) neg = neg || b.data()[i] < 0;  // host access launches it as it is
        small::ReLUActivation(K1, H, W, b, c);                        // not in place: a kernel of its own
        expect_close("Conv2D, host access, then ReLU out of place", c, fused, n);
        std::printf("%-46s %s\n", "  the plain result keeps its negative values", neg ? "ok" : "FAIL");
        failures += !neg;
        {
            Buf *tmp = new Buf(x.size());
            for (size_t i = 0; i < x.size(); ++i) tmp->data()[i] = x.data()[i];
            small::Conv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, *tmp, w, c);
            delete tmp;                                               // the input goes away before anything else is called
            small::ReLUActivation(K1, H, W, c, c);
            expect_close("Conv2D, input destroyed, then ReLU", c, fused, n);
        }
        Buf lf(n), lu(n);
        small::Bias(K1, H, W, bias, lu);
        small::PartialConv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, lu);
        small::LeakyReLUActivation(K1, H, W, lu, slope, lu);          // joins the partial convolution
        small::Bias(K1, H, W, bias, lf);
        small::PartialConv2D(3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, lf);
        (void)lf.data();                                              // launched without the activation
        small::LeakyReLUActivation(K1, H, W, lf, slope, lf);
        expect_close("Bias, PartialConv2D, LeakyReLU in place", lu, lf, n);
        {
            Buf wd((size_t)C1 * 9), xd((size_t)C1 * H * W), d1((size_t)C1 * H * W), d2((size_t)C1 * H * W);
            fill(wd, -0.3f, 0.3f); fill(xd, -1, 1);
            small::DepthwiseConv2D_ReLU(3, 3, 1, 1, 1, 1, 1, C1, H, W, xd, wd, d1);
            small::DepthwiseConv2D(3, 3, 1, 1, 1, 1, 1, C1, H, W, xd, wd, d2);
            small::ReLUActivation(C1, H, W, d2, d2);                  // joins the depthwise convolution
            expect_close("DepthwiseConv2D, then ReLU in place", d2, d1, d1.size());
        }
        bool thrown = false;
        try { small::Conv2D(3, 3, 3, 0, 0, 0, 0, K1, C1, H, W, x, w, a); }
        catch (std::invalid_argument const &) { thrown = true; }
        std::printf("%-46s %s\n", "Conv2D with stride 3 throws at the call", thrown ? "ok" : "FAIL");
        failures += !thrown;
    }
    // ---- quint8 Conv2D_ReLU_DepthwiseConv2D_ReLU: one kernel (1x1 64 -> 64 on a 25x5 image, depthwise 3x3)
    // against the two calls, bit for bit
    {
        const int C1 = 64, K1 = 64, H = 25, W = 5;
        small::QUInt8Buffer x((size_t)C1 * H * W), w((size_t)K1 * C1), wd((size_t)K1 * 9);
        std::uniform_int_distribution<int> d(0, 255);
        for (size_t i = 0; i < x.size(); ++i) x.data()[i] = (uint8_t)d(rng);
        for (size_t i = 0; i < w.size(); ++i) w.data()[i] = (uint8_t)d(rng);
        for (size_t i = 0; i < wd.size(); ++i) wd.data()[i] = (uint8_t)d(rng);
        x.m_zero = 0; w.m_zero = -128; wd.m_zero = -128;
        const size_t n = (size_t)K1 * H * W;
        small::QUInt8Buffer mid(n), fused(n), mid2(n), two(n);
        for (auto *b : {&mid, &mid2}) { b->m_zero = 0; b->multiplier = 1 << 30; b->rshift = 13; b->lshift = 0; }
        for (auto *b : {&fused, &two}) { b->multiplier = 1 << 30; b->rshift = 9; b->lshift = 0; }
        small::Conv2D_ReLU_DepthwiseConv2D_ReLU(1, 1, 1, 0, 0, 0, 0, 3, 3, 1, 1, 1, 1, 1, K1, C1, H, W, x, w, mid, wd, fused);
        small::Conv2D(1, 1, 1, 0, 0, 0, 0, K1, C1, H, W, x, w, mid2);
        small::DepthwiseConv2D(3, 3, 1, 1, 1, 1, 1, K1, H, W, mid2, wd, two);
        bool same = true;
        int lo = 255, hi = 0;
        for (size_t i = 0; i < n; ++i)
        {
            same = same && fused.data()[i] == two.data()[i];
            lo = std::min<int>(lo, two.data()[i]); hi = std::max<int>(hi, two.data()[i]);
        }
        same = same && lo < hi;
        std::printf("%-46s %s (values %d..%d)\n", "Conv2D_ReLU_DepthwiseConv2D_ReLU<quint8>", same ? "ok" : "FAIL", lo, hi);
        failures += !same;
    }
    std::printf(failures ? "FAILED (%d)\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
