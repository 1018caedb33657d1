// model_graph.cpp -- the reference's Model classes on the B200 platform, eager and as one CUDA graph.
//
// Builds small::TinyYoloV2<FloatBuffer> (include/small/models/TinyYoloV2.hpp of the reference, used
// unchanged) with seeded random filters, runs inference() the way the reference's drivers do
// (every layer call is a kernel launch from the host), then records the same inference() with
// small::b200::InferenceGraph and replays it.  Checks:
//   - the replayed graph leaves bit-identical results to the eager run, on repeated replays too;
//   - with small::b200::BatchScope(B) and an input shape whose batch entry is B, every image of
//     the batch equals the single-image result of that image (bit for bit where both launches split
//     the reductions alike, within fp32 rounding otherwise);
//   - host access to a buffer inside a capture is refused with an exception, and the graph object
//     can be used again afterwards.
// Prints the time per inference of both forms.  Exit code 0 = all checks passed.
//
// With a fourth argument (a directory) the filters, the single input image and the model's output
// for it are written there as raw float32 files (f0.bin .. f8.bin, image.bin, out.bin), so that a
// second party -- the test-suite's CPU restatement of the reference -- can recompute the output.
//
//   model_graph [image size = 416] [batch = 4] [timed runs = 20] [dump directory]
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include <small.h>
#include <small/models/TinyYoloV2.hpp>

using BufferT = small::FloatBuffer;

static double now_ms()
{
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

static void dump(const std::string &dir, const std::string &name, const float *p, size_t n)
{
    if (dir.empty())
        return;
    FILE *f = std::fopen((dir + "/" + name).c_str(), "wb");
    if (!f || std::fwrite(p, sizeof(float), n, f) != n)
    {
        std::printf("FAIL: cannot write %s/%s\n", dir.c_str(), name.c_str());
        std::exit(2);
    }
    std::fclose(f);
}

static void fill(BufferT &b, std::mt19937 &rng, float lo, float hi)
{
    std::uniform_real_distribution<float> d(lo, hi);
    float *p = b.data();
    for (size_t i = 0; i < b.size(); ++i)
        p[i] = d(rng);
}

int main(int argc, char **argv)
{
    const uint32_t size = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 416;
    const uint32_t batch = argc > 2 ? (uint32_t)std::atoi(argv[2]) : 4;
    const int runs = argc > 3 ? std::atoi(argv[3]) : 20;
    const std::string dump_dir = argc > 4 ? argv[4] : "";
    int failures = 0;
    std::mt19937 rng(4);

    // filters of the nine convolutions, already in the packed layout (random numbers have no order)
    const uint32_t chans[10] = {3, 16, 32, 64, 128, 256, 512, 1024, 1024, 16};
    std::vector<BufferT *> filters;
    for (int l = 0; l < 9; ++l)
    {
        const uint32_t k = (l == 8) ? 1 : 3;
        BufferT *f = new BufferT((size_t)chans[l + 1] * chans[l] * k * k);
        const float bound = std::sqrt(6.0f / (float)(chans[l] * k * k)); // He-uniform keeps activations O(1)
        fill(*f, rng, -bound, bound);
        filters.push_back(f);
        dump(dump_dir, "f" + std::to_string(l) + ".bin", f->data(), f->size());
    }

    // ---- one image: eager, then recorded and replayed
    std::vector<float> single;
    {
        small::shape_type shape({1UL, 3UL, size, size});
        BufferT image((size_t)3 * size * size);
        fill(image, rng, 0.f, 1.f);
        small::TinyYoloV2<BufferT> model(shape, filters, true);
        small::Tensor<BufferT> input(shape, image);

        auto out = model.inference(&input);
        const size_t n = out[0]->size();
        single.assign(out[0]->buffer().data(), out[0]->buffer().data() + n);
        dump(dump_dir, "image.bin", image.data(), image.size());
        dump(dump_dir, "out.bin", single.data(), n);

        double t0 = now_ms();
        for (int r = 0; r < runs; ++r)
            out = model.inference(&input);
        (void)out[0]->buffer().data(); // waits for the device
        const double eager_ms = (now_ms() - t0) / runs;

        small::b200::InferenceGraph graph;
        std::vector<small::Tensor<BufferT> *> gout;
        graph.capture([&] { gout = model.inference(&input); });
        for (int rep = 0; rep < 2; ++rep)
        {
            graph.launch();
            const float *g = gout[0]->buffer().data();
            if (gout[0]->size() != n || std::memcmp(g, single.data(), n * sizeof(float)) != 0)
            {
                std::printf("FAIL: replay %d differs from the eager run\n", rep);
                ++failures;
            }
        }
        t0 = now_ms();
        for (int r = 0; r < runs; ++r)
            graph.launch();
        graph.sync();
        const double graph_ms = (now_ms() - t0) / runs;
        std::printf("TinyYoloV2 %ux%u, 1 image: eager %.3f ms, graph %.3f ms per inference\n", size, size,
                    eager_ms, graph_ms);

        // host access inside a capture is an error, and the object survives it
        bool threw = false;
        try
        {
            graph.capture([&] {
                gout = model.inference(&input);
                (void)gout[0]->buffer().data();
            });
        }
        catch (std::runtime_error const &)
        {
            threw = true;
        }
        if (!threw)
        {
            std::printf("FAIL: host access inside a capture was not refused\n");
            ++failures;
        }
        graph.capture([&] { gout = model.inference(&input); });
        graph.launch();
        if (std::memcmp(gout[0]->buffer().data(), single.data(), n * sizeof(float)) != 0)
        {
            std::printf("FAIL: replay after a refused capture differs\n");
            ++failures;
        }
    }

    // ---- a batch: image-major [B][C/16][H][W][16]; every image must equal its single-image result
    {
        small::shape_type shape({(size_t)batch, 3UL, size, size});
        const size_t per_image = (size_t)3 * size * size;
        BufferT images(per_image * batch);
        fill(images, rng, 0.f, 1.f);
        small::b200::BatchScope scope((int)batch);
        small::TinyYoloV2<BufferT> model(shape, filters, true);
        small::Tensor<BufferT> input(shape, images);
        small::b200::InferenceGraph graph;
        std::vector<small::Tensor<BufferT> *> gout;
        graph.capture([&] { gout = model.inference(&input); });
        graph.launch();
        const size_t n = gout[0]->size() / batch;
        std::vector<float> batched(gout[0]->buffer().data(), gout[0]->buffer().data() + n * batch);
        double t0 = now_ms();
        for (int r = 0; r < runs; ++r)
            graph.launch();
        graph.sync();
        std::printf("TinyYoloV2 %ux%u, %u images: graph %.4f ms per image\n", size, size, batch,
                    (now_ms() - t0) / runs / batch);

        small::b200::BatchScope one(1);
        small::shape_type shape1({1UL, 3UL, size, size});
        small::TinyYoloV2<BufferT> model1(shape1, filters, true);
        uint32_t inexact = 0;
        for (uint32_t b = 0; b < batch; ++b)
        {
            BufferT image(per_image);
            std::memcpy(image.data(), images.data() + b * per_image, per_image * sizeof(float));
            small::Tensor<BufferT> input1(shape1, image);
            auto out = model1.inference(&input1);
            // Bit-identical wherever the library splits the reductions of an image's tiles the same way
            // in both launches.  It decides per launch, from the number of tiles, whether the two CTAs of
            // a cluster share a tile's reduction (the last, partial wave of a large batch does), so the
            // sums of some images may be associated differently than in their single-image run: a
            // difference of fp32 rounding, held here to 2e-6 of the output range.
            bool same = out[0]->size() == n;
            double worst = 0, top = 0;
            if (same)
            {
                const float *s1 = out[0]->buffer().data(), *sb = batched.data() + b * n;
                if (std::memcmp(s1, sb, n * sizeof(float)) != 0)
                {
                    ++inexact;
                    for (size_t i = 0; i < n; ++i)
                    {
                        worst = std::fmax(worst, std::fabs((double)s1[i] - sb[i]));
                        top = std::fmax(top, std::fabs((double)s1[i]));
                    }
                    same = worst <= 2e-6 * (top > 0 ? top : 1);
                }
            }
            if (!same)
            {
                std::printf("FAIL: image %u of the batch differs from its single-image result (%.3g of %.3g)\n", b,
                            worst, top);
                ++failures;
            }
        }
        std::printf("batch: %u of %u images bit-identical to their single-image result, the others within 2e-6\n",
                    batch - inexact, batch);
    }

    for (auto f : filters)
        delete f;
    std::printf(failures ? "FAILED (%d)\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
