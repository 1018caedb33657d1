// yolo.cu -- what follows the last convolution of a detection network, on the device:
//   * box decoding, small::YOLOLayer::compute_output (include/small/YOLOLayer.hpp:96-222): the packed
//     activation [C/16][H][W][16] seen as [anchor][5 + classes][H][W] becomes one record
//     [x, y, w, h, objectness, class scores...] per anchor and pixel;
//   * detection collection and non-maximum suppression, Darknet::process_outputs
//     (include/small/models/Darknet.hpp:78-122) + small::basic_nms
//     (include/small/non_max_suppression.hpp:98-155): every (prediction, class) pair above the
//     confidence threshold is a detection; detections are ordered by objectness, and a detection
//     suppresses the later ones of its class whose IoU with it is not below the threshold.
// The reference does both on the host, element by element; here decoding is one elementwise kernel
// that reads the activation in its packed order, and NMS is collect (atomic append) -> rank sort ->
// one CTA that walks the ranking.  Box arithmetic uses the reference's operations one by one with
// round-to-nearest intrinsics (no fused multiply-add), so that for the same records the same
// detections survive as on the host.
#include "common.cuh"

namespace
{
using namespace sb;

constexpr int MAX_ANCHORS = 16;
struct Anchors
{
    float w[MAX_ANCHORS], h[MAX_ANCHORS];
};

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

// thread = one element of the packed activation (coalesced reads); its record slot is computed
__global__ void __launch_bounds__(256)
yolo_decode_kernel(int N, int Cp, int H, int W, int A, int rec, float stride, const Anchors an,
                   const float *__restrict__ in, float *__restrict__ out)
{
    const long long total = (long long)N * Cp * H * W;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    const float v = in[i];
    const int c16 = (int)(i & 15); i >>= 4;
    const int w = (int)(i % W); i /= W;
    const int h = (int)(i % H); i /= H;
    const int cb = (int)(i % (Cp / CB));
    const int n = (int)(i / (Cp / CB));
    const int ch = cb * CB + c16;
    if (ch >= A * rec)
        return; // channels the layer before padded up to the block
    const int a = ch / rec, j = ch - a * rec;
    float r;
    if (j == 0)
        r = stride * (sigmoidf_(v) + (float)w);
    else if (j == 1)
        r = stride * (sigmoidf_(v) + (float)h);
    else if (j == 2)
        r = expf(v) * an.w[a];
    else if (j == 3)
        r = expf(v) * an.h[a];
    else
        r = sigmoidf_(v);
    out[(((size_t)n * A + a) * H * W + (size_t)h * W + w) * rec + j] = r;
}

// ---- detections
struct Det
{
    float x, y, w, h, obj, score;
    int cls;
    int src; // prediction * classes + class: the order the host loop would have met it in
};

__global__ void __launch_bounds__(256)
collect_kernel(int P, int classes, float thr, const float *__restrict__ pred, Det *cand, int cap, int *count)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P)
        return;
    const float *r = pred + (size_t)p * (classes + 5);
    if (!(r[4] > thr))
        return;
    for (int c = 0; c < classes; ++c)
        if (r[5 + c] > thr)
        {
            const int slot = atomicAdd(count, 1);
            if (slot < cap)
                cand[slot] = Det{r[0], r[1], r[2], r[3], r[4], r[5 + c], c, p * classes + c};
        }
}

// rank of every candidate in the order (objectness descending, source position ascending)
__global__ void __launch_bounds__(256)
rank_kernel(const Det *cand, const int *count, int cap, Det *sorted)
{
    const int n = *count < cap ? *count : cap;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const Det me = cand[i];
    int rank = 0;
    for (int j = 0; j < n; ++j)
    {
        const float o = cand[j].obj;
        const int s = cand[j].src;
        rank += (o > me.obj || (o == me.obj && s < me.src)) ? 1 : 0;
    }
    sorted[rank] = me;
}

__device__ __forceinline__ float overlap_(float x1, float w1, float x2, float w2)
{
    const float l1 = __fsub_rn(x1, __fdiv_rn(w1, 2.f)), l2 = __fsub_rn(x2, __fdiv_rn(w2, 2.f));
    const float left = l1 > l2 ? l1 : l2;
    const float r1 = __fadd_rn(x1, __fdiv_rn(w1, 2.f)), r2 = __fadd_rn(x2, __fdiv_rn(w2, 2.f));
    const float right = r1 < r2 ? r1 : r2;
    return __fsub_rn(right, left);
}
__device__ __forceinline__ float iou_(const Det &a, const Det &b)
{
    const float area_a = __fmul_rn(a.w, a.h), area_b = __fmul_rn(b.w, b.h);
    const float wo = overlap_(a.x, a.w, b.x, b.w), ho = overlap_(a.y, a.h, b.y, b.h);
    const float inter = (wo < 0.f || ho < 0.f) ? 0.f : __fmul_rn(wo, ho);
    const float uni = __fsub_rn(__fadd_rn(area_a, area_b), inter);
    return __fdiv_rn(inter, uni);
}

// One CTA walks the ranking: the first detection still alive is kept and removes the later ones of
// its class it overlaps too much; then the next one alive, and so on (basic_nms).
__global__ void __launch_bounds__(1024)
nms_kernel(const Det *sorted, const int *count, int cap, float iou_thr, unsigned char *alive, int max_det, float *out,
           int *out_count)
{
    const int n = *count < cap ? *count : cap;
    __shared__ Det cur;
    __shared__ int take;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
        alive[j] = 1;
    int kept = 0;
    __syncthreads();
    for (int i = 0; i < n; ++i)
    {
        if (threadIdx.x == 0)
        {
            take = alive[i];
            if (take)
                cur = sorted[i];
        }
        __syncthreads();
        if (take)
        {
            if (threadIdx.x == 0 && kept < max_det)
            {
                float *o = out + (size_t)kept * 7;
                o[0] = cur.x; o[1] = cur.y; o[2] = cur.w; o[3] = cur.h; o[4] = cur.obj; o[5] = cur.score;
                o[6] = (float)cur.cls;
            }
            ++kept;
            for (int j = i + 1 + threadIdx.x; j < n; j += blockDim.x)
                if (alive[j])
                {
                    const Det d = sorted[j];
                    if (d.cls == cur.cls && !(iou_(cur, d) < iou_thr))
                        alive[j] = 0;
                }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        out_count[0] = kept;          // detections that survive
        out_count[1] = *count;        // (prediction, class) pairs above the confidence threshold
    }
}
} // namespace

extern "C"
{
int small_b200_yolo_decode_f32(int32_t N, int32_t C_padded, int32_t H, int32_t W, int32_t num_anchors,
                               int32_t num_classes, float stride, const float *anchor_wh, const float *in, float *out,
                               void *stream)
{
    if (C_padded <= 0 || C_padded % CB != 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "YOLOLayer ERROR: in_channels unsupported.");
    if (num_anchors <= 0 || num_anchors > MAX_ANCHORS || num_classes < 0 || !anchor_wh ||
        (long long)num_anchors * (num_classes + 5) > C_padded)
        return fail(SMALL_B200_INVALID_ARGUMENT, "YOLOLayer ERROR: incorrect input buffer shape.");
    if (N <= 0 || H <= 0 || W <= 0)
        return SMALL_B200_OK;
    Anchors an{};
    for (int a = 0; a < num_anchors; ++a)
    {
        an.w[a] = anchor_wh[2 * a];
        an.h[a] = anchor_wh[2 * a + 1];
    }
    const long long total = (long long)N * C_padded * H * W;
    yolo_decode_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        N, C_padded, H, W, num_anchors, num_classes + 5, stride, an, in, out);
    return launched("yolo_decode_kernel");
}

size_t small_b200_nms_scratch_bytes(int32_t max_candidates)
{
    const size_t cap = max_candidates > 0 ? (size_t)max_candidates : 0;
    return 2 * cap * sizeof(Det) + ((cap + 15) & ~(size_t)15) + 16;
}

int small_b200_nms_f32(const float *pred, int32_t num_pred, int32_t num_classes, float confidence_threshold,
                       float iou_threshold, int32_t max_candidates, void *scratch, int32_t max_detections,
                       float *detections, int32_t *counts, void *stream)
{
    if (num_pred < 0 || num_classes <= 0 || max_candidates <= 0 || max_detections < 0 || !scratch || !counts)
        return fail(SMALL_B200_INVALID_ARGUMENT, "NMS ERROR: bad arguments.");
    if ((long long)num_pred * num_classes > 0x7fffffffLL)
        return fail(SMALL_B200_INVALID_ARGUMENT, "NMS ERROR: too many predictions.");
    cudaStream_t st = as_stream(stream);
    uint8_t *base = static_cast<uint8_t *>(scratch);
    Det *cand = reinterpret_cast<Det *>(base);
    Det *sorted = cand + max_candidates;
    unsigned char *alive = reinterpret_cast<unsigned char *>(sorted + max_candidates);
    int *count = reinterpret_cast<int *>(alive + (((size_t)max_candidates + 15) & ~(size_t)15));
    SB_CUDA(cudaMemsetAsync(count, 0, sizeof(int), st));
    if (num_pred > 0)
    {
        collect_kernel<<<(num_pred + 255) / 256, 256, 0, st>>>(num_pred, num_classes, confidence_threshold, pred, cand,
                                                              max_candidates, count);
        if (int rc = launched("collect_kernel"))
            return rc;
    }
    rank_kernel<<<(max_candidates + 255) / 256, 256, 0, st>>>(cand, count, max_candidates, sorted);
    if (int rc = launched("rank_kernel"))
        return rc;
    nms_kernel<<<1, 1024, 0, st>>>(sorted, count, max_candidates, iou_threshold, alive, max_detections, detections, counts);
    return launched("nms_kernel");
}
} // extern "C"
