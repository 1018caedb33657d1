/*
 * small_b200.h -- C ABI of libsmall_b200.so, the sm_100a implementation of SMaLL's layer
 * loop nest and microkernels.
 *
 * Each entry point replaces one instantiation family of the reference's templated loop
 * nest (small::detail::abstract_layer, include/small/abstract_layer.hpp:1358-1823, and
 * small::quint8_detail::abstract_layer, include/small/q_abstract_layer.hpp:884-1571) as
 * reached through the functional interface (include/small/interface_abstract.hpp).  The
 * reference-side binding is include/small/platforms/b200/ (C++ headers that keep the
 * small:: signatures and forward here).
 *
 * Conventions
 *   - all data pointers are DEVICE pointers (or managed memory) on the current device;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *     calls only enqueue work, they do not synchronise;
 *   - every function returns SMALL_B200_OK or an error code; the text of the last error of
 *     the calling thread is available from small_b200_last_error();
 *   - layouts are SMaLL's packed layouts with channel block 16 for both element types:
 *       activations  [N][C/16][H][W][16]        (image-major batch; N = 1 is the reference)
 *       conv filter  [K/16][C/16][Fh][Fw][16][16]
 *       dw filter    [C/16][Fh][Fw][16]
 *     with the reference's first-layer exception: C in {1,2,3} means block = C
 *     (include/small/buffers.hpp:52-57), i.e. an HWC-interleaved image;
 *   - output size: Ho = (H + pad_t + pad_b - Fh)/stride + 1 (include/small/utils.hpp:159).
 */
#ifndef SMALL_B200_H
#define SMALL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMALL_B200_CB 16 /* FLOAT_C_ob = FLOAT_C_ib = QUINT8_C_ob = QUINT8_C_ib */

enum
{
    SMALL_B200_OK = 0,
    SMALL_B200_INVALID_ARGUMENT = 1, /* maps to std::invalid_argument (unsupported stride/channels) */
    SMALL_B200_CUDA_ERROR = 2,       /* maps to std::runtime_error */
    SMALL_B200_OUT_OF_MEMORY = 3,    /* maps to std::bad_alloc */
    SMALL_B200_DEVICE_TIMEOUT = 4    /* a bounded device-side wait ran out */
};

enum
{
    SMALL_B200_ACT_NONE = 0,
    SMALL_B200_ACT_RELU = 1, /* max(x, 0)        FLOAT_MAX_TILE_C on a zeroed tile        */
    SMALL_B200_ACT_LEAKY = 2 /* x>0 ? x : x*slope FLOAT_COND_SCALE_TILE_C                 */
};

/* Shape of one windowed layer call.  Mirrors the argument list the functional interface
 * passes to the loop nest (interface_abstract.hpp:46-58 -> abstract_layer.hpp:1368-1385),
 * plus the batch and what the fused interface adds (fused_interface_abstract.hpp:217). */
typedef struct small_b200_layer
{
    int32_t N;      /* images in the batch                                               */
    int32_t C;      /* input channels                                                    */
    int32_t K;      /* output channels of a dense conv; ignored by per-channel layers    */
    int32_t H, W;   /* input height / width                                              */
    int32_t Fh, Fw; /* window                                                            */
    int32_t stride;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t accumulate; /* 1 = Partial* form: start from the existing output            */
    int32_t act;        /* SMALL_B200_ACT_*, applied after the full reduction            */
    float slope;        /* LeakyReLU negative slope                                      */
    /* uint8 path (ignored by float entry points); semantics of
     * include/small/platforms/reference/intrinsics_quint8.h:191-206,481-531:
     * acc = k_zero + bias[k] + sum over VALID taps (a + zero_in) * (w + zero_filt),
     * out = clamp(rounding_shift(high_mul(acc << lshift, multiplier), rshift), 0, 255) */
    int32_t zero_in, zero_filt;
    int32_t lshift, rshift, multiplier;
    int32_t k_zero;
    /* Stride along the height when it differs from `stride` (which then is the stride along the
     * width only); 0 = the same stride on both axes.  The reference's 1-D family is its 2-D loop
     * nest with the batch in place of the height (abstract_layer.hpp:1838-1846): a 1-D layer of
     * stride s is a layer with Fh = 1, stride_h = 1, stride = s.  Honoured by the fp32 windowed
     * layers (convolution on the CUDA cores, depthwise, grouped, pools); other entry points refuse
     * a row stride that differs. */
    int32_t stride_h;
} small_b200_layer;

/* ---- library / device ------------------------------------------------------------ */
const char *small_b200_last_error(void);
int small_b200_device_count(int *count);
int small_b200_set_device(int device);
/* Synchronises the device and reports whether any kernel gave up on a bounded device-side
 * wait (tensor-core kernels poll their mbarriers with an iteration limit instead of
 * spinning forever).  *status = 0 when all is well; otherwise SMALL_B200_DEVICE_TIMEOUT is
 * returned and the word is cleared (a failure is reported once; while it is set, every other
 * bounded wait gives up early too, so that a whole launch drains quickly).  No counterpart in
 * the reference (a CPU loop nest has nothing to wait for). */
int small_b200_device_status(int *status);
/* Self-test of that mechanism: launches one warp that holds tensor memory and waits, with the
 * same bounded wait the tensor-core kernels use and a limit of `polls` polls (1..4096), on a
 * barrier nobody arrives on.  The wait gives up by construction, the kernel frees its tensor
 * memory and returns; the next small_b200_device_status() reports SMALL_B200_DEVICE_TIMEOUT
 * (code 99) and clears it.  No counterpart in the reference. */
int small_b200_selftest_bounded_wait(uint32_t polls, void *stream);
/* What a pipe of the current device delivers when only issue stands in the way (operands resident
 * in registers / shared memory / tensor memory): kind 0 = fp32 FMA pipe, 1 = tcgen05 kind::tf32
 * MMA, 2 = tcgen05 kind::i8 MMA.  Runs a short probe kernel on the default stream, synchronously,
 * and returns tera-operations per second (2 per multiply-add) in *tera_ops.  These are the
 * denominators of the benchmark's per-layer roofline figures.  kind 3 / 4: the same probe with
 * M = 128, N = 32 instructions of kind::tf32 / kind::i8; the result is then the pipe's CYCLES PER
 * INSTRUCTION at the device's maximum clock -- the floor a narrow MMA costs, which bounds layers
 * that need many small instructions.  No counterpart in the reference. */
int small_b200_peak_probe(int kind, double *tera_ops);
/* Number of kernels this library has launched in this process since it was loaded. */
uint64_t small_b200_launch_count(void);

/* ---- memory (the platform's alloc_buffer/free_buffer,
 *      include/small/platforms/reference/Buffer.hpp:36-61, FloatBuffer.hpp:59-77) ------- */
int small_b200_malloc(size_t bytes, void **ptr);         /* device memory                  */
int small_b200_malloc_managed(size_t bytes, void **ptr); /* host-visible (Buffer::data()) */
int small_b200_malloc_host(size_t bytes, void **ptr);    /* pinned host staging            */
/* Pinned, write-combined host memory for staging buffers the host only WRITES (sequentially) and the
 * device reads: the device's reads do not snoop the CPU caches.  Host reads from it are very slow.
 * Freed with small_b200_free_host. */
int small_b200_malloc_host_upload(size_t bytes, void **ptr);
int small_b200_free(void *ptr);
int small_b200_free_host(void *ptr);
int small_b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
int small_b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
int small_b200_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
int small_b200_prefetch(const void *managed_ptr, size_t bytes, void *stream); /* to the device */

/* ---- streams and graphs ------------------------------------------------------------ */
int small_b200_stream_create(void **stream);
int small_b200_stream_destroy(void *stream);
int small_b200_stream_sync(void *stream);
int small_b200_device_sync(void);
/* Capture everything enqueued on `stream` between begin and end into one executable graph. */
int small_b200_graph_begin(void *stream);
int small_b200_graph_end(void *stream, void **graph_exec);
int small_b200_graph_launch(void *graph_exec, void *stream);
int small_b200_graph_destroy(void *graph_exec);

/* ---- float layers ------------------------------------------------------------------ */
/* small::Conv2D / PartialConv2D<FloatBuffer> (interface_abstract.hpp:46-221, :416-587) with
 * the bias-before / activation-after slots of the fused interface
 * (fused_interface_abstract.hpp:55, :217).  bias may be NULL.  K % 16 == 0;
 * C % 16 == 0 or C in {1,2,3}; stride in {1,2}. */
int small_b200_conv2d_f32(const small_b200_layer *L, const float *in, const float *filt,
                          const float *bias, float *out, void *stream);
/* small::Conv2D_Maxpool2D / Conv2D_ReLU_Maxpool2D / Conv2D_Bias_ReLU_Maxpool2D<FloatBuffer>
 * (fused_interface_abstract.hpp:463-1418): the convolution `conv` (stride 1, bias / activation
 * slots as above) followed by the 2x2 stride-2 unpadded max pool `pool` in ONE kernel; the
 * full-size activation never reaches memory.  `out` holds the pooled tensor
 * [N][K/16][Ho/2][Wo/2][16].  ..._supported() says whether the pair of shapes is covered (even
 * Ho and Wo, K % 32 == 0 unless it is a first layer with C in {1,2,3}, pool 2x2/2 without padding); other pairs run as two calls. */
int small_b200_conv2d_maxpool_f32_supported(const small_b200_layer *conv, const small_b200_layer *pool);
int small_b200_conv2d_maxpool_f32(const small_b200_layer *conv, const small_b200_layer *pool, const float *in,
                                  const float *filt, const float *bias, float *out, void *stream);
/* The same layer on the tensor cores (tcgen05 kind::tf32 with the 3xTF32 operand split, fp32
 * accumulation in tensor memory), stride 1 only.  Each fp32 operand x enters the tensor core as
 * hi = x (its 13 low mantissa bits are ignored) and lo = x - hi; the lo copy of the activations
 * is made inside the kernel, in shared memory.  The caller provides the filter re-laid for the
 * tensor core:
 *   filt_prepared  small_b200_filter_prepare_tf32x3(filt), once per set of weights,
 *                  2 * K*C*Fh*Fw floats: per CTA tile and tap the filter as [c/4][k][4 c]
 *                  (what the tensor core reads directly) followed by its lo copy; for K = 16 or 32
 *                  the lo rows of every 4-channel chunk follow its hi rows directly
 *                  ([c/4][hi k | lo k][4 c]).  The layout depends on K alone; treat it as opaque.
 * ..._supported() says whether a shape is covered (1) or not (0).  The reference has no
 * counterpart of the preparation call (its filters are used as packed). */
int small_b200_conv2d_f32_tf32x3_supported(const small_b200_layer *L);
/* The library's own choice between the two fp32 convolutions for a shape and batch: 1 when the
 * tensor-core kernel covers it and is the faster one (at least 16 input channels, and either an
 * image of at least 9 output pixels or a 1x1 layer whose tiles run across the images of a batch
 * of at least 256 pixels in all), else 0.  The C++ platform headers and the Python executor both
 * ask here, so they pick the same kernel for the same call. */
int small_b200_conv2d_f32_tf32x3_preferred(const small_b200_layer *L);
int small_b200_filter_prepare_tf32x3(const small_b200_layer *L, const float *filt, float *prepared, void *stream);
int small_b200_conv2d_f32_tf32x3(const small_b200_layer *L, const float *in, const float *filt_prepared,
                                 const float *bias, float *out, void *stream);
/* small::Conv2D_Maxpool2D / Conv2D_ReLU_Maxpool2D / Conv2D_Bias_ReLU_Maxpool2D<FloatBuffer>
 * (fused_interface_abstract.hpp:463-1418) on the tensor cores: the convolution above with the 2x2
 * stride-2 unpadded max pool `pool` in its epilogue; `out` holds the pooled tensor
 * [N][K/16][Ho/2][Wo/2][16].  Covered: 32 or 64 output channels on images wider than 64 pixels
 * (with padding), odd filter width, even Ho and Wo, no accumulation, an activation that does not
 * decrease (it is applied after the maximum); ..._supported() says so, other pairs run as two calls. */
int small_b200_conv2d_maxpool_f32_tf32x3_supported(const small_b200_layer *conv, const small_b200_layer *pool);
int small_b200_conv2d_maxpool_f32_tf32x3(const small_b200_layer *conv, const small_b200_layer *pool, const float *in,
                                         const float *filt_prepared, const float *bias, float *out, void *stream);
/* The tensor-core convolution above for callers that cannot allocate device memory (code
 * running where cudaMalloc is forbidden or would stall the device, plug-ins that are handed
 * nothing but their input and output pointers).  It takes the PACKED filter as the reference
 * lays it out and keeps its scratch -- the re-laid filter and its lo copy -- in a fixed 16 MiB
 * array inside the library, so it calls no allocator of any kind.  Limits and rules:
 *   - 2*K*C*Fh*Fw floats must fit in 4 Mi floats; larger calls are
 *     refused with SMALL_B200_INVALID_ARGUMENT and a message that states both sizes;
 *   - the first call on each device looks up the array's device address; make that first call
 *     outside any stream capture;
 *   - all calls share the one array, which keeps whatever the last call left in it (nothing in
 *     it needs clearing: every call rewrites what it reads); two calls whose kernels overlap
 *     on the GPU -- different streams, or graphs launched side by side -- race on it;
 *   - the filter is re-laid on every call, so with fixed weights the variant with
 *     caller-provided scratch is faster.
 * This entry point has no counterpart in the reference. */
int small_b200_conv2d_f32_tf32x3_noalloc(const small_b200_layer *L, const float *in, const float *filt,
                                         const float *bias, float *out, void *stream);
/* small::DepthwiseConv2D / PartialDepthwiseConv2D<FloatBuffer> (:994, :1127) and
 * DepthwiseConv2D_Bias_ReLU (fused_interface_abstract.hpp:1419). */
int small_b200_dwconv2d_f32(const small_b200_layer *L, const float *in, const float *filt,
                            const float *bias, float *out, void *stream);
/* small::GroupConv2D / PartialGroupConv2D<FloatBuffer> (:1265, :1402): `groups` independent
 * convolutions, each from L->C input channels to L->K output channels (the reference's
 * interface passes its input_channels argument for both).  Layouts of the loop nest with
 * G_b = 16, K_b = F_cb = 1 (abstract_layer.hpp:1419-1432): the 16 lanes of a block are 16
 * groups,
 *   in [N][G/16][C][H][W][16]   filt [G/16][K][C][Fh][Fw][16]   out [N][G/16][K][Ho][Wo][16]
 * bias (may be NULL) is laid out like one output pixel, [G/16][K][16].  groups % 16 == 0;
 * stride in {1,2}.  The reference's own float instantiation treats the lanes of a block as a
 * dense channel block (op_class 2, :1291), which is a grouped convolution only for a channel
 * block of 1; this entry point computes the grouped convolution the layout describes and is
 * checked against the reference built with a channel block of 1. */
int small_b200_groupconv2d_f32(const small_b200_layer *L, int32_t groups, const float *in, const float *filt,
                               const float *bias, float *out, void *stream);
/* The grouped convolution of the reference's FUSED interface (GroupConv2D_ReLU, Conv2D_GroupConv, ...,
 * fused_interface_abstract.hpp:2507-3667), which is a different layer from small::GroupConv2D: there
 * G = output_groups, K = C_ob, F_c = C_ib (:2740-2760), i.e. `groups` dense convolutions from 16 to 16
 * channels, group g on channel block g:
 *   in [N][G][H][W][16]   filt [G][Fh][Fw][16 c][16 k]   out [N][G][Ho][Wo][16]
 * bias (may be NULL) [G][16]; L->C and L->K are ignored; stride in {1,2}; act / accumulate as usual. */
int small_b200_blockconv2d_f32(const small_b200_layer *L, int32_t groups, const float *in, const float *filt,
                               const float *bias, float *out, void *stream);
/* small::MaxPool2D<FloatBuffer> (:778): border windows start from 0, interior from the
 * first tap. */
int small_b200_maxpool2d_f32(const small_b200_layer *L, const float *in, float *out, void *stream);
/* small::AveragePool2D<FloatBuffer> (:910): sum of valid taps times 1/(Fh*Fw); strides 1,2,3. */
int small_b200_avgpool2d_f32(const small_b200_layer *L, const float *in, float *out, void *stream);
/* small::ReLUActivation (:1541), LeakyReLUActivation (:1616), Accum (:1950); n = elements. */
int small_b200_relu_f32(int64_t n, const float *in, float *out, void *stream);
int small_b200_leaky_relu_f32(int64_t n, const float *in, float slope, float *out, void *stream);
int small_b200_accum_f32(int64_t n, const float *in, float *out, void *stream);
/* small::Dropout (:1697): every element times the rate held in the filter buffer (OP_MUL,
 * abstract_layer.hpp:82-86: the tile is loaded from the input and multiplied). */
int small_b200_scale_f32(int64_t n, const float *in, float scale, float *out, void *stream);
/* small::Bias / PartialBias (:1992, :2035): out[n][c][h][w] (+)= bias[c]. */
int small_b200_bias_f32(int32_t N, int32_t C, int32_t H, int32_t W, const float *bias,
                        int32_t accumulate, float *out, void *stream);
/* small::UpSample2D (:1845), scale 2: out[h][w] = in[h/2][w/2]. */
int small_b200_upsample2d_f32(int32_t N, int32_t C, int32_t H, int32_t W, const float *in,
                              float *out, void *stream);
/* small::UpSample1D (interface_abstract_1D.hpp:1614), scale 2 along the width only:
 * out[row][w] = in[row][w/2] over [C/16][rows][W][16] (rows = the 1-D family's batch). */
int small_b200_upsample1d_f32(int32_t N, int32_t C, int32_t rows, int32_t W, const float *in,
                              float *out, void *stream);
/* small::SoftMax (:1778): per image, exp / sum over all C*H*W elements, no max subtraction. */
int small_b200_softmax_f32(int32_t N, int64_t elems_per_image, const float *in, float *out,
                           void *stream);
/* small::Concat (:2072): per image, channel concatenation = two contiguous copies.
 * bytes0 / bytes1 are per-image sizes. */
int small_b200_concat(int32_t N, size_t bytes0, const void *in0, size_t bytes1, const void *in1,
                      void *out, void *stream);

/* ---- weights ----------------------------------------------------------------------- */
/* detail::initialize_conv2d_buffers (include/small/Conv2DLayer.hpp:135-341) on the device: the
 * unpacked filter [K_effective][C][Fh][Fw] is packed to [K_padded/16][C/cib][Fh][Fw][cib][16] with
 * zero filters for the padded output channels (:393-404), the bias (may be NULL) is padded with
 * zeros, and batch-normalisation parameters (all four or none) are folded into both:
 * scale = gamma / sqrt(var + eps), filters *= scale, bias = beta - mean * scale (no bias) or
 * beta + scale * (bias - mean).  packed_bias (K_padded floats) may be NULL when there is neither a
 * bias nor batch normalisation.  All pointers are device pointers.  Bit-identical to the host code. */
int small_b200_conv_weights_prepare_f32(int32_t K_padded, int32_t K_effective, int32_t C, int32_t Fh, int32_t Fw,
                                        const float *filters, const float *bias, const float *bn_weight,
                                        const float *bn_bias, const float *bn_running_mean,
                                        const float *bn_running_var, float bn_eps, float *packed_filters,
                                        float *packed_bias, void *stream);

/* ---- detection head ---------------------------------------------------------------- */
/* small::YOLOLayer::compute_output (include/small/YOLOLayer.hpp:96-222): the packed activation
 * [N][C_padded/16][H][W][16], read as [anchor][5 + classes][H][W], becomes one record
 * [x, y, w, h, objectness, class scores...] per anchor and pixel:
 *   x = stride * (sigmoid(v) + column), y = stride * (sigmoid(v) + row), w = exp(v) * anchor_w,
 *   h = exp(v) * anchor_h, everything else sigmoid(v).
 * out: [N][num_anchors * H * W][5 + num_classes], prediction index (anchor * H + row) * W + column.
 * anchor_wh is a HOST array of num_anchors (width, height) pairs (at most 16).  Channels beyond
 * num_anchors * (5 + num_classes) are the padding of the layer before and are ignored. */
int small_b200_yolo_decode_f32(int32_t N, int32_t C_padded, int32_t H, int32_t W, int32_t num_anchors,
                               int32_t num_classes, float stride, const float *anchor_wh, const float *in,
                               float *out, void *stream);
/* Darknet::process_outputs + small::basic_nms (include/small/models/Darknet.hpp:78-122,
 * include/small/non_max_suppression.hpp:98-155) for num_pred records of 5 + num_classes floats (the
 * outputs of one or several decode calls, back to back): every (record, class) pair whose objectness
 * AND class score exceed confidence_threshold is a detection; detections are ordered by objectness,
 * descending (ties: the order the host loop meets them in), and a kept detection removes every later
 * one of its class whose IoU with it is not below iou_threshold.
 *   detections  [max_detections][7] = x, y, w, h, objectness, class score, class id; in keep order
 *   counts      [2] (device) = detections that survive (may exceed max_detections: only that many
 *               are written), pairs above the confidence threshold (if it exceeds max_candidates,
 *               the surplus was dropped and the result is incomplete)
 *   scratch     small_b200_nms_scratch_bytes(max_candidates) bytes of device memory */
size_t small_b200_nms_scratch_bytes(int32_t max_candidates);
int small_b200_nms_f32(const float *pred, int32_t num_pred, int32_t num_classes, float confidence_threshold,
                       float iou_threshold, int32_t max_candidates, void *scratch, int32_t max_detections,
                       float *detections, int32_t *counts, void *stream);

/* ---- uint8 layers ------------------------------------------------------------------ */
/* small::Conv2D<QUInt8Buffer> (:229-404) with an optional per-channel int32 bias added to
 * the accumulator seed.  The int32 partial sums never leave the chip, so the output buffer
 * needs no 4x over-allocation (the reference's does, q_abstract_layer.hpp:1144).
 * L->accumulate = 1 is small::PartialConv2D<QUInt8Buffer> (:595-767): `out` holds int32 partial sums
 * [Ho*Wo][16] on entry (4 * 16 * Ho*Wo bytes) and the bytes [Ho*Wo][16] of requantise(entry +
 * convolution) at its start on return.  The reference keeps the int32 sums of output channel block k
 * at BYTE k * Ho*Wo*block of the uint8 buffer, four times the block's length, so the sums of one block
 * lie over the next three: the form has a defined result for one block only, and this entry point
 * takes K = 16, N = 1, bias = NULL and refuses the rest (SMALL_B200_INVALID_ARGUMENT). */
int small_b200_conv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                         const int32_t *bias, uint8_t *out, void *stream);
/* The same layer on a path of the caller's choosing.  small_b200_conv2d_u8 picks, per shape, the faster
 * of two implementations of the same arithmetic: tcgen05 kind::i8 kernels (1x1 layers from shared-memory
 * resident filters, the one-channel first layer as an im2col GEMM, and an implicit GEMM over a ring of
 * im2col stages that covers every window, stride, padding, channel count and zero point) and CUDA-core
 * kernels (dp4a / direct), which keep the layers whose reduction is a single 32-byte step.
 * ..._cuda_cores never uses the tensor cores; ..._tensor_core always does and fails with
 * SMALL_B200_INVALID_ARGUMENT for what they do not cover (the int32 partial-sum form, unaligned
 * buffers).  All three give identical bits.  No reference counterpart. */
int small_b200_conv2d_u8_cuda_cores(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                                    const int32_t *bias, uint8_t *out, void *stream);
int small_b200_conv2d_u8_tensor_core(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                                     const int32_t *bias, uint8_t *out, void *stream);
/* Two uint8 layers as ONE kernel, the intermediate activation kept in shared memory: the
 * reference's Conv2D_ReLU_DepthwiseConv2D_ReLU fusion (fused_interface_abstract.hpp:1840, float
 * there) for quint8 buffers, where the clamp of the requantisation is the ReLU.  `conv` is a 1x1
 * convolution (C % 32 == 0, C <= 128) or a one-channel first layer (Fw <= 4, Fh <= 16), K in
 * {32, 64}, on an image whose OUTPUT has at most 128 pixels; `dw` is the 3x3 stride-1 depthwise
 * convolution with pads 1,1,1,1 of that output.  Both run on the tensor cores (a depthwise tap
 * as a GEMM with a diagonal weight block).  Filter zero points must be -128, the intermediate's
 * zero point (dw->zero_in) 0 or -128.  Each layer carries its own requantisation in its
 * descriptor; biases may be NULL.  ..._supported() says whether a pair is covered; other pairs
 * run as two calls.  Bit-identical to the two calls. */
int small_b200_conv2d_dwconv2d_u8_supported(const small_b200_layer *conv, const small_b200_layer *dw);
int small_b200_conv2d_dwconv2d_u8(const small_b200_layer *conv, const small_b200_layer *dw, const uint8_t *in,
                                  const uint8_t *conv_filt, const int32_t *conv_bias, const uint8_t *dw_filt,
                                  const int32_t *dw_bias, uint8_t *out, void *stream);
/* The tail of the keyword-spotting network (include/small/models/DSCNNTiny.hpp) as one kernel:
 * `conv` as above, the global average pool `pool` of its output (window = the whole image) and
 * the dense layer `dense` (a 1x1 convolution on the pooled 1x1 image, K <= 128) on the pooled
 * vector.  `out` holds [N][dense->K] bytes.  Bit-identical to the three calls.  The reference has
 * no such entry (it has no quint8 average pool at all). */
int small_b200_conv2d_avgpool_dense_u8_supported(const small_b200_layer *conv, const small_b200_layer *pool,
                                                 const small_b200_layer *dense);
int small_b200_conv2d_avgpool_dense_u8(const small_b200_layer *conv, const small_b200_layer *pool,
                                       const small_b200_layer *dense, const uint8_t *in, const uint8_t *conv_filt,
                                       const int32_t *conv_bias, const uint8_t *dense_filt, const int32_t *dense_bias,
                                       uint8_t *out, void *stream);
/* small::DepthwiseConv2D<QUInt8Buffer> (:1059); with L->accumulate = 1 PartialDepthwiseConv2D (:1194)
 * under the conditions of the partial convolution above (C = 16, N = 1, bias = NULL). */
int small_b200_dwconv2d_u8(const small_b200_layer *L, const uint8_t *in, const uint8_t *filt,
                           const int32_t *bias, uint8_t *out, void *stream);
/* small::GroupConv2D<QUInt8Buffer> (:1332; lane-wise op_class 1 at :1358), layouts as in the
 * float form, arithmetic as in small_b200_conv2d_u8.  The Partial form (:1470) keeps the int32
 * sums of output channel k of the groups at byte k * Ho*Wo*16, four times the channel's length: for
 * the multiples of 16 channels per group the interface accepts they always overlap, so no shape has
 * a defined result and L->accumulate = 1 is refused. */
int small_b200_groupconv2d_u8(const small_b200_layer *L, int32_t groups, const uint8_t *in, const uint8_t *filt,
                              const int32_t *bias, uint8_t *out, void *stream);
/* small::MaxPool2D<QUInt8Buffer> (:843): interior windows start from the raw first tap,
 * border windows from k_zero; taps enter as a + zero_in; the maximum is requantised. */
int small_b200_maxpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream);
/* No counterpart in the reference (it has no quint8 average pool): sum over valid taps of
 * (a + zero_in), requantised with the layer's multiplier and shifts. */
int small_b200_avgpool2d_u8(const small_b200_layer *L, const uint8_t *in, uint8_t *out, void *stream);
/* small::ReLUActivation<QUInt8Buffer> (:1577): requantise max(a + zero_in, k_zero). */
int small_b200_relu_u8(int64_t n, const small_b200_layer *L, const uint8_t *in, uint8_t *out,
                       void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SMALL_B200_H */
