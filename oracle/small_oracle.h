/*
 * small_oracle.h -- CPU restatement of SMaLL's layer semantics (TEST INFRASTRUCTURE).
 *
 * This is the checker, not the product: only the parity tests, the smoke check and
 * the CPU-baseline leg of the benchmark may link or load it.  The shipped library
 * never calls into it.
 *
 * Every function works on ONE image in SMaLL's packed layout
 *     activations  [C/cb][H][W][cb]
 *     conv filter  [K/cob][C/cib][Fh][Fw][cib][cob]
 *     dw filter    [C/cb][Fh][Fw][cb]
 * (include/small/abstract_layer.hpp:1419-1432, include/small/buffers.hpp:33-120),
 * with the first-layer exception cib := C when C is 1, 2 or 3 and C < cib
 * (include/small/buffers.hpp:52-57).  With cib = cob = 1 the arithmetic order is the
 * one the reference's REF platform executes, so float results are bit-identical to it
 * when this file is compiled with -ffp-contract=off.
 *
 * Parity pinning: checked against the reference's own golden vectors
 * (test/regression_data) and against the reference compiled from its own headers
 * (oracle/_ref/libsmall_ref.so, built by oracle/Makefile) in tests/test_oracle_*.py.
 */
#ifndef SMALL_ORACLE_H
#define SMALL_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Shape of a windowed layer.  Output size follows include/small/utils.hpp:159-165
 * applied to the padded extent: Ho = (H + pad_t + pad_b - Fh)/stride + 1. */
typedef struct so_shape
{
    int32_t C;      /* input channels (reduction dim of a conv; channels of a pool) */
    int32_t K;      /* output channels of a dense conv (ignored elsewhere)          */
    int32_t H, W;   /* input height, width                                          */
    int32_t Fh, Fw; /* window                                                       */
    int32_t stride;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t cib, cob; /* channel blocking of input / output                         */
} so_shape;

/* Quantisation parameters of the uint8 path
 * (include/small/platforms/reference/QUInt8Buffer.hpp:222-230). */
typedef struct so_quant
{
    int32_t zero_in;     /* I.zero(), ADDED to every activation                  */
    int32_t zero_filt;   /* F.zero(), ADDED to every weight                      */
    int32_t lshift, rshift, multiplier; /* taken from the OUTPUT buffer          */
    int32_t k_zero;      /* accumulator seed (q_abstract_layer.hpp:915)          */
} so_quant;

int32_t so_out_dim(int32_t in, int32_t pad_front, int32_t pad_back, int32_t f, int32_t stride);
void    so_calc_padding(int32_t in, int32_t f, int32_t stride, int32_t *front, int32_t *back);

/* ---- float ------------------------------------------------------------- */
/* accumulate != 0 -> PartialConv2D (seed = existing output). bias may be NULL.
 * act: 0 none, 1 ReLU, 2 LeakyReLU(slope); applied after the full reduction, which is
 * what the unfused chain Bias -> PartialConv2D -> activation computes. */
void so_conv2d_f32(const so_shape *s, const float *in, const float *filt,
                   const float *bias, int act, float slope, int accumulate, float *out);
void so_dwconv2d_f32(const so_shape *s, const float *in, const float *filt,
                     const float *bias, int act, float slope, int accumulate, float *out);
/* Grouped convolution: `groups` convolutions from s->C to s->K channels each; s->cob is the
 * group block gb.  I [G/gb][C][H][W][gb], F [G/gb][K][C][Fh][Fw][gb], O [G/gb][K][Ho][Wo][gb];
 * bias is laid out like one output pixel. */
void so_groupconv2d_f32(const so_shape *s, int32_t groups, const float *in, const float *filt,
                        const float *bias, int act, float slope, int accumulate, float *out);
void so_maxpool2d_f32(const so_shape *s, const float *in, float *out);
void so_avgpool2d_f32(const so_shape *s, const float *in, float *out);
void so_relu_f32(int64_t n, const float *in, float *out);
void so_leaky_relu_f32(int64_t n, const float *in, float slope, float *out);
void so_accum_f32(int64_t n, const float *in, float *out);
void so_bias_f32(int32_t C, int32_t H, int32_t W, int32_t cb, const float *bias,
                 int accumulate, float *out);
void so_upsample2d_f32(int32_t C, int32_t H, int32_t W, int32_t cb, int32_t scale,
                       const float *in, float *out);
/* Global softmax over the first n_valid... the reference normalises over every element
 * of the C*H*W tensor (interface_abstract.hpp:1806-1814); n is that count. */
void so_softmax_f32(int32_t C, int32_t H, int32_t W, int32_t cb, const float *in, float *out);

/* ---- uint8 ------------------------------------------------------------- */
int32_t so_requant(int32_t acc, int32_t lshift, int32_t rshift, int32_t multiplier);
/* bias (int32, per output channel, may be NULL) is added to the accumulator seed; the
 * reference itself only has the scalar k_zero seed. */
void so_conv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                  const uint8_t *filt, const int32_t *bias, uint8_t *out);
void so_dwconv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                    const uint8_t *filt, const int32_t *bias, uint8_t *out);
void so_groupconv2d_u8(const so_shape *s, const so_quant *q, int32_t groups, const uint8_t *in,
                       const uint8_t *filt, const int32_t *bias, uint8_t *out);
/* PartialConv2D / PartialDepthwiseConv2D<QUInt8Buffer> (interface_abstract.hpp:595-767, :1194): the
 * accumulators start from the int32 values `partial`, laid out like the output ([Ho][Wo][cob] for the one
 * block of cob output channels for which the reference's in-buffer int32 storage does not overlap
 * itself: s->K == s->cob, resp. s->C == s->cob), and the requantised bytes go to `out`. */
void so_partial_conv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                          const uint8_t *filt, const int32_t *partial, uint8_t *out);
void so_partial_dwconv2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in,
                            const uint8_t *filt, const int32_t *partial, uint8_t *out);
void so_maxpool2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in, uint8_t *out);
void so_relu_u8(int64_t n, const so_quant *q, const uint8_t *in, uint8_t *out);
/* NOT in the reference (no quint8 AveragePool2D exists there): sum of (a+zero_in)
 * over valid taps, requantised with the output's parameters. Parity unpinned. */
void so_avgpool2d_u8(const so_shape *s, const so_quant *q, const uint8_t *in, uint8_t *out);

/* Weight preparation of a convolution layer (include/small/Conv2DLayer.hpp:135-341): zero-padded
 * packing of [Keff][C][Fh][Fw] into K output channels, padded bias, batch-normalisation folding
 * (gamma/beta/mean/var all given or all NULL).  packed_bias may be NULL without bias and BN. */
void so_conv_weights_prepare_f32(int32_t K, int32_t Keff, int32_t C, int32_t Fh, int32_t Fw, int32_t cb,
                                 const float *filt, const float *bias, const float *gamma, const float *beta,
                                 const float *mean, const float *var, float eps, float *packed, float *packed_bias);

/* Detection head.  Box decoding of one packed activation [Cp/cb][H][W][cb] into
 * [num_anchors*H*W][5 + num_classes] records (include/small/YOLOLayer.hpp:96-222); collection of the
 * (record, class) pairs above a confidence threshold and non-maximum suppression
 * (include/small/models/Darknet.hpp:78-122, include/small/non_max_suppression.hpp:98-155): writes up
 * to max_det rows [x, y, w, h, objectness, class score, class id] in keep order, returns how many
 * detections survive, *candidates = pairs above the threshold. */
void so_yolo_decode_f32(int32_t Cp, int32_t H, int32_t W, int32_t cb, int32_t num_anchors, int32_t num_classes,
                        float stride, const float *anchor_wh, const float *in, float *out);
int32_t so_nms_f32(const float *pred, int32_t num_pred, int32_t num_classes, float conf_thr, float iou_thr,
                   int32_t max_det, float *out, int32_t *candidates);

#ifdef __cplusplus
}
#endif
#endif
