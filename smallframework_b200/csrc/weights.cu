// weights.cu -- what a convolution layer does to its weights once, when a model is built:
// detail::initialize_conv2d_buffers of the reference (include/small/Conv2DLayer.hpp:135-341):
//   * output channels are padded up to the block (zero filters, zero biases),
//   * the filter [K][C][Fh][Fw] is packed to [K/16][C/cib][Fh][Fw][cib][16]
//     (small::packed_weight_index, include/small/buffers.hpp:33-79; cib = C for C in {1,2,3}),
//   * batch normalisation is folded in: scale = gamma * (1 / sqrt(var + eps)); filters of channel k
//     are multiplied by scale[k]; bias[k] = beta - mean * scale without a convolution bias, else
//     beta + scale * (bias - mean)  (:295-331).
// The reference does this on the host per layer; for a network whose weights already live on the
// device (a loader that streams a weight file to the GPU) it is one kernel per layer: a thread per
// packed filter element looks up its source element, and the first K threads also make the bias.
// Arithmetic uses the reference's operations one by one (round-to-nearest, no fused multiply-add),
// so the results are the host's bit for bit.
#include "common.cuh"

namespace
{
using namespace sb;

struct PrepArgs
{
    int K, Keff, C, Fh, Fw, cib;
    float eps;
};

__device__ __forceinline__ float bn_scale(const PrepArgs &a, const float *gamma, const float *var, int k)
{
    const float rsq = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var[k], a.eps)));
    return __fmul_rn(gamma[k], rsq);
}

__global__ void __launch_bounds__(256)
prepare_conv_weights_kernel(const PrepArgs a, const float *__restrict__ filt, const float *__restrict__ bias,
                            const float *__restrict__ gamma, const float *__restrict__ beta,
                            const float *__restrict__ mean, const float *__restrict__ var,
                            float *__restrict__ packed, float *__restrict__ packed_bias)
{
    const long long total = (long long)a.K * a.C * a.Fh * a.Fw;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a.K && packed_bias)
    {
        const int k = (int)i;
        float b = 0.f;
        if (k < a.Keff)
        {
            b = bias ? bias[k] : 0.f;
            if (gamma)
            {
                const float s = bn_scale(a, gamma, var, k);
                b = bias ? __fadd_rn(beta[k], __fmul_rn(s, __fsub_rn(b, mean[k])))
                         : __fsub_rn(beta[k], __fmul_rn(mean[k], s));
            }
        }
        packed_bias[k] = b;
    }
    if (i >= total)
        return;
    // packed position -> (k, c, kh, kw): [K/16][C/cib][Fh][Fw][cib][16]
    const long long o = i;
    const int k16 = (int)(i % CB); i /= CB;
    const int ci = (int)(i % a.cib); i /= a.cib;
    const int kw = (int)(i % a.Fw); i /= a.Fw;
    const int kh = (int)(i % a.Fh); i /= a.Fh;
    const int cbk = (int)(i % (a.C / a.cib));
    const int kb = (int)(i / (a.C / a.cib));
    const int k = kb * CB + k16, c = cbk * a.cib + ci;
    float v = 0.f;
    if (k < a.Keff)
    {
        v = filt[(((size_t)k * a.C + c) * a.Fh + kh) * a.Fw + kw];
        if (gamma)
            v = __fmul_rn(v, bn_scale(a, gamma, var, k));
    }
    packed[o] = v;
}
} // namespace

extern "C" int small_b200_conv_weights_prepare_f32(int32_t K_padded, int32_t K_effective, int32_t C, int32_t Fh,
                                                   int32_t Fw, const float *filters, const float *bias,
                                                   const float *bn_weight, const float *bn_bias,
                                                   const float *bn_running_mean, const float *bn_running_var,
                                                   float bn_eps, float *packed_filters, float *packed_bias,
                                                   void *stream)
{
    if (K_padded <= 0 || K_padded % CB != 0 || K_effective <= 0 || K_effective > K_padded)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2DLayer::ctor error: invalid number of output channels.");
    if (C <= 0 || (C % CB != 0 && C != 1 && C != 2 && C != 3) || Fh <= 0 || Fw <= 0)
        return fail(SMALL_B200_INVALID_ARGUMENT, "Conv2DLayer::ctor ERROR: in_channels unsupported.");
    const int bn = (bn_weight ? 1 : 0) + (bn_bias ? 1 : 0) + (bn_running_mean ? 1 : 0) + (bn_running_var ? 1 : 0);
    if (bn != 0 && bn != 4) // all or nothing, Conv2DLayer.hpp:241-253
        return fail(SMALL_B200_INVALID_ARGUMENT, "*Conv2DLayer::ctor ERROR: BN buffers incorrect size.");
    if (!filters || !packed_filters || ((bias || bn) && !packed_bias))
        return fail(SMALL_B200_INVALID_ARGUMENT, "*Conv2DLayer::ctor ERROR: filters buffer is incorrect size.");
    PrepArgs a{K_padded, K_effective, C, Fh, Fw, C < CB ? C : CB, bn_eps};
    const long long total = (long long)K_padded * C * Fh * Fw;
    prepare_conv_weights_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        a, filters, bias, bn_weight, bn_bias, bn_running_mean, bn_running_var, packed_filters, packed_bias);
    return launched("prepare_conv_weights_kernel");
}
