// The small operators a MobileNetV1 training step needs around the convolutions: Threshold (ReLU),
// SpatialAveragePooling, LogSoftMax, ClassNLLCriterion and the plain SGD parameter update.  All are
// bandwidth-bound or tiny; they exist so that the whole step runs on the GPU behind the same C ABI.
#include "common.cuh"

#include <float.h>
#include <algorithm>

namespace cunn {
namespace sup {

static int grid_for(long long n, int per_thread = 4)
{
    const long long want = ceil_div_ll(n, 256LL * per_thread);
    return (int)std::max(1LL, std::min(want, (long long)sm_count() * 32));
}

// y = x > th ? x : val  (lib/THCUNN/Threshold.cu:6-38); y may alias x.
__global__ void __launch_bounds__(256)
threshold_fwd_kernel(const float *x, float *y, long long n, float th, float val)
{
    const long long n4 = n >> 2;
    const bool vec = ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (vec) {
        for (long long q = i; q < n4; q += stride) {
            float4 v = reinterpret_cast<const float4 *>(x)[q];
            v.x = v.x > th ? v.x : val; v.y = v.y > th ? v.y : val; v.z = v.z > th ? v.z : val; v.w = v.w > th ? v.w : val;
            reinterpret_cast<float4 *>(y)[q] = v;
        }
        for (long long q = n4 * 4 + i; q < n; q += stride) y[q] = x[q] > th ? x[q] : val;
    } else {
        for (long long q = i; q < n; q += stride) y[q] = x[q] > th ? x[q] : val;
    }
}

// gx = x > th ? gy : 0  (lib/THCUNN/Threshold.cu:40-72); gx may alias gy.
__global__ void __launch_bounds__(256)
threshold_bwd_kernel(const float *x, const float *gy, float *gx, long long n, float th)
{
    const long long n4 = n >> 2;
    const bool vec = ((((uintptr_t)x | (uintptr_t)gy | (uintptr_t)gx) & 15) == 0);
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (vec) {
        for (long long q = i; q < n4; q += stride) {
            const float4 v = reinterpret_cast<const float4 *>(x)[q];
            float4 g = reinterpret_cast<const float4 *>(gy)[q];
            g.x = v.x > th ? g.x : 0.f; g.y = v.y > th ? g.y : 0.f; g.z = v.z > th ? g.z : 0.f; g.w = v.w > th ? g.w : 0.f;
            reinterpret_cast<float4 *>(gx)[q] = g;
        }
        for (long long q = n4 * 4 + i; q < n; q += stride) gx[q] = x[q] > th ? gy[q] : 0.f;
    } else {
        for (long long q = i; q < n; q += stride) gx[q] = x[q] > th ? gy[q] : 0.f;
    }
}

// Average pooling.  The divisor rule is the reference's and has to be (lib/THCUNN/SpatialAveragePooling.cu:7-82): a
// window is first clipped to input + padding, which gives the count_include_pad divisor, then to the input, which gives
// the summed range and the other divisor.  Both kernels treat the two axes separately through Span1D, so the 2-D divisor
// is a product of two per-axis extents; the backward pass is in gather form (one thread per input pixel, no atomics).
struct Span1D {
    int lo, hi;      // taps inside the input: [lo, hi)
    int padded;      // taps inside input + padding
};

__device__ __forceinline__ Span1D window_span(int o, int k, int d, int pad, int size)
{
    const int start = o * d - pad;
    const int stop = min(start + k, size + pad);
    Span1D s;
    s.padded = stop - start;
    s.lo = max(start, 0);
    s.hi = min(stop, size);
    return s;
}

__device__ __forceinline__ float window_divisor(const Span1D &r, const Span1D &c, int include_pad)
{
    return (float)(include_pad ? r.padded * c.padded : (r.hi - r.lo) * (c.hi - c.lo));
}

// outputs whose window covers input coordinate i (already shifted by the padding): [first, last)
__device__ __forceinline__ void covering_outputs(int i_padded, int k, int d, int osize, int &first, int &last)
{
    first = i_padded < k ? 0 : (i_padded - k) / d + 1;
    last = min(i_padded / d + 1, osize);
}

__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, int H, int W, int oH, int oW, int kH, int kW, int dH,
                   int dW, int padH, int padW, int include_pad, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(idx % oW);
        const long long t = idx / oW;
        const int oh = (int)(t % oH);
        const Span1D r = window_span(oh, kH, dH, padH, H), c = window_span(ow, kW, dW, padW, W);
        const float *xp = x + (t / oH) * (long long)H * W;
        float s = 0.f;
        for (int h = r.lo; h < r.hi; ++h)
            for (int w = c.lo; w < c.hi; ++w) s += __ldg(xp + h * W + w);
        y[idx] = s / window_divisor(r, c, include_pad);
    }
}

__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const float *__restrict__ gy, float *__restrict__ gx, int H, int W, int oH, int oW, int kH, int kW,
                   int dH, int dW, int padH, int padW, int include_pad, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / W;
        int oh0, oh1, ow0, ow1;
        covering_outputs((int)(t % H) + padH, kH, dH, oH, oh0, oh1);
        covering_outputs((int)(idx % W) + padW, kW, dW, oW, ow0, ow1);
        const float *gp = gy + (t / H) * (long long)oH * oW;
        float g = 0.f;
        for (int oh = oh0; oh < oh1; ++oh) {
            const Span1D r = window_span(oh, kH, dH, padH, H);
            for (int ow = ow0; ow < ow1; ++ow)
                g += __ldg(gp + oh * oW + ow) / window_divisor(r, window_span(ow, kW, dW, padW, W), include_pad);
        }
        gx[idx] = g;
    }
}

__device__ __forceinline__ float block_reduce(float v, float *sh, bool is_max)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
    return r;
}

// y = x - max - log(sum exp(x - max)) per row (lib/THCUNN/LogSoftMax.cu:246-296).
__global__ void __launch_bounds__(256)
logsoftmax_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, int D)
{
    __shared__ float sh[8];
    const float *xp = x + (size_t)blockIdx.x * D;
    float *yp = y + (size_t)blockIdx.x * D;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < D; i += blockDim.x) m = fmaxf(m, xp[i]);
    m = block_reduce(m, sh, true);
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += expf(xp[i] - m);
    s = block_reduce(s, sh, false);
    const float l = m + logf(s);
    for (int i = threadIdx.x; i < D; i += blockDim.x) yp[i] = xp[i] - l;
}

// gx = gy - exp(y) * sum(gy) per row (lib/THCUNN/LogSoftMax.cu:298-344).
__global__ void __launch_bounds__(256)
logsoftmax_bwd_kernel(const float *__restrict__ y, const float *__restrict__ gy, float *__restrict__ gx, int D)
{
    __shared__ float sh[8];
    const size_t off = (size_t)blockIdx.x * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += gy[off + i];
    s = block_reduce(s, sh, false);
    for (int i = threadIdx.x; i < D; i += blockDim.x) gx[off + i] = gy[off + i] - expf(y[off + i]) * s;
}

// loss = -sum_b w[t_b] lp[b][t_b] (/ sum w when size_average); targets carry CUNN_B200_INDEX_BASE
// (lib/THCUNN/ClassNLLCriterion.cu:38-84).  One CTA; out[0] = loss, out[1] = total weight.
__global__ void __launch_bounds__(256)
classnll_fwd_kernel(const float *__restrict__ lp, const long long *__restrict__ target, const float *__restrict__ weights,
                    float *__restrict__ out, int B, int D, int size_average, long long ignore_index)
{
    __shared__ float sh[8];
    float s = 0.f, tw = 0.f;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const long long t = target[b] - CUNN_B200_INDEX_BASE;
        if (t == ignore_index - CUNN_B200_INDEX_BASE || t < 0 || t >= D) continue;
        const float w = weights ? weights[t] : 1.f;
        s -= w * lp[(size_t)b * D + t];
        tw += w;
    }
    s = block_reduce(s, sh, false);
    tw = block_reduce(tw, sh, false);
    if (threadIdx.x == 0) {
        out[0] = (size_average && tw > 0.f) ? s / tw : s;
        out[1] = tw;
    }
}

// Writes only the target entries of gx (the caller zeroes it, as nn.ClassNLLCriterion does)
// (lib/THCUNN/ClassNLLCriterion.cu:108-132).
__global__ void __launch_bounds__(256)
classnll_bwd_kernel(const long long *__restrict__ target, const float *__restrict__ weights,
                    const float *__restrict__ total_weight, float *__restrict__ gx, int B, int D, int size_average,
                    long long ignore_index)
{
    const float tw = *total_weight;
    if (tw <= 0.f) return;
    const float norm = size_average ? 1.f / tw : 1.f;
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < B; b += gridDim.x * blockDim.x) {
        const long long t = target[b] - CUNN_B200_INDEX_BASE;
        if (t == ignore_index - CUNN_B200_INDEX_BASE || t < 0 || t >= D) continue;
        gx[(size_t)b * D + t] = -(weights ? weights[t] : 1.f) * norm;
    }
}

// p -= lr * g  (nn.Module:updateParameters as DataParallelTable.lua:315-321 applies it)
__global__ void __launch_bounds__(256)
sgd_kernel(float *__restrict__ p, const float *__restrict__ g, long long n, float lr)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        p[i] = fmaf(-lr, g[i], p[i]);
}

}  // namespace sup
}  // namespace cunn

using namespace cunn;
using namespace cunn::sup;

extern "C" CUNN_API int cunn_b200_threshold_forward(const float *x, float *y, long long n, float threshold, float value,
                                                    cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(n >= 0, "negative element count");
    if (n == 0) return 0;
    CUNN_CHECK_ARG(x && y, "null tensor pointer");
    threshold_fwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, y, n, threshold, value);
    CUNN_LAUNCH_CHECK("threshold forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_threshold_backward(const float *x, const float *gy, float *gx, long long n,
                                                     float threshold, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(n >= 0, "negative element count");
    if (n == 0) return 0;
    CUNN_CHECK_ARG(x && gy && gx, "null tensor pointer");
    threshold_bwd_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, gy, gx, n, threshold);
    CUNN_LAUNCH_CHECK("threshold backward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_avgpool_forward(const float *x, float *y, int N, int C, int H, int W, int oH, int oW,
                                                  int kH, int kW, int dH, int dW, int padH, int padW,
                                                  int count_include_pad, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0 && oH > 0 && oW > 0 && N >= 0 && C > 0 && H > 0 && W > 0,
                   "bad average-pooling sizes");
    CUNN_CHECK_ARG(kW / 2 >= padW && kH / 2 >= padH, "pad should be smaller than half of kernel size, but got padW = %d, padH = %d, kW = %d, kH = %d", padW, padH, kW, kH);
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && y, "null tensor pointer");
    const long long total = (long long)N * C * oH * oW;
    avgpool_fwd_kernel<<<grid_for(total, 1), 256, 0, (cudaStream_t)stream>>>(x, y, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                                                            count_include_pad, total);
    CUNN_LAUNCH_CHECK("average pooling forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_avgpool_backward(const float *gy, float *gx, int N, int C, int H, int W, int oH, int oW,
                                                   int kH, int kW, int dH, int dW, int padH, int padW,
                                                   int count_include_pad, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0 && oH > 0 && oW > 0 && N >= 0 && C > 0 && H > 0 && W > 0,
                   "bad average-pooling sizes");
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && gx, "null tensor pointer");
    const long long total = (long long)N * C * H * W;
    avgpool_bwd_kernel<<<grid_for(total, 1), 256, 0, (cudaStream_t)stream>>>(gy, gx, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                                                            count_include_pad, total);
    CUNN_LAUNCH_CHECK("average pooling backward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_logsoftmax_forward(const float *x, float *y, int B, int D, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(B >= 0 && D > 0, "bad log-softmax sizes");
    if (B == 0) return 0;
    CUNN_CHECK_ARG(x && y, "null tensor pointer");
    logsoftmax_fwd_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(x, y, D);
    CUNN_LAUNCH_CHECK("log-softmax forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_logsoftmax_backward(const float *y, const float *gy, float *gx, int B, int D,
                                                      cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(B >= 0 && D > 0, "bad log-softmax sizes");
    if (B == 0) return 0;
    CUNN_CHECK_ARG(y && gy && gx, "null tensor pointer");
    logsoftmax_bwd_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(y, gy, gx, D);
    CUNN_LAUNCH_CHECK("log-softmax backward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_classnll_forward(const float *logprob, const int64_t *target, const float *weights,
                                                   float *loss_and_total_weight, int B, int D, int size_average,
                                                   long long ignore_index, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(B >= 0 && D > 0, "bad criterion sizes");
    CUNN_CHECK_ARG(logprob && target && loss_and_total_weight, "null tensor pointer");
    classnll_fwd_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(logprob, (const long long *)target, weights,
                                                            loss_and_total_weight, B, D, size_average, ignore_index);
    CUNN_LAUNCH_CHECK("class NLL forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_classnll_backward(const int64_t *target, const float *weights, const float *total_weight,
                                                    float *gx, int B, int D, int size_average, long long ignore_index,
                                                    cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(B >= 0 && D > 0, "bad criterion sizes");
    if (B == 0) return 0;
    CUNN_CHECK_ARG(target && total_weight && gx, "null tensor pointer");
    classnll_bwd_kernel<<<ceil_div(B, 256), 256, 0, (cudaStream_t)stream>>>((const long long *)target, weights, total_weight,
                                                                           gx, B, D, size_average, ignore_index);
    CUNN_LAUNCH_CHECK("class NLL backward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_sgd_update(float *params, const float *grads, long long n, float lr, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(n >= 0, "negative element count");
    if (n == 0) return 0;
    CUNN_CHECK_ARG(params && grads, "null tensor pointer");
    sgd_kernel<<<grid_for(n, 1), 256, 0, (cudaStream_t)stream>>>(params, grads, n, lr);
    CUNN_LAUNCH_CHECK("sgd update");
    return 0;
}

namespace cunn {
namespace sup {
__global__ void __launch_bounds__(256)
fill_kernel(float *__restrict__ p, long long n, float v)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) p[i] = v;
}
}  // namespace sup
}  // namespace cunn

extern "C" CUNN_API int cunn_b200_fill(float *p, long long n, float value, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(n >= 0, "negative element count");
    if (n == 0) return 0;
    CUNN_CHECK_ARG(p, "null tensor pointer");
    cunn::sup::fill_kernel<<<cunn::sup::grid_for(n, 1), 256, 0, (cudaStream_t)stream>>>(p, n, value);
    CUNN_LAUNCH_CHECK("fill");
    return 0;
}
