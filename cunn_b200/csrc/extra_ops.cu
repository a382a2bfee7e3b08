// Operators beside the benchmarked path that the reference builds on the same unfold + GEMM or pooling loops:
// SpatialConvolutionLocal (lib/THCUNN/generic/SpatialConvolutionLocal.cu), SpatialAdaptiveMaxPooling and
// SpatialAdaptiveAveragePooling (lib/THCUNN/SpatialAdaptive{Max,Average}Pooling.cu).  fp32, NCHW.
//
// SpatialConvolutionLocal has one weight matrix per OUTPUT POSITION (weight [oH*oW, K, C*kH*kW], bias [K, oH, oW]), so
// every weight is used once per image: the operator is bound by reading the weights, not by arithmetic, and there is
// no reuse for a tensor-core tile to exploit.  The kernels therefore stream the weights once with coalesced loads
// (a warp walks the C*kH*kW values of one (position, filter) row) and keep the whole batch of that position in the
// inner loop, where the reference runs a batched GEMM with one 1-column matrix per position and image
// (THCTensor_(baddbmm), :149-156).  No unfolded copy of the input (the reference's finput) is made.
//
// Adaptive pooling: window bounds are computed in float arithmetic exactly as the reference kernels do, because the
// stored argmax offsets are relative to the window start.  The backward passes are gathers over the (few) windows
// that cover an input pixel, so they need no atomics and are deterministic, where the reference scatters with atomicAdd.
#include "common.cuh"

#include <float.h>
#include <algorithm>

namespace cunn {
namespace extra {

static int grid_for(long long items, int per_cta = 256)
{
    return (int)std::max(1LL, std::min(ceil_div_ll(items, per_cta), (long long)sm_count() * 16));
}

struct LocalGeom {
    int N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW;
};

// One warp per (position p, filter k): lanes stride over the row's C*kH*kW weights; up to NB images are carried per
// pass so that a weight is loaded once for all of them.
constexpr int NB = 8;

__global__ void __launch_bounds__(256)
local_forward_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y,
                     const LocalGeom g)
{
    const int P = g.oH * g.oW, R = g.C * g.kH * g.kW, kk = g.kH * g.kW;
    const int lane = threadIdx.x & 31;
    const long long rows = (long long)P * g.K;
    for (long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int p = (int)(row / g.K), k = (int)(row % g.K), oh = p / g.oW, ow = p % g.oW;
        const float *wp = w + row * R;
        for (int n0 = 0; n0 < g.N; n0 += NB) {
            float acc[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) acc[i] = 0.f;
            for (int r = lane; r < R; r += 32) {
                const int c = r / kk, t = r - c * kk, kh = t / g.kW, kw = t - kh * g.kW;
                const int ih = oh * g.dH - g.padH + kh, iw = ow * g.dW - g.padW + kw;
                if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) continue;
                const float wv = __ldg(wp + r);
                const float *xp = x + ((long long)c * g.H + ih) * g.W + iw;
#pragma unroll
                for (int i = 0; i < NB; ++i)
                    if (n0 + i < g.N) acc[i] = fmaf(wv, __ldg(xp + (long long)(n0 + i) * g.C * g.H * g.W), acc[i]);
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const float s = warp_sum(acc[i]);
                if (lane == 0 && n0 + i < g.N) y[((long long)(n0 + i) * g.K + k) * P + p] = s + (bias ? __ldg(bias + (long long)k * P + p) : 0.f);
            }
        }
    }
}

// One thread per input pixel (n, c, h, w): gathers over the positions whose window holds the pixel and over the filters.
__global__ void __launch_bounds__(256)
local_grad_input_kernel(const float *__restrict__ gy, const float *__restrict__ w, float *__restrict__ gx, const LocalGeom g, long long total)
{
    const int P = g.oH * g.oW, R = g.C * g.kH * g.kW;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int wi = (int)(idx % g.W);
        long long t = idx / g.W;
        const int h = (int)(t % g.H); t /= g.H;
        const int c = (int)(t % g.C);
        const long long n = t / g.C;
        float s = 0.f;
        for (int kh = 0; kh < g.kH; ++kh) {
            const int a = h + g.padH - kh;
            if (a < 0 || a % g.dH || a / g.dH >= g.oH) continue;
            for (int kw = 0; kw < g.kW; ++kw) {
                const int b = wi + g.padW - kw;
                if (b < 0 || b % g.dW || b / g.dW >= g.oW) continue;
                const int p = (a / g.dH) * g.oW + b / g.dW;
                const float *wp = w + (long long)p * g.K * R + (c * g.kH + kh) * g.kW + kw;
                const float *gp = gy + n * g.K * P + p;
                for (int k = 0; k < g.K; ++k) s = fmaf(__ldg(wp + (long long)k * R), __ldg(gp + (long long)k * P), s);
            }
        }
        gx[idx] = s;
    }
}

// One thread per weight (p, k, r): sums over the images; threads of a warp hold consecutive r, so the gradient row is
// read and written coalesced.  The bias gradient is one thread per (k, p).
__global__ void __launch_bounds__(256)
local_acc_grad_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ gw, const LocalGeom g, float scale, long long total)
{
    const int P = g.oH * g.oW, R = g.C * g.kH * g.kW, kk = g.kH * g.kW;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx % R);
        const long long row = idx / R;
        const int p = (int)(row / g.K), k = (int)(row % g.K), oh = p / g.oW, ow = p % g.oW;
        const int c = r / kk, t = r - c * kk, kh = t / g.kW, kw = t - kh * g.kW;
        const int ih = oh * g.dH - g.padH + kh, iw = ow * g.dW - g.padW + kw;
        if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) continue;          // the weight never meets a pixel: its gradient is zero
        const float *xp = x + ((long long)c * g.H + ih) * g.W + iw;
        const float *gp = gy + (long long)k * P + p;
        float s = 0.f;
        for (int n = 0; n < g.N; ++n) s = fmaf(__ldg(gp + (long long)n * g.K * P), __ldg(xp + (long long)n * g.C * g.H * g.W), s);
        gw[idx] = fmaf(scale, s, gw[idx]);
    }
}

__global__ void __launch_bounds__(256)
local_bias_grad_kernel(const float *__restrict__ gy, float *__restrict__ gb, int N, long long KP, float scale)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < KP; idx += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int n = 0; n < N; ++n) s += __ldg(gy + (long long)n * KP + idx);
        gb[idx] = fmaf(scale, s, gb[idx]);
    }
}

// ---- adaptive pooling -----------------------------------------------------------------------------------------------
// window bounds with every rounding pinned, so that host, oracle and device agree
__device__ __forceinline__ int amax_start(int i, int o, int n) { return (int)floorf(__fmul_rn(__fdiv_rn((float)i, (float)o), (float)n)); }
__device__ __forceinline__ int amax_end(int i, int o, int n) { return (int)ceilf(__fmul_rn(__fdiv_rn((float)(i + 1), (float)o), (float)n)); }
__device__ __forceinline__ int aavg_start(int i, int o, int n) { return (int)floorf(__fdiv_rn((float)(i * n), (float)o)); }
__device__ __forceinline__ int aavg_end(int i, int o, int n) { return (int)ceilf(__fdiv_rn((float)((i + 1) * n), (float)o)); }

// candidate outputs whose window can hold input coordinate h (a superset, each is then tested exactly)
__device__ __forceinline__ void window_candidates(int h, int o, int n, int *lo, int *hi)
{
    *lo = max(0, (int)(((long long)h * o) / n) - 1);
    *hi = min(o - 1, (int)(((long long)(h + 1) * o + n - 1) / n));
}

__global__ void __launch_bounds__(256)
adaptive_max_forward_kernel(const float *__restrict__ x, float *__restrict__ y, long long *__restrict__ ind, int H, int W, int oH, int oW,
                            long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int xx = (int)(idx % oW);
        const long long t = idx / oW;
        const int yy = (int)(t % oH);
        const float *xp = x + (t / oH) * (long long)H * W;
        const int y0 = amax_start(yy, oH, H), y1 = amax_end(yy, oH, H), x0 = amax_start(xx, oW, W), x1 = amax_end(xx, oW, W);
        float best = -FLT_MAX;
        int by = -1, bx = -1;
        for (int h = y0; h < y1; ++h)
            for (int w = x0; w < x1; ++w) {
                const float v = __ldg(xp + h * W + w);
                if (v > best) { best = v; by = h - y0; bx = w - x0; }
            }
        y[idx] = best;
        ind[idx] = (long long)by + CUNN_B200_INDEX_BASE;              // first plane: row offset inside the window
        ind[total + idx] = (long long)bx + CUNN_B200_INDEX_BASE;      // second plane: column offset
    }
}

__global__ void __launch_bounds__(256)
adaptive_max_backward_kernel(const float *__restrict__ gy, const long long *__restrict__ ind, float *__restrict__ gx, int H, int W, int oH,
                             int oW, long long total_in, long long total_out)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_in; idx += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(idx % W);
        const long long t = idx / W;
        const int h = (int)(t % H);
        const long long plane = t / H;
        int ylo, yhi, xlo, xhi;
        window_candidates(h, oH, H, &ylo, &yhi);
        window_candidates(w, oW, W, &xlo, &xhi);
        float g = 0.f;
        for (int yy = ylo; yy <= yhi; ++yy) {
            const int y0 = amax_start(yy, oH, H);
            for (int xx = xlo; xx <= xhi; ++xx) {
                const long long o = (plane * oH + yy) * oW + xx;
                if (y0 + (int)(__ldg(ind + o) - CUNN_B200_INDEX_BASE) == h &&
                    amax_start(xx, oW, W) + (int)(__ldg(ind + total_out + o) - CUNN_B200_INDEX_BASE) == w)
                    g += __ldg(gy + o);
            }
        }
        gx[idx] = g;
    }
}

__global__ void __launch_bounds__(256)
adaptive_avg_forward_kernel(const float *__restrict__ x, float *__restrict__ y, int H, int W, int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int xx = (int)(idx % oW);
        const long long t = idx / oW;
        const int yy = (int)(t % oH);
        const float *xp = x + (t / oH) * (long long)H * W;
        const int y0 = aavg_start(yy, oH, H), y1 = aavg_end(yy, oH, H), x0 = aavg_start(xx, oW, W), x1 = aavg_end(xx, oW, W);
        float s = 0.f;
        for (int h = y0; h < y1; ++h)
            for (int w = x0; w < x1; ++w) s += __ldg(xp + h * W + w);
        y[idx] = s / (float)(y1 - y0) / (float)(x1 - x0);
    }
}

__global__ void __launch_bounds__(256)
adaptive_avg_backward_kernel(const float *__restrict__ gy, float *__restrict__ gx, int H, int W, int oH, int oW, long long total_in)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_in; idx += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(idx % W);
        const long long t = idx / W;
        const int h = (int)(t % H);
        const long long plane = t / H;
        int ylo, yhi, xlo, xhi;
        window_candidates(h, oH, H, &ylo, &yhi);
        window_candidates(w, oW, W, &xlo, &xhi);
        float g = 0.f;
        for (int yy = ylo; yy <= yhi; ++yy) {
            const int y0 = aavg_start(yy, oH, H), y1 = aavg_end(yy, oH, H);
            if (h < y0 || h >= y1) continue;
            for (int xx = xlo; xx <= xhi; ++xx) {
                const int x0 = aavg_start(xx, oW, W), x1 = aavg_end(xx, oW, W);
                if (w < x0 || w >= x1) continue;
                g += __ldg(gy + (plane * oH + yy) * oW + xx) / (float)(x1 - x0) / (float)(y1 - y0);
            }
        }
        gx[idx] = g;
    }
}

static int local_check(LocalGeom &g)
{
    CUNN_CHECK_ARG(g.kW > 0 && g.kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", g.kH, g.kW);
    CUNN_CHECK_ARG(g.dW > 0 && g.dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", g.dH, g.dW);
    CUNN_CHECK_ARG(g.N >= 0 && g.C > 0 && g.K > 0 && g.H > 0 && g.W > 0 && g.oH > 0 && g.oW > 0 && g.padH >= 0 && g.padW >= 0,
                   "bad local-convolution sizes");
    CUNN_CHECK_ARG((g.H + 2 * g.padH - g.kH) / g.dH + 1 == g.oH && (g.W + 2 * g.padW - g.kW) / g.dW + 1 == g.oW && g.H + 2 * g.padH >= g.kH &&
                       g.W + 2 * g.padW >= g.kW,
                   "output size %d x %d does not follow from input %d x %d, kernel %d x %d, stride %d x %d, padding %d x %d", g.oH, g.oW, g.H,
                   g.W, g.kH, g.kW, g.dH, g.dW, g.padH, g.padW);
    CUNN_CHECK_ARG((long long)g.N * g.C * (long long)g.H * g.W < (1LL << 31) && (long long)g.N * g.K * (long long)g.oH * g.oW < (1LL << 31) &&
                       (long long)g.oH * g.oW * g.K * (long long)g.C * g.kH * g.kW < (1LL << 40),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

static int adaptive_check(int planes, int H, int W, int oH, int oW)
{
    CUNN_CHECK_ARG(planes >= 0 && H > 0 && W > 0 && oH > 0 && oW > 0, "bad adaptive-pooling sizes planes=%d H=%d W=%d oH=%d oW=%d", planes, H, W, oH, oW);
    CUNN_CHECK_ARG((long long)planes * H * W < (1LL << 31) && (long long)planes * oH * oW < (1LL << 31) && H < (1 << 15) && W < (1 << 15) &&
                       oH < (1 << 15) && oW < (1 << 15),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

}  // namespace extra
}  // namespace cunn

using namespace cunn;
using namespace cunn::extra;

extern "C" CUNN_API int cunn_b200_local_conv_forward(const float *x, const float *weight, const float *bias, float *y, int N, int C, int H,
                                                     int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW,
                                                     cunn_stream_t stream)
{
    clear_error();
    LocalGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW};
    if (local_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    local_forward_kernel<<<grid_for((long long)oH * oW * K, 8), 256, 0, (cudaStream_t)stream>>>(x, weight, bias, y, g);
    CUNN_LAUNCH_CHECK("local convolution forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_local_conv_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H, int W, int K,
                                                        int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW,
                                                        cunn_stream_t stream)
{
    clear_error();
    LocalGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW};
    if (local_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    const long long total = (long long)N * C * H * W;
    local_grad_input_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(gy, weight, gx, g, total);
    CUNN_LAUNCH_CHECK("local convolution grad input");
    return 0;
}

extern "C" CUNN_API int cunn_b200_local_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias, int N, int C,
                                                      int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, int oH,
                                                      int oW, float scale, cunn_stream_t stream)
{
    clear_error();
    LocalGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW};
    if (local_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    const long long total = (long long)oH * oW * K * C * kH * kW;
    local_acc_grad_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(x, gy, grad_weight, g, scale, total);
    CUNN_LAUNCH_CHECK("local convolution acc grad");
    if (grad_bias) {
        const long long KP = (long long)K * oH * oW;
        local_bias_grad_kernel<<<grid_for(KP), 256, 0, (cudaStream_t)stream>>>(gy, grad_bias, N, KP, scale);
        CUNN_LAUNCH_CHECK("local convolution bias grad");
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_adaptive_maxpool_forward(const float *x, float *y, int64_t *indices, int planes, int H, int W, int oH,
                                                           int oW, cunn_stream_t stream)
{
    clear_error();
    if (adaptive_check(planes, H, W, oH, oW)) return 1;
    if (planes == 0) return 0;
    CUNN_CHECK_ARG(x && y && indices, "null tensor pointer");
    const long long total = (long long)planes * oH * oW;
    adaptive_max_forward_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(x, y, (long long *)indices, H, W, oH, oW, total);
    CUNN_LAUNCH_CHECK("adaptive max pooling forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_adaptive_maxpool_backward(const float *gy, const int64_t *indices, float *gx, int planes, int H, int W,
                                                            int oH, int oW, cunn_stream_t stream)
{
    clear_error();
    if (adaptive_check(planes, H, W, oH, oW)) return 1;
    if (planes == 0) return 0;
    CUNN_CHECK_ARG(gy && gx && indices, "null tensor pointer");
    const long long tin = (long long)planes * H * W, tout = (long long)planes * oH * oW;
    adaptive_max_backward_kernel<<<grid_for(tin), 256, 0, (cudaStream_t)stream>>>(gy, (const long long *)indices, gx, H, W, oH, oW, tin, tout);
    CUNN_LAUNCH_CHECK("adaptive max pooling backward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_adaptive_avgpool_forward(const float *x, float *y, int planes, int H, int W, int oH, int oW,
                                                           cunn_stream_t stream)
{
    clear_error();
    if (adaptive_check(planes, H, W, oH, oW)) return 1;
    if (planes == 0) return 0;
    CUNN_CHECK_ARG(x && y, "null tensor pointer");
    const long long total = (long long)planes * oH * oW;
    adaptive_avg_forward_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(x, y, H, W, oH, oW, total);
    CUNN_LAUNCH_CHECK("adaptive average pooling forward");
    return 0;
}

extern "C" CUNN_API int cunn_b200_adaptive_avgpool_backward(const float *gy, float *gx, int planes, int H, int W, int oH, int oW,
                                                            cunn_stream_t stream)
{
    clear_error();
    if (adaptive_check(planes, H, W, oH, oW)) return 1;
    if (planes == 0) return 0;
    CUNN_CHECK_ARG(gy && gx, "null tensor pointer");
    const long long tin = (long long)planes * H * W;
    adaptive_avg_backward_kernel<<<grid_for(tin), 256, 0, (cudaStream_t)stream>>>(gy, gx, H, W, oH, oW, tin);
    CUNN_LAUNCH_CHECK("adaptive average pooling backward");
    return 0;
}
