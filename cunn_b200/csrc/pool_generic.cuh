// Shape-generic max pooling with argmax, any element type: the correctness path for every kernel size, stride,
// padding and dilation (the 3x3 / stride 2 / pad 1 fp32 case has dedicated kernels in maxpool.cu).
#pragma once

#include "common.cuh"

#include <float.h>

namespace cunn {
namespace pool {

template <typename T> __device__ __forceinline__ T lowest_finite();
template <> __device__ __forceinline__ float lowest_finite<float>() { return -FLT_MAX; }
template <> __device__ __forceinline__ double lowest_finite<double>() { return -DBL_MAX; }

// One thread per output.  The window is visited tap by tap, rows then columns ascending, and a value replaces
// the running maximum only when strictly greater: the visiting order and the compare of the reference kernel
// (lib/THCUNN/SpatialDilatedMaxPooling.cu:28-38), which the stored index depends on.  The scan starts from the
// lowest finite value with index -1, so NaN and -inf never win; the stored index is h*W + w plus the index base.
template <typename T>
__global__ void __launch_bounds__(256)
forward_taps_kernel(const T *__restrict__ x, T *__restrict__ y, long long *__restrict__ ind, int H, int W, int oH, int oW,
                    int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int pw = (int)(idx % oW);
        const long long t = idx / oW;
        const int ph = (int)(t % oH);
        const T *xp = x + (t / oH) * (long long)H * W;
        T best = lowest_finite<T>();
        int bi = -1;
        for (int kh = 0; kh < kH; ++kh) {
            const int h = ph * dH - padH + kh * dilH;
            if (h < 0 || h >= H) continue;
            for (int kw = 0; kw < kW; ++kw) {
                const int w = pw * dW - padW + kw * dilW;
                if (w < 0 || w >= W) continue;
                const T v = __ldg(xp + h * W + w);
                if (v > best) { best = v; bi = h * W + w; }
            }
        }
        y[idx] = best;
        ind[idx] = (long long)bi + CUNN_B200_INDEX_BASE;
    }
}

// One thread per input pixel, gather form (no atomics): the pixel adds the gradients of the windows whose stored
// index names it.  A tap (kh, kw) of the pixel belongs to the window at ((h + padH - kh dilH) / dH, ...); taps are
// taken from the last to the first so that the windows come in ascending (row, column) order, the order in which
// the reference adds them (lib/THCUNN/SpatialDilatedMaxPooling.cu:69-78).
template <typename T>
__global__ void __launch_bounds__(256)
backward_taps_kernel(const T *__restrict__ gy, const long long *__restrict__ ind, T *__restrict__ gx, int H, int W, int oH,
                     int oW, int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(idx % W);
        const long long t = idx / W;
        const int h = (int)(t % H);
        const long long plane = t / H;
        const T *gp = gy + plane * (long long)oH * oW;
        const long long *ip = ind + plane * (long long)oH * oW;
        const long long me = (long long)h * W + w + CUNN_B200_INDEX_BASE;
        T g = (T)0;
        for (int kh = kH - 1; kh >= 0; --kh) {
            const int a = h + padH - kh * dilH;
            if (a < 0 || a % dH || a / dH >= oH) continue;
            for (int kw = kW - 1; kw >= 0; --kw) {
                const int b = w + padW - kw * dilW;
                if (b < 0 || b % dW || b / dW >= oW) continue;
                const int o = (a / dH) * oW + b / dW;
                if (__ldg(ip + o) == me) g += __ldg(gp + o);
            }
        }
        gx[idx] = g;
    }
}

}  // namespace pool
}  // namespace cunn
