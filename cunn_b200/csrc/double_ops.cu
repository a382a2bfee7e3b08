// fp64 instantiations of the hot path: the kernels behind the THNN_CudaDouble* entry points
// (the reference instantiates every operator for float and double, e.g.
// lib/THCUNN/SpatialDepthWiseConvolution.cu:9 via THCGenerateFloatTypes.h, and its binding installs the
// CudaDouble table unconditionally, THCUNN.lua:131-132).
//
// Double tensors are the reference-checking path of a Lua-Torch user (its tests loop over both types,
// test.lua:12-15), not the throughput path, and sm_100a has no tcgen05 form for fp64 (the tensor
// cores' fp64 instruction is the legacy DMMA).  So these are plain CUDA-core kernels, written for
// correctness and full-machine occupancy rather than tuned tiles:
//   * depthwise convolution, pooling, batch norm: one pass each way, HBM-bound like their fp32 twins
//     (8 bytes per element); accumulation in fp64;
//   * SpatialConvolutionMM: implicit GEMM on the fp64 FMA pipes (64x64x16 tiles staged in shared
//     memory, operands gathered on the fly, no column buffer).  Its roofline is the fp64 FMA rate,
//     not the tensor pipe.
// Semantics (accumulate-with-scale, saved inverse std, unbiased running variance, first-maximum
// pooling indices from the lowest finite value) are those of the fp32 entry points; accreal is
// double (THCUNN.lua:54), so `scale` is a double here.
#include "common.cuh"
#include "pool_generic.cuh"

#include <float.h>
#include <algorithm>

namespace cunn {
namespace dbl {

static int grid_for(long long items)
{
    const long long want = ceil_div_ll(items, 256);
    const long long cap = (long long)sm_count() * 16;
    return (int)std::max(1LL, std::min(want, cap));
}

__device__ __forceinline__ double block_sum_d(double v, double *sh)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double r = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r += sh[i];
    return r;
}

// ---------------------------------------------------------------------------------------------------------
// Depthwise convolution (any kernel, stride, padding, multiplier)
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dw_forward_kernel(const double *__restrict__ x, const double *__restrict__ w, const double *__restrict__ bias,
                  double *__restrict__ y, int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                  int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(idx % oW);
        long long t = idx / oW;
        const int oh = (int)(t % oH); t /= oH;
        const int j = (int)(t % M); t /= M;
        const int c = (int)(t % C);
        const long long n = t / C;
        const double *xp = x + (n * C + c) * (long long)H * W;
        const double *wp = w + ((long long)j * C + c) * kH * kW;
        double s = bias ? bias[(long long)j * C + c] : 0.0;
        for (int kh = 0; kh < kH; ++kh) {
            const int ih = oh * dH - padH + kh;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < kW; ++kw) {
                const int iw = ow * dW - padW + kw;
                if (iw >= 0 && iw < W) s = fma(wp[kh * kW + kw], xp[ih * W + iw], s);
            }
        }
        y[idx] = s;
    }
}

__global__ void __launch_bounds__(256)
dw_grad_input_kernel(const double *__restrict__ gy, const double *__restrict__ w, double *__restrict__ gx, int C, int H, int W,
                     int M, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int wi = (int)(idx % W);
        long long t = idx / W;
        const int h = (int)(t % H); t /= H;
        const int c = (int)(t % C);
        const long long n = t / C;
        double s = 0.0;
        for (int j = 0; j < M; ++j) {
            const double *wp = w + ((long long)j * C + c) * kH * kW;
            const double *gp = gy + ((n * C + c) * M + j) * (long long)oH * oW;
            for (int kh = 0; kh < kH; ++kh) {
                const int a = h + padH - kh;
                if (a < 0 || a % dH || a / dH >= oH) continue;
                for (int kw = 0; kw < kW; ++kw) {
                    const int b = wi + padW - kw;
                    if (b < 0 || b % dW || b / dW >= oW) continue;
                    s = fma(wp[kh * kW + kw], gp[(a / dH) * oW + b / dW], s);
                }
            }
        }
        gx[idx] = s;
    }
}

// One CTA per (filter, channel, tap); tap == kH*kW is the bias sum.
__global__ void __launch_bounds__(256)
dw_acc_grad_kernel(const double *__restrict__ x, const double *__restrict__ gy, double *__restrict__ gw, double *__restrict__ gb,
                   int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW,
                   double scale)
{
    __shared__ double sh[8];
    const int kk = kH * kW, tap = blockIdx.x % (kk + 1), jc = blockIdx.x / (kk + 1), j = jc / C, c = jc % C;
    if (tap == kk && gb == nullptr) return;
    const int kh = tap / kW, kw = tap % kW, ohw = oH * oW;
    double acc = 0.0;
    for (int n = 0; n < N; ++n) {
        const double *xp = x + ((long long)n * C + c) * H * W;
        const double *gp = gy + (((long long)n * C + c) * M + j) * ohw;
        for (int i = threadIdx.x; i < ohw; i += blockDim.x) {
            if (tap == kk) {
                acc += gp[i];
            } else {
                const int ih = (i / oW) * dH - padH + kh, iw = (i % oW) * dW - padW + kw;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) acc = fma(gp[i], xp[ih * W + iw], acc);
            }
        }
    }
    acc = block_sum_d(acc, sh);
    if (threadIdx.x == 0) {
        if (tap == kk) gb[(long long)j * C + c] += scale * acc;
        else gw[((long long)j * C + c) * kk + tap] += scale * acc;
    }
}

// ---------------------------------------------------------------------------------------------------------
// SpatialConvolutionMM: implicit GEMM, C[m, n] = sum_k A(m, k) B(k, n), operands fetched by functors
// ---------------------------------------------------------------------------------------------------------
struct ConvGeom {
    int N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW, oH, oW;
};

// forward, image z: A = weight [K, C*kH*kW], B(r, p) = unfolded input, out y[z, m, p] = acc + bias[m]
struct FwdProblem {
    ConvGeom g;
    const double *x, *w, *bias;
    double *y;
    __device__ int M() const { return g.K; }
    __device__ int Ncols() const { return g.oH * g.oW; }
    __device__ int Kd() const { return g.C * g.kH * g.kW; }
    __device__ double a(int z, int m, int k) const { return w[(long long)m * Kd() + k]; }
    __device__ double b(int z, int k, int p) const
    {
        const int kw = k % g.kW, kh = (k / g.kW) % g.kH, c = k / (g.kW * g.kH);
        const int ih = (p / g.oW) * g.dH - g.padH + kh * g.dilH, iw = (p % g.oW) * g.dW - g.padW + kw * g.dilW;
        if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) return 0.0;
        return x[(((long long)z * g.C + c) * g.H + ih) * g.W + iw];
    }
    __device__ void store(int z, int m, int p, double v) const
    {
        y[((long long)z * g.K + m) * Ncols() + p] = v + (bias ? bias[m] : 0.0);
    }
};

// input gradient, image z: rows = input channels, columns = input pixels, reduction over (k, kh, kw)
struct DgradProblem {
    ConvGeom g;
    const double *gy, *w;
    double *gx;
    __device__ int M() const { return g.C; }
    __device__ int Ncols() const { return g.H * g.W; }
    __device__ int Kd() const { return g.K * g.kH * g.kW; }
    __device__ double a(int z, int c, int r) const
    {
        const int kk = g.kH * g.kW, k = r / kk, t = r % kk;
        return w[((long long)k * g.C + c) * kk + t];
    }
    __device__ double b(int z, int r, int q) const
    {
        const int kw = r % g.kW, kh = (r / g.kW) % g.kH, k = r / (g.kW * g.kH);
        const int a_ = q / g.W + g.padH - kh * g.dilH, b_ = q % g.W + g.padW - kw * g.dilW;
        if (a_ < 0 || b_ < 0 || a_ % g.dH || b_ % g.dW) return 0.0;
        const int oh = a_ / g.dH, ow = b_ / g.dW;
        if (oh >= g.oH || ow >= g.oW) return 0.0;
        return gy[(((long long)z * g.K + k) * g.oH + oh) * g.oW + ow];
    }
    __device__ void store(int z, int c, int q, double v) const { gx[((long long)z * g.C + c) * Ncols() + q] = v; }
};

// weight gradient (one "image" z = 0): rows = filters, columns = (c, kh, kw), reduction over (n, pixel)
struct WgradProblem {
    ConvGeom g;
    const double *x, *gy;
    double *gw;
    double scale;
    __device__ int M() const { return g.K; }
    __device__ int Ncols() const { return g.C * g.kH * g.kW; }
    __device__ int Kd() const { return g.N * g.oH * g.oW; }
    __device__ double a(int, int k, int t) const
    {
        const int ohw = g.oH * g.oW, n = t / ohw, p = t % ohw;
        return gy[((long long)n * g.K + k) * ohw + p];
    }
    __device__ double b(int, int t, int r) const
    {
        const int ohw = g.oH * g.oW, n = t / ohw, p = t % ohw;
        const int kw = r % g.kW, kh = (r / g.kW) % g.kH, c = r / (g.kW * g.kH);
        const int ih = (p / g.oW) * g.dH - g.padH + kh * g.dilH, iw = (p % g.oW) * g.dW - g.padW + kw * g.dilW;
        if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) return 0.0;
        return x[(((long long)n * g.C + c) * g.H + ih) * g.W + iw];
    }
    __device__ void store(int, int k, int r, double v) const { gw[(long long)k * Ncols() + r] += scale * v; }
};

constexpr int TM = 64, TN = 64, TK = 16;

template <class Problem>
__global__ void __launch_bounds__(256)
gemm_kernel(const Problem p)
{
    __shared__ double As[TK][TM + 1];
    __shared__ double Bs[TK][TN + 1];
    const int z = blockIdx.z, m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int M = p.M(), Nc = p.Ncols(), Kd = p.Kd();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // 4 x 4 outputs per thread: rows ty*4.., columns tx*4..
    double acc[4][4] = {};
    for (int k0 = 0; k0 < Kd; k0 += TK) {
        for (int e = threadIdx.x; e < TK * TM; e += 256) {
            const int kk = e / TM, mm = e % TM;
            As[kk][mm] = (m0 + mm < M && k0 + kk < Kd) ? p.a(z, m0 + mm, k0 + kk) : 0.0;
        }
        for (int e = threadIdx.x; e < TK * TN; e += 256) {
            const int kk = e / TN, nn = e % TN;
            Bs[kk][nn] = (n0 + nn < Nc && k0 + kk < Kd) ? p.b(z, k0 + kk, n0 + nn) : 0.0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            double av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < Nc) p.store(z, m, n, acc[i][j]);
        }
}

// gb[k] += scale * sum over images and pixels of gy[n, k, :]
__global__ void __launch_bounds__(256)
bias_grad_kernel(const double *__restrict__ gy, double *__restrict__ gb, int N, int K, int ohw, double scale)
{
    __shared__ double sh[8];
    const int k = blockIdx.x;
    double acc = 0.0;
    for (int n = 0; n < N; ++n) {
        const double *gp = gy + ((long long)n * K + k) * ohw;
        for (int i = threadIdx.x; i < ohw; i += blockDim.x) acc += gp[i];
    }
    acc = block_sum_d(acc, sh);
    if (threadIdx.x == 0) gb[k] += scale * acc;
}

static int conv_check(ConvGeom &g)
{
    CUNN_CHECK_ARG(g.kW > 0 && g.kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", g.kH, g.kW);
    CUNN_CHECK_ARG(g.dW > 0 && g.dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", g.dH, g.dW);
    CUNN_CHECK_ARG(g.N >= 0 && g.C > 0 && g.K > 0 && g.H > 0 && g.W > 0 && g.padH >= 0 && g.padW >= 0, "bad convolution sizes");
    const int spanH = g.dilH * (g.kH - 1) + 1, spanW = g.dilW * (g.kW - 1) + 1;
    g.oH = (g.H + 2 * g.padH - spanH) / g.dH + 1;
    g.oW = (g.W + 2 * g.padW - spanW) / g.dW + 1;
    CUNN_CHECK_ARG(g.H + 2 * g.padH >= spanH && g.W + 2 * g.padW >= spanW && g.oH >= 1 && g.oW >= 1,
                   "Given input size: (%d x %d x %d). Calculated output size: (%d x %d x %d). Output size is too small", g.C,
                   g.H, g.W, g.K, g.oH, g.oW);
    CUNN_CHECK_ARG((long long)g.N * g.C * (long long)g.H * g.W < (1LL << 31) && (long long)g.N * g.K * (long long)g.oH * g.oW < (1LL << 31),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

// ---------------------------------------------------------------------------------------------------------
// Batch normalisation over [N, C, S]
// ---------------------------------------------------------------------------------------------------------
static int bn_chunks(int N, int C) { return std::max(1, std::min(N, ceil_div(sm_count() * 4, C))); }

// grid (chunks, C): sums of (x - K) and (x - K)^2 over the chunk's images, K = the channel's first element
__global__ void __launch_bounds__(256)
bn_stats_kernel(const double *__restrict__ x, double2 *__restrict__ part, int N, int C, int S, int chunks)
{
    __shared__ double sh[8];
    const int j = blockIdx.x, c = blockIdx.y;
    const int per = N / chunks, extra = N % chunks, n0 = j * per + min(j, extra), n1 = n0 + per + (j < extra ? 1 : 0);
    const double K = x[(long long)c * S];
    double s1 = 0.0, s2 = 0.0;
    for (int n = n0; n < n1; ++n) {
        const double *xp = x + ((long long)n * C + c) * S;
        for (int i = threadIdx.x; i < S; i += blockDim.x) {
            const double d = xp[i] - K;
            s1 += d;
            s2 = fma(d, d, s2);
        }
    }
    s1 = block_sum_d(s1, sh);
    s2 = block_sum_d(s2, sh);
    if (threadIdx.x == 0) part[(long long)c * chunks + j] = make_double2(s1, s2);
}

// one thread per channel (lib/THCUNN/BatchNormalization.cu:185-200: inverse std of the biased variance, running
// variance from the unbiased one)
__global__ void bn_stats_finish_kernel(const double *__restrict__ x, const double2 *__restrict__ part, int N, int C, int S, int chunks,
                                       double *running_mean, double *running_var, double *save_mean, double *save_std,
                                       double momentum, double eps)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    double s1 = 0.0, s2 = 0.0;
    for (int j = 0; j < chunks; ++j) { s1 += part[(long long)c * chunks + j].x; s2 += part[(long long)c * chunks + j].y; }
    const double n = (double)N * S, K = x[(long long)c * S];
    const double mean = K + s1 / n;
    double m2 = s2 - s1 * s1 / n;
    if (m2 < 0.0) m2 = 0.0;
    double invstd = 0.0;
    if (m2 != 0.0 || eps != 0.0) invstd = 1.0 / sqrt(m2 / n + eps);
    save_mean[c] = mean;
    save_std[c] = invstd;
    running_mean[c] = (1.0 - momentum) * running_mean[c] + momentum * mean;
    running_var[c] = (1.0 - momentum) * running_var[c] + momentum * (m2 / (n - 1.0));
}

__global__ void __launch_bounds__(256)
bn_apply_kernel(const double *__restrict__ x, double *__restrict__ y, const double *__restrict__ weight, const double *__restrict__ bias,
                const double *__restrict__ mean_v, const double *__restrict__ std_or_var, int train, double eps, int C, int S,
                long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int c = (int)((idx / S) % C);
        const double invstd = train ? std_or_var[c] : 1.0 / sqrt(std_or_var[c] + eps);
        y[idx] = (weight ? weight[c] : 1.0) * (x[idx] - mean_v[c]) * invstd + (bias ? bias[c] : 0.0);
    }
}

// grid (chunks, C): sums of gy and gy * (x - mean)
__global__ void __launch_bounds__(256)
bn_grad_stats_kernel(const double *__restrict__ x, const double *__restrict__ gy, double2 *__restrict__ part, const double *__restrict__ mean_v,
                     int N, int C, int S, int chunks)
{
    __shared__ double sh[8];
    const int j = blockIdx.x, c = blockIdx.y;
    const int per = N / chunks, extra = N % chunks, n0 = j * per + min(j, extra), n1 = n0 + per + (j < extra ? 1 : 0);
    const double mean = mean_v[c];
    double s = 0.0, d = 0.0;
    for (int n = n0; n < n1; ++n) {
        const double *xp = x + ((long long)n * C + c) * S, *gp = gy + ((long long)n * C + c) * S;
        for (int i = threadIdx.x; i < S; i += blockDim.x) {
            s += gp[i];
            d = fma(gp[i], xp[i] - mean, d);
        }
    }
    s = block_sum_d(s, sh);
    d = block_sum_d(d, sh);
    if (threadIdx.x == 0) part[(long long)c * chunks + j] = make_double2(s, d);
}

struct BnCoef {
    double mean, proj, gmean, gscale;
};

// lib/THCUNN/BatchNormalization.cu:246-281
__global__ void bn_grad_finish_kernel(const double2 *__restrict__ part, int C, int chunks, double count, const double *weight,
                                      const double *mean_v, const double *std_or_var, int train, double eps, double scale,
                                      double *grad_weight, double *grad_bias, BnCoef *coef)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    double s = 0.0, d = 0.0;
    for (int j = 0; j < chunks; ++j) { s += part[(long long)c * chunks + j].x; d += part[(long long)c * chunks + j].y; }
    const double stdv = train ? std_or_var[c] : 1.0 / sqrt(std_or_var[c] + eps);
    const double w = weight ? weight[c] : 1.0;
    coef[c] = BnCoef{mean_v[c], d / count * stdv * stdv, s / count, stdv * w};
    if (grad_weight) grad_weight[c] += scale * d * stdv;
    if (grad_bias) grad_bias[c] += scale * s;
}

__global__ void __launch_bounds__(256)
bn_grad_apply_kernel(const double *__restrict__ x, const double *__restrict__ gy, double *__restrict__ gx, const BnCoef *__restrict__ coef,
                     int train, int C, int S, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const BnCoef k = coef[(idx / S) % C];
        gx[idx] = train ? (gy[idx] - (x[idx] - k.mean) * k.proj - k.gmean) * k.gscale : gy[idx] * k.gscale;
    }
}

}  // namespace dbl
}  // namespace cunn

using namespace cunn;
using namespace cunn::dbl;

// ---- depthwise ------------------------------------------------------------------------------------------------
static int dw_check(int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW, int *oH, int *oW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && H > 0 && W > 0 && M > 0 && padH >= 0 && padW >= 0, "bad depthwise sizes N=%d C=%d H=%d W=%d M=%d pad=%d,%d",
                   N, C, H, W, M, padH, padW);
    *oH = (H + 2 * padH - kH) / dH + 1;
    *oW = (W + 2 * padW - kW) / dW + 1;
    CUNN_CHECK_ARG(H + 2 * padH >= kH && W + 2 * padW >= kW && *oH >= 1 && *oW >= 1,
                   "Given input size: (%d x %d x %d). Calculated output size: (%d x %d x %d). Output size is too small", C, H, W,
                   C * M, *oH, *oW);
    CUNN_CHECK_ARG((long long)N * C * M * (long long)(*oH) * (*oW) < (1LL << 31) && (long long)N * C * (long long)H * W < (1LL << 31),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_dwconv_forward(const double *x, const double *weight, const double *bias, double *y, int N,
                                                        int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                                        cunn_stream_t stream)
{
    clear_error();
    int oH, oW;
    if (dw_check(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    const long long total = (long long)N * C * M * oH * oW;
    dw_forward_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(x, weight, bias, y, C, H, W, M, kH, kW, dH, dW, padH, padW, oH, oW, total);
    CUNN_LAUNCH_CHECK("dwconv forward (double)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_dwconv_grad_input(const double *gy, const double *weight, double *gx, int N, int C, int H, int W,
                                                           int M, int kH, int kW, int dH, int dW, int padH, int padW, cunn_stream_t stream)
{
    clear_error();
    int oH, oW;
    if (dw_check(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    const long long total = (long long)N * C * H * W;
    dw_grad_input_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(gy, weight, gx, C, H, W, M, kH, kW, dH, dW, padH, padW, oH, oW, total);
    CUNN_LAUNCH_CHECK("dwconv grad input (double)");
    return 0;
}

// The fp64 parameter-gradient kernels need no scratch; the workspace arguments exist so that the float and double
// entry points have the same shape.
extern "C" CUNN_API size_t cunn_b200_double_dwconv_acc_grad_workspace(int, int, int, int, int, int, int, int, int, int, int) { return 0; }
extern "C" CUNN_API size_t cunn_b200_double_convmm_acc_grad_workspace(int, int, int, int, int, int, int, int, int, int, int) { return 0; }

extern "C" CUNN_API int cunn_b200_double_dwconv_acc_grad(const double *x, const double *gy, double *grad_weight, double *grad_bias, int N,
                                                         int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                                         double scale, void *, size_t, cunn_stream_t stream)
{
    clear_error();
    int oH, oW;
    if (dw_check(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    dw_acc_grad_kernel<<<M * C * (kH * kW + 1), 256, 0, (cudaStream_t)stream>>>(x, gy, grad_weight, grad_bias, N, C, H, W, M, kH, kW, dH, dW,
                                                                               padH, padW, oH, oW, scale);
    CUNN_LAUNCH_CHECK("dwconv acc grad (double)");
    return 0;
}

// ---- SpatialConvolutionMM ------------------------------------------------------------------------------------------
extern "C" CUNN_API int cunn_b200_double_convmm_forward(const double *x, const double *weight, const double *bias, double *y, int N,
                                                        int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                                        cunn_stream_t stream)
{
    clear_error();
    ConvGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, 0, 0};
    if (conv_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    CUNN_CHECK_ARG(N <= 65535, "batches of more than 65535 images are not supported for double tensors");
    FwdProblem p{g, x, weight, bias, y};
    gemm_kernel<<<dim3(ceil_div(g.oH * g.oW, TN), ceil_div(K, TM), N), 256, 0, (cudaStream_t)stream>>>(p);
    CUNN_LAUNCH_CHECK("convmm forward (double)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_convmm_grad_input(const double *gy, const double *weight, double *gx, int N, int C, int H, int W,
                                                           int K, int kH, int kW, int dH, int dW, int padH, int padW, cunn_stream_t stream)
{
    clear_error();
    ConvGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, 0, 0};
    if (conv_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    CUNN_CHECK_ARG(N <= 65535, "batches of more than 65535 images are not supported for double tensors");
    DgradProblem p{g, gy, weight, gx};
    gemm_kernel<<<dim3(ceil_div(H * W, TN), ceil_div(C, TM), N), 256, 0, (cudaStream_t)stream>>>(p);
    CUNN_LAUNCH_CHECK("convmm grad input (double)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_convmm_acc_grad(const double *x, const double *gy, double *grad_weight, double *grad_bias, int N,
                                                         int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                                         double scale, void *, size_t, cunn_stream_t stream)
{
    clear_error();
    ConvGeom g{N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, 0, 0};
    if (conv_check(g)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    CUNN_CHECK_ARG((long long)N * g.oH * g.oW < (1LL << 31), "reduction length too large");
    WgradProblem p{g, x, gy, grad_weight, scale};
    gemm_kernel<<<dim3(ceil_div(C * kH * kW, TN), ceil_div(K, TM), 1), 256, 0, (cudaStream_t)stream>>>(p);
    CUNN_LAUNCH_CHECK("convmm acc grad (double)");
    if (grad_bias) {
        bias_grad_kernel<<<K, 256, 0, (cudaStream_t)stream>>>(gy, grad_bias, N, K, g.oH * g.oW, scale);
        CUNN_LAUNCH_CHECK("convmm bias grad (double)");
    }
    return 0;
}

// ---- batch normalisation -----------------------------------------------------------------------------------------
// Workspace: [per-(channel, chunk) partials][per-channel gradient coefficients]; no state between calls.
extern "C" CUNN_API size_t cunn_b200_double_batchnorm_workspace(int N, int C)
{
    if (N <= 0 || C <= 0) return 0;
    return (size_t)C * bn_chunks(N, C) * sizeof(double2) + (size_t)C * sizeof(BnCoef) + 256;
}

extern "C" CUNN_API int cunn_b200_double_batchnorm_forward(const double *x, double *y, const double *weight, const double *bias,
                                                           double *running_mean, double *running_var, double *save_mean, double *save_std,
                                                           int N, int C, int S, int train, double momentum, double eps, void *workspace,
                                                           size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    CUNN_CHECK_ARG(N >= 0 && C > 0 && S > 0, "bad batch-norm sizes N=%d C=%d S=%d", N, C, S);
    CUNN_CHECK_ARG((long long)N * C * (long long)S < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && y && running_mean && running_var, "null tensor pointer");
    const long long total = (long long)N * C * S;
    if (train) {
        CUNN_CHECK_ARG(save_mean && save_std, "training-mode batch norm needs save_mean and save_std");
        const int chunks = bn_chunks(N, C);
        CUNN_CHECK_ARG(workspace && workspace_bytes >= cunn_b200_double_batchnorm_workspace(N, C) && ((uintptr_t)workspace & 15) == 0,
                       "batch norm (double) needs %zu bytes of 16-byte aligned workspace, got %zu",
                       cunn_b200_double_batchnorm_workspace(N, C), workspace ? workspace_bytes : (size_t)0);
        double2 *part = (double2 *)workspace;
        bn_stats_kernel<<<dim3(chunks, C), 256, 0, stream>>>(x, part, N, C, S, chunks);
        bn_stats_finish_kernel<<<ceil_div(C, 128), 128, 0, stream>>>(x, part, N, C, S, chunks, running_mean, running_var, save_mean, save_std,
                                                                     momentum, eps);
        bn_apply_kernel<<<grid_for(total), 256, 0, stream>>>(x, y, weight, bias, save_mean, save_std, 1, eps, C, S, total);
    } else {
        bn_apply_kernel<<<grid_for(total), 256, 0, stream>>>(x, y, weight, bias, running_mean, running_var, 0, eps, C, S, total);
    }
    CUNN_LAUNCH_CHECK("batch norm (double)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_batchnorm_backward(const double *x, const double *gy, double *gx, double *grad_weight,
                                                            double *grad_bias, const double *weight, const double *running_mean,
                                                            const double *running_var, const double *save_mean, const double *save_std,
                                                            int N, int C, int S, int train, double scale, double eps, void *workspace,
                                                            size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    CUNN_CHECK_ARG(N >= 0 && C > 0 && S > 0, "bad batch-norm sizes N=%d C=%d S=%d", N, C, S);
    CUNN_CHECK_ARG((long long)N * C * (long long)S < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy, "null tensor pointer");
    CUNN_CHECK_ARG(train ? (save_mean && save_std) : (running_mean && running_var), "batch norm backward needs %s",
                   train ? "save_mean and save_std" : "running_mean and running_var");
    CUNN_CHECK_ARG(workspace && workspace_bytes >= cunn_b200_double_batchnorm_workspace(N, C) && ((uintptr_t)workspace & 15) == 0,
                   "batch norm backward (double) needs %zu bytes of 16-byte aligned workspace, got %zu",
                   cunn_b200_double_batchnorm_workspace(N, C), workspace ? workspace_bytes : (size_t)0);
    const int chunks = bn_chunks(N, C);
    double2 *part = (double2 *)workspace;
    BnCoef *coef = (BnCoef *)((char *)workspace + (((size_t)C * chunks * sizeof(double2) + 255) & ~(size_t)255));
    const double *mean_v = train ? save_mean : running_mean, *sv = train ? save_std : running_var;
    const long long total = (long long)N * C * S;
    bn_grad_stats_kernel<<<dim3(chunks, C), 256, 0, stream>>>(x, gy, part, mean_v, N, C, S, chunks);
    bn_grad_finish_kernel<<<ceil_div(C, 128), 128, 0, stream>>>(part, C, chunks, (double)N * S, weight, mean_v, sv, train, eps, scale, grad_weight,
                                                                grad_bias, coef);
    if (gx) bn_grad_apply_kernel<<<grid_for(total), 256, 0, stream>>>(x, gy, gx, coef, train, C, S, total);
    CUNN_LAUNCH_CHECK("batch norm backward (double)");
    return 0;
}

// ---- max pooling -----------------------------------------------------------------------------------------------
static int pool_check(int N, int C, int H, int W, int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int ceil_mode,
                      int *oH, int *oW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(dilH > 0 && dilW > 0, "dilation should be greater than zero, but got dilationH: %d dilationW: %d", dilH, dilW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && H > 0 && W > 0 && padH >= 0 && padW >= 0, "bad pooling sizes N=%d C=%d H=%d W=%d", N, C, H, W);
    CUNN_CHECK_ARG(kW / 2 >= padW && kH / 2 >= padH, "pad should be smaller than half of kernel size, but got padW = %d, padH = %d, kW = %d, kH = %d",
                   padW, padH, kW, kH);
    *oH = cunn_b200_maxpool_out_size(H, kH, dH, padH, dilH, ceil_mode);
    *oW = cunn_b200_maxpool_out_size(W, kW, dW, padW, dilW, ceil_mode);
    CUNN_CHECK_ARG(*oH >= 1 && *oW >= 1, "Given input size: (%dx%dx%d). Calculated output size: (%dx%dx%d). Output size is too small", C, H, W,
                   C, *oH, *oW);
    CUNN_CHECK_ARG((long long)N * C * (long long)H * W < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_maxpool_forward(const double *x, double *y, int64_t *indices, int N, int C, int H, int W, int kH,
                                                         int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int ceil_mode,
                                                         cunn_stream_t stream)
{
    clear_error();
    int oH, oW;
    if (pool_check(N, C, H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, ceil_mode, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && y && indices, "null tensor pointer");
    const long long total = (long long)N * C * oH * oW;
    pool::forward_taps_kernel<double><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(x, y, (long long *)indices, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
                                                                          dilH, dilW, total);
    CUNN_LAUNCH_CHECK("maxpool forward (double)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_double_maxpool_backward(const double *gy, const int64_t *indices, double *gx, int N, int C, int H, int W,
                                                          int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW,
                                                          int ceil_mode, cunn_stream_t stream)
{
    clear_error();
    int oH, oW;
    if (pool_check(N, C, H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, ceil_mode, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && gx && indices, "null tensor pointer");
    const long long total = (long long)N * C * H * W;
    pool::backward_taps_kernel<double><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(gy, (const long long *)indices, gx, H, W, oH, oW, kH, kW, dH, dW,
                                                                           padH, padW, dilH, dilW, total);
    CUNN_LAUNCH_CHECK("maxpool backward (double)");
    return 0;
}
