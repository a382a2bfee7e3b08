/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the math of the THCUNN convolutional hot path: depthwise
 * convolution, im2col+GEMM convolution, batch normalisation, max pooling and
 * the four small ops a MobileNetV1 training step needs around them.  It exists
 * only so that tests, the smoke check and the CPU-baseline leg of the
 * benchmark have something to compare the CUDA kernels with.  Nothing in the
 * shipped library links, loads or calls it.
 *
 * The file is compiled three times (see the Makefile next to it):
 *   -DREF_ACC=double -DREF_PREFIX=ref64_   the oracle proper: fp32 tensors,
 *                                          every sum carried in fp64;
 *   -DREF_REAL=double -DREF_ACC=double -DREF_PREFIX=refd_   the oracle of the
 *                                          CudaDouble entry points: fp64 tensors;
 *   -DREF_ACC=float  -DREF_PREFIX=ref32_   the timed CPU baseline: the same
 *                                          loops with fp32 accumulators, which
 *                                          is the arithmetic torch/nn's CPU
 *                                          THNN uses for float tensors.
 *
 * PARITY STATUS: the reference ships no golden vectors and its CPU comparison
 * library (torch/nn THNN) is absent from the reference tree.  This restatement
 * is pinned against (a) the reference's OWN device kernels, compiled unchanged
 * from the reference tree (oracle/_ref, see ref_kernels_*.cu): max and average
 * pooling run on the host and must agree bit for bit (values, int64 indices);
 * batch normalisation and the unfold + SGEMM convolution schedules ran on a
 * B200 and their outputs are committed as tests/golden/refk_*.npz; (b) the
 * reference's in-tree self-consistency tests (depthwise == per-channel
 * SpatialConvolution, average-pool known answers); (c) fixtures produced by
 * PyTorch's CPU operators, a descendant of the same THNN code.  Against
 * torch/nn's CPU library itself: unpinned (absent).
 *
 * Each function cites the reference file:line whose arithmetic it follows
 * (paths relative to the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <float.h>
#include <string.h>
#include <stdlib.h>

#ifndef REF_ACC
#define REF_ACC double
#endif
#ifndef REF_PREFIX
#define REF_PREFIX ref64_
#endif
#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)
#define FN(name) CAT(REF_PREFIX, name)

typedef REF_ACC acc_t;

/* Element type of every tensor: float for the Cuda (float) entry points, double for the CudaDouble ones. */
#ifndef REF_REAL
#define REF_REAL float
#endif
typedef REF_REAL real_t;
#define REAL_IS_DOUBLE (sizeof(real_t) == 8)
/* lowest finite value of the element type: the start value of the max-pooling scan
 * (THCNumerics<AccType>::min(), lib/THCUNN/SpatialDilatedMaxPooling.cu:28) */
#define REAL_LOWEST ((real_t)(REAL_IS_DOUBLE ? -DBL_MAX : -FLT_MAX))

/* Index base of stored pooling indices and class targets.  libTH defines
 * TH_INDEX_BASE as 1 for the Lua build the reference's tests run under
 * (lib/THCUNN/SpatialDilatedMaxPooling.cu:40 adds it to every stored index). */
#ifndef REF_INDEX_BASE
#define REF_INDEX_BASE 1
#endif

int FN(index_base)(void) { return REF_INDEX_BASE; }

/* Number of OpenMP threads the routines below use from now on (launchers such as
 * torch.distributed.run export OMP_NUM_THREADS=1, which the timed baseline must not inherit). */
#ifdef _OPENMP
#include <omp.h>
void FN(set_threads)(int n) { if (n > 0) omp_set_num_threads(n); }
int FN(max_threads)(void) { return omp_get_max_threads(); }
#else
void FN(set_threads)(int n) { (void)n; }
int FN(max_threads)(void) { return 1; }
#endif

/* ------------------------------------------------------------------------ */
/* Depthwise convolution.                                                   */
/* Layouts: x [N,C,H,W]; weight [M,C,kH,kW]; bias [M,C]; y [N,C*M,oH,oW]     */
/* with output channel c*M+j  (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:76-121,244). */
/* ------------------------------------------------------------------------ */

/* Forward: per (image, channel) a [M x k*k]*[k*k x oHW] product on the unfolded
 * plane plus a bias broadcast
 * (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:150-226; unfold with zero
 * padding: lib/THCUNN/im2col.h:18-37). */
void FN(dwconv_forward)(const real_t *x, const real_t *w, const real_t *bias, real_t *y,
                        int N, int C, int H, int W, int M, int kH, int kW,
                        int dH, int dW, int padH, int padW)
{
    const int oH = (H + 2 * padH - kH) / dH + 1;
    const int oW = (W + 2 * padW - kW) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const real_t *xp = x + ((size_t)n * C + c) * H * W;
            for (int j = 0; j < M; ++j) {
                const real_t *wp = w + ((size_t)j * C + c) * kH * kW;
                real_t *yp = y + (((size_t)n * C + c) * M + j) * oH * oW;
                const acc_t b = bias ? (acc_t)bias[(size_t)j * C + c] : (acc_t)0;
                for (int oh = 0; oh < oH; ++oh)
                    for (int ow = 0; ow < oW; ++ow) {
                        acc_t s = b;
                        for (int kh = 0; kh < kH; ++kh) {
                            const int ih = oh * dH - padH + kh;
                            if (ih < 0 || ih >= H) continue;
                            for (int kw = 0; kw < kW; ++kw) {
                                const int iw = ow * dW - padW + kw;
                                if (iw < 0 || iw >= W) continue;
                                s += (acc_t)wp[kh * kW + kw] * (acc_t)xp[ih * W + iw];
                            }
                        }
                        yp[oh * oW + ow] = (real_t)s;
                    }
            }
        }
}

/* Input gradient: W^T * gy per (image, channel), folded back with col2im
 * (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:346-400; fold:
 * lib/THCUNN/im2col.h:72-101).  gy is read as contiguous [N,C,M,oH,oW]. */
void FN(dwconv_grad_input)(const real_t *gy, const real_t *w, real_t *gx,
                           int N, int C, int H, int W, int M, int kH, int kW,
                           int dH, int dW, int padH, int padW)
{
    const int oH = (H + 2 * padH - kH) / dH + 1;
    const int oW = (W + 2 * padW - kW) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            real_t *gxp = gx + ((size_t)n * C + c) * H * W;
            for (int h = 0; h < H; ++h)
                for (int wi = 0; wi < W; ++wi) {
                    acc_t s = 0;
                    for (int j = 0; j < M; ++j) {
                        const real_t *wp = w + ((size_t)j * C + c) * kH * kW;
                        const real_t *gyp = gy + (((size_t)n * C + c) * M + j) * oH * oW;
                        for (int kh = 0; kh < kH; ++kh) {
                            const int t = h + padH - kh;
                            if (t < 0 || t % dH) continue;
                            const int oh = t / dH;
                            if (oh >= oH) continue;
                            for (int kw = 0; kw < kW; ++kw) {
                                const int u = wi + padW - kw;
                                if (u < 0 || u % dW) continue;
                                const int ow = u / dW;
                                if (ow >= oW) continue;
                                s += (acc_t)wp[kh * kW + kw] * (acc_t)gyp[oh * oW + ow];
                            }
                        }
                    }
                    gxp[h * W + wi] = (real_t)s;
                }
        }
}

/* Parameter gradients, ACCUMULATED into gw / gb (GEMM and GEMV with beta = 1:
 * lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:546-613). gb may be NULL. */
void FN(dwconv_acc_grad)(const real_t *x, const real_t *gy, real_t *gw, real_t *gb,
                         int N, int C, int H, int W, int M, int kH, int kW,
                         int dH, int dW, int padH, int padW, real_t scale)
{
    const int oH = (H + 2 * padH - kH) / dH + 1;
    const int oW = (W + 2 * padW - kW) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int c = 0; c < C; ++c)
        for (int j = 0; j < M; ++j) {
            acc_t sb = 0;
            acc_t sw[64];
            const int kk = kH * kW;
            for (int i = 0; i < kk && i < 64; ++i) sw[i] = 0;
            for (int n = 0; n < N; ++n) {
                const real_t *xp = x + ((size_t)n * C + c) * H * W;
                const real_t *gyp = gy + (((size_t)n * C + c) * M + j) * oH * oW;
                for (int oh = 0; oh < oH; ++oh)
                    for (int ow = 0; ow < oW; ++ow) {
                        const acc_t g = gyp[oh * oW + ow];
                        sb += g;
                        for (int kh = 0; kh < kH; ++kh) {
                            const int ih = oh * dH - padH + kh;
                            if (ih < 0 || ih >= H) continue;
                            for (int kw = 0; kw < kW; ++kw) {
                                const int iw = ow * dW - padW + kw;
                                if (iw < 0 || iw >= W) continue;
                                sw[kh * kW + kw] += g * (acc_t)xp[ih * W + iw];
                            }
                        }
                    }
            }
            real_t *gwp = gw + ((size_t)j * C + c) * kk;
            for (int i = 0; i < kk; ++i) gwp[i] = (real_t)((acc_t)gwp[i] + (acc_t)scale * sw[i]);
            if (gb) gb[(size_t)j * C + c] = (real_t)((acc_t)gb[(size_t)j * C + c] + (acc_t)scale * sb);
        }
}

/* ------------------------------------------------------------------------ */
/* SpatialConvolutionMM.  x [N,C,H,W]; weight [K, C*kH*kW]; bias [K];        */
/* y [N,K,oH,oW].                                                            */
/* ------------------------------------------------------------------------ */

/* The three passes below take dilation factors: SpatialConvolutionMM is the case dilH = dilW = 1,
 * SpatialDilatedConvolution (lib/THCUNN/generic/SpatialDilatedConvolution.cu:49-50,104-105: output size
 * (in + 2 pad - (dil (k - 1) + 1)) / stride + 1; unfold with dilation, lib/THCUNN/im2col.h:18-37) the general one. */

/* Forward: y_n = bias*ones + W * im2col(x_n)
 * (lib/THCUNN/generic/SpatialConvolutionMM.cu:129-194, SpatialDilatedConvolution.cu:140-196). */
void FN(dilconv_forward)(const real_t *x, const real_t *w, const real_t *bias, real_t *y,
                         int N, int C, int H, int W, int K, int kH, int kW,
                         int dH, int dW, int padH, int padW, int dilH, int dilW)
{
    const int oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) / dH + 1;
    const int oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            real_t *yp = y + ((size_t)n * K + k) * oH * oW;
            const acc_t b = bias ? (acc_t)bias[k] : (acc_t)0;
            for (int oh = 0; oh < oH; ++oh)
                for (int ow = 0; ow < oW; ++ow) {
                    acc_t s = b;
                    for (int c = 0; c < C; ++c) {
                        const real_t *xp = x + ((size_t)n * C + c) * H * W;
                        const real_t *wp = w + ((size_t)k * C + c) * kH * kW;
                        for (int kh = 0; kh < kH; ++kh) {
                            const int ih = oh * dH - padH + kh * dilH;
                            if (ih < 0 || ih >= H) continue;
                            for (int kw = 0; kw < kW; ++kw) {
                                const int iw = ow * dW - padW + kw * dilW;
                                if (iw < 0 || iw >= W) continue;
                                s += (acc_t)wp[kh * kW + kw] * (acc_t)xp[ih * W + iw];
                            }
                        }
                    }
                    yp[oh * oW + ow] = (real_t)s;
                }
        }
}

/* Input gradient: gx_n = col2im(W^T * gy_n)
 * (lib/THCUNN/generic/SpatialConvolutionMM.cu:272-308, SpatialDilatedConvolution.cu:244-290). */
void FN(dilconv_grad_input)(const real_t *gy, const real_t *w, real_t *gx,
                            int N, int C, int H, int W, int K, int kH, int kW,
                            int dH, int dW, int padH, int padW, int dilH, int dilW)
{
    const int oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) / dH + 1;
    const int oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            real_t *gxp = gx + ((size_t)n * C + c) * H * W;
            for (int h = 0; h < H; ++h)
                for (int wi = 0; wi < W; ++wi) {
                    acc_t s = 0;
                    for (int kh = 0; kh < kH; ++kh) {
                        const int t = h + padH - kh * dilH;
                        if (t < 0 || t % dH) continue;
                        const int oh = t / dH;
                        if (oh >= oH) continue;
                        for (int kw = 0; kw < kW; ++kw) {
                            const int u = wi + padW - kw * dilW;
                            if (u < 0 || u % dW) continue;
                            const int ow = u / dW;
                            if (ow >= oW) continue;
                            for (int k = 0; k < K; ++k)
                                s += (acc_t)w[((size_t)k * C + c) * kH * kW + kh * kW + kw] *
                                     (acc_t)gy[((size_t)n * K + k) * oH * oW + oh * oW + ow];
                        }
                    }
                    gxp[h * W + wi] = (real_t)s;
                }
        }
}

/* Parameter gradients, accumulated: gW += scale * sum_n gy_n * im2col(x_n)^T,
 * gb += scale * sum gy  (lib/THCUNN/generic/SpatialConvolutionMM.cu:396-470,
 * SpatialDilatedConvolution.cu:350-440). */
void FN(dilconv_acc_grad)(const real_t *x, const real_t *gy, real_t *gw, real_t *gb,
                          int N, int C, int H, int W, int K, int kH, int kW,
                          int dH, int dW, int padH, int padW, int dilH, int dilW, real_t scale)
{
    const int oH = (H + 2 * padH - (dilH * (kH - 1) + 1)) / dH + 1;
    const int oW = (W + 2 * padW - (dilW * (kW - 1) + 1)) / dW + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int k = 0; k < K; ++k)
        for (int c = 0; c < C; ++c) {
            for (int kh = 0; kh < kH; ++kh)
                for (int kw = 0; kw < kW; ++kw) {
                    acc_t s = 0;
                    for (int n = 0; n < N; ++n) {
                        const real_t *xp = x + ((size_t)n * C + c) * H * W;
                        const real_t *gyp = gy + ((size_t)n * K + k) * oH * oW;
                        for (int oh = 0; oh < oH; ++oh) {
                            const int ih = oh * dH - padH + kh * dilH;
                            if (ih < 0 || ih >= H) continue;
                            for (int ow = 0; ow < oW; ++ow) {
                                const int iw = ow * dW - padW + kw * dilW;
                                if (iw < 0 || iw >= W) continue;
                                s += (acc_t)gyp[oh * oW + ow] * (acc_t)xp[ih * W + iw];
                            }
                        }
                    }
                    real_t *p = gw + ((size_t)k * C + c) * kH * kW + kh * kW + kw;
                    *p = (real_t)((acc_t)*p + (acc_t)scale * s);
                }
        }
    if (gb) {
#pragma omp parallel for schedule(static)
        for (int k = 0; k < K; ++k) {
            acc_t s = 0;
            for (int n = 0; n < N; ++n) {
                const real_t *gyp = gy + ((size_t)n * K + k) * oH * oW;
                for (int i = 0; i < oH * oW; ++i) s += (acc_t)gyp[i];
            }
            gb[k] = (real_t)((acc_t)gb[k] + (acc_t)scale * s);
        }
    }
}

void FN(convmm_forward)(const real_t *x, const real_t *w, const real_t *bias, real_t *y,
                        int N, int C, int H, int W, int K, int kH, int kW,
                        int dH, int dW, int padH, int padW)
{
    FN(dilconv_forward)(x, w, bias, y, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1);
}

void FN(convmm_grad_input)(const real_t *gy, const real_t *w, real_t *gx,
                           int N, int C, int H, int W, int K, int kH, int kW,
                           int dH, int dW, int padH, int padW)
{
    FN(dilconv_grad_input)(gy, w, gx, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1);
}

void FN(convmm_acc_grad)(const real_t *x, const real_t *gy, real_t *gw, real_t *gb,
                         int N, int C, int H, int W, int K, int kH, int kW,
                         int dH, int dW, int padH, int padW, real_t scale)
{
    FN(dilconv_acc_grad)(x, gy, gw, gb, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, scale);
}

/* ------------------------------------------------------------------------ */
/* Transposed ("full") dilated convolution: x [N,P,H,W], weight [P,Q,kH,kW],  */
/* y [N,Q,OH,OW] with OH = (H-1)*dH - 2*padH + dilH*(kH-1) + 1 + adjH.         */
/* ------------------------------------------------------------------------ */

/* Forward: y_n = col2im(W^T * x_n) + bias
 * (lib/THCUNN/generic/SpatialFullDilatedConvolution.cu:68-209; output size :51-52). */
void FN(fullconv_forward)(const real_t *x, const real_t *w, const real_t *bias, real_t *y,
                          int N, int P, int H, int W, int Q, int kH, int kW,
                          int dH, int dW, int padH, int padW, int dilH, int dilW, int adjH, int adjW)
{
    const int OH = (H - 1) * dH - 2 * padH + dilH * (kH - 1) + 1 + adjH;
    const int OW = (W - 1) * dW - 2 * padW + dilW * (kW - 1) + 1 + adjW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int q = 0; q < Q; ++q) {
            real_t *yp = y + ((size_t)n * Q + q) * OH * OW;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    acc_t s = bias ? (acc_t)bias[q] : (acc_t)0;
                    for (int kh = 0; kh < kH; ++kh) {
                        const int t = oh + padH - kh * dilH;
                        if (t < 0 || t % dH || t / dH >= H) continue;
                        for (int kw = 0; kw < kW; ++kw) {
                            const int u = ow + padW - kw * dilW;
                            if (u < 0 || u % dW || u / dW >= W) continue;
                            for (int p = 0; p < P; ++p)
                                s += (acc_t)w[((size_t)p * Q + q) * kH * kW + kh * kW + kw] *
                                     (acc_t)x[(((size_t)n * P + p) * H + t / dH) * W + u / dW];
                        }
                    }
                    yp[oh * OW + ow] = (real_t)s;
                }
        }
}

/* Input gradient: gx_n = W * im2col(gy_n)
 * (lib/THCUNN/generic/SpatialFullDilatedConvolution.cu:211-317). */
void FN(fullconv_grad_input)(const real_t *gy, const real_t *w, real_t *gx,
                             int N, int P, int H, int W, int Q, int kH, int kW,
                             int dH, int dW, int padH, int padW, int dilH, int dilW, int adjH, int adjW)
{
    const int OH = (H - 1) * dH - 2 * padH + dilH * (kH - 1) + 1 + adjH;
    const int OW = (W - 1) * dW - 2 * padW + dilW * (kW - 1) + 1 + adjW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int p = 0; p < P; ++p)
            for (int ih = 0; ih < H; ++ih)
                for (int iw = 0; iw < W; ++iw) {
                    acc_t s = 0;
                    for (int q = 0; q < Q; ++q) {
                        const real_t *gyp = gy + ((size_t)n * Q + q) * OH * OW;
                        const real_t *wp = w + ((size_t)p * Q + q) * kH * kW;
                        for (int kh = 0; kh < kH; ++kh) {
                            const int oh = ih * dH - padH + kh * dilH;
                            if (oh < 0 || oh >= OH) continue;
                            for (int kw = 0; kw < kW; ++kw) {
                                const int ow = iw * dW - padW + kw * dilW;
                                if (ow < 0 || ow >= OW) continue;
                                s += (acc_t)wp[kh * kW + kw] * (acc_t)gyp[oh * OW + ow];
                            }
                        }
                    }
                    gx[(((size_t)n * P + p) * H + ih) * W + iw] = (real_t)s;
                }
}

/* Parameter gradients, accumulated: gW += scale * sum_n x_n * im2col(gy_n)^T, gb += scale * sum gy
 * (lib/THCUNN/generic/SpatialFullDilatedConvolution.cu:319-461). */
void FN(fullconv_acc_grad)(const real_t *x, const real_t *gy, real_t *gw, real_t *gb,
                           int N, int P, int H, int W, int Q, int kH, int kW,
                           int dH, int dW, int padH, int padW, int dilH, int dilW, int adjH, int adjW, real_t scale)
{
    const int OH = (H - 1) * dH - 2 * padH + dilH * (kH - 1) + 1 + adjH;
    const int OW = (W - 1) * dW - 2 * padW + dilW * (kW - 1) + 1 + adjW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int p = 0; p < P; ++p)
        for (int q = 0; q < Q; ++q)
            for (int kh = 0; kh < kH; ++kh)
                for (int kw = 0; kw < kW; ++kw) {
                    acc_t s = 0;
                    for (int n = 0; n < N; ++n) {
                        const real_t *xp = x + ((size_t)n * P + p) * H * W;
                        const real_t *gyp = gy + ((size_t)n * Q + q) * OH * OW;
                        for (int ih = 0; ih < H; ++ih) {
                            const int oh = ih * dH - padH + kh * dilH;
                            if (oh < 0 || oh >= OH) continue;
                            for (int iw = 0; iw < W; ++iw) {
                                const int ow = iw * dW - padW + kw * dilW;
                                if (ow < 0 || ow >= OW) continue;
                                s += (acc_t)xp[ih * W + iw] * (acc_t)gyp[oh * OW + ow];
                            }
                        }
                    }
                    real_t *g = gw + ((size_t)p * Q + q) * kH * kW + kh * kW + kw;
                    *g = (real_t)((acc_t)*g + (acc_t)scale * s);
                }
    if (gb) {
#pragma omp parallel for schedule(static)
        for (int q = 0; q < Q; ++q) {
            acc_t s = 0;
            for (int n = 0; n < N; ++n) {
                const real_t *gyp = gy + ((size_t)n * Q + q) * OH * OW;
                for (int i = 0; i < OH * OW; ++i) s += (acc_t)gyp[i];
            }
            gb[q] = (real_t)((acc_t)gb[q] + (acc_t)scale * s);
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Batch normalisation over [N,C,S] (S = H*W).                               */
/* ------------------------------------------------------------------------ */

/* Forward.  Train: batch mean, biased variance, save_std = 1/sqrt(var+eps)
 * (0 when var == 0 and eps == 0), running stats updated with the UNBIASED
 * variance (lib/THCUNN/BatchNormalization.cu:167-212).  Eval: running stats
 * (lib/THCUNN/BatchNormalization.cu:141-164).  weight/bias may be NULL. */
void FN(bn_forward)(const real_t *x, real_t *y, const real_t *weight, const real_t *bias,
                    real_t *running_mean, real_t *running_var, real_t *save_mean, real_t *save_std,
                    int N, int C, int S, int train, double momentum, double eps)
{
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; ++c) {
        acc_t mean, invstd;
        if (train) {
            const acc_t cnt = (acc_t)N * S;
            acc_t s = 0;
            for (int n = 0; n < N; ++n) {
                const real_t *xp = x + ((size_t)n * C + c) * S;
                for (int i = 0; i < S; ++i) s += (acc_t)xp[i];
            }
            mean = s / cnt;
            acc_t v = 0;
            for (int n = 0; n < N; ++n) {
                const real_t *xp = x + ((size_t)n * C + c) * S;
                for (int i = 0; i < S; ++i) {
                    const acc_t d = (acc_t)xp[i] - mean;
                    v += d * d;
                }
            }
            invstd = 0;
            if (v != 0 || eps != 0) invstd = (acc_t)1 / (acc_t)sqrt((double)(v / cnt + (acc_t)eps));
            const acc_t unbiased = v / (cnt - 1);
            save_mean[c] = (real_t)mean;
            save_std[c] = (real_t)invstd;
            running_mean[c] = (real_t)((1 - momentum) * running_mean[c] + momentum * mean);
            running_var[c] = (real_t)((1 - momentum) * running_var[c] + momentum * unbiased);
        } else {
            mean = running_mean[c];
            invstd = (acc_t)1 / (acc_t)sqrt((double)((acc_t)running_var[c] + (acc_t)eps));
        }
        const acc_t g = weight ? (acc_t)weight[c] : (acc_t)1;
        const acc_t b = bias ? (acc_t)bias[c] : (acc_t)0;
        for (int n = 0; n < N; ++n) {
            const real_t *xp = x + ((size_t)n * C + c) * S;
            real_t *yp = y + ((size_t)n * C + c) * S;
            for (int i = 0; i < S; ++i) yp[i] = (real_t)(g * ((acc_t)xp[i] - mean) * invstd + b);
        }
    }
}

/* Backward (lib/THCUNN/BatchNormalization.cu:215-283).  gx, gw, gb may each be
 * NULL; gw and gb are accumulated with `scale`. */
void FN(bn_backward)(const real_t *x, const real_t *gy, real_t *gx, real_t *gw, real_t *gb,
                     const real_t *weight, const real_t *running_mean, const real_t *running_var,
                     const real_t *save_mean, const real_t *save_std,
                     int N, int C, int S, int train, double scale, double eps)
{
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; ++c) {
        acc_t mean, stdv;
        if (train) {
            mean = save_mean[c];
            stdv = save_std[c];
        } else {
            mean = running_mean[c];
            stdv = (acc_t)1 / (acc_t)sqrt((double)((acc_t)running_var[c] + (acc_t)eps));
        }
        const acc_t wv = weight ? (acc_t)weight[c] : (acc_t)1;
        const acc_t norm = (acc_t)1 / ((acc_t)N * S);
        acc_t sum = 0, dot = 0;
        for (int n = 0; n < N; ++n) {
            const real_t *xp = x + ((size_t)n * C + c) * S;
            const real_t *gp = gy + ((size_t)n * C + c) * S;
            for (int i = 0; i < S; ++i) {
                sum += (acc_t)gp[i];
                dot += (acc_t)gp[i] * ((acc_t)xp[i] - mean);
            }
        }
        const acc_t grad_mean = sum * norm;
        const acc_t proj_scale = dot * norm * stdv * stdv;
        const acc_t grad_scale = stdv * wv;
        if (gx) {
            for (int n = 0; n < N; ++n) {
                const real_t *xp = x + ((size_t)n * C + c) * S;
                const real_t *gp = gy + ((size_t)n * C + c) * S;
                real_t *op = gx + ((size_t)n * C + c) * S;
                for (int i = 0; i < S; ++i) {
                    if (train)
                        op[i] = (real_t)(((acc_t)gp[i] - ((acc_t)xp[i] - mean) * proj_scale - grad_mean) * grad_scale);
                    else
                        op[i] = (real_t)((acc_t)gp[i] * grad_scale);
                }
            }
        }
        if (gw) gw[c] = (real_t)((acc_t)gw[c] + (acc_t)scale * dot * stdv);
        if (gb) gb[c] = (real_t)((acc_t)gb[c] + (acc_t)scale * sum);
    }
}

/* ------------------------------------------------------------------------ */
/* Max pooling with argmax.                                                  */
/* ------------------------------------------------------------------------ */

/* Output extent along one axis, floor or ceil mode, with the "last window must
 * start inside input + pad" fix-up
 * (lib/THCUNN/generic/SpatialDilatedMaxPooling.cu:118-135), in integers. */
int FN(pool_out_size)(int in, int k, int d, int pad, int dil, int ceil_mode)
{
    const int num = in - (dil * (k - 1) + 1) + 2 * pad;
    int o;
    if (ceil_mode) o = (num >= 0 ? (num + d - 1) / d : -((-num) / d)) + 1;
    else           o = (num >= 0 ? num / d : -((-num + d - 1) / d)) + 1;
    if (pad && (o - 1) * d >= in + pad) --o;
    return o;
}

/* Forward: first strict maximum in row-major window order starting from
 * -FLT_MAX with index -1; stored index = per-plane flat h*W+w + index base
 * (lib/THCUNN/SpatialDilatedMaxPooling.cu:8-42).  NaN never wins. */
void FN(maxpool_forward)(const real_t *x, real_t *y, int64_t *ind,
                         int N, int C, int H, int W, int oH, int oW,
                         int kH, int kW, int dH, int dW, int padH, int padW,
                         int dilH, int dilW)
{
#pragma omp parallel for schedule(static)
    for (long p = 0; p < (long)N * C; ++p) {
        const real_t *xp = x + (size_t)p * H * W;
        for (int ph = 0; ph < oH; ++ph)
            for (int pw = 0; pw < oW; ++pw) {
                int hs = ph * dH - padH, ws = pw * dW - padW;
                int he = hs + (kH - 1) * dilH + 1; if (he > H) he = H;
                int we = ws + (kW - 1) * dilW + 1; if (we > W) we = W;
                while (hs < 0) hs += dilH;
                while (ws < 0) ws += dilW;
                real_t best = REAL_LOWEST;
                int bi = -1;
                for (int h = hs; h < he; h += dilH)
                    for (int w = ws; w < we; w += dilW)
                        if (xp[h * W + w] > best) { bi = h * W + w; best = xp[bi]; }
                y[(size_t)p * oH * oW + ph * oW + pw] = best;
                ind[(size_t)p * oH * oW + ph * oW + pw] = (int64_t)bi + REF_INDEX_BASE;
            }
    }
}

/* Backward, gather form: every input pixel sums gy over the outputs whose
 * stored index names it (lib/THCUNN/SpatialDilatedMaxPooling.cu:46-80). */
void FN(maxpool_backward)(const real_t *gy, const int64_t *ind, real_t *gx,
                          int N, int C, int H, int W, int oH, int oW,
                          int kH, int kW, int dH, int dW, int padH, int padW,
                          int dilH, int dilW)
{
#pragma omp parallel for schedule(static)
    for (long p = 0; p < (long)N * C; ++p) {
        const real_t *gp = gy + (size_t)p * oH * oW;
        const int64_t *ip = ind + (size_t)p * oH * oW;
        for (int h = 0; h < H; ++h)
            for (int w = 0; w < W; ++w) {
                const int eh = (kH - 1) * dilH + 1, ew = (kW - 1) * dilW + 1;
                const int phs = (h + padH < eh) ? 0 : (h + padH - eh) / dH + 1;
                int phe = (h + padH) / dH + 1; if (phe > oH) phe = oH;
                const int pws = (w + padW < ew) ? 0 : (w + padW - ew) / dW + 1;
                int pwe = (w + padW) / dW + 1; if (pwe > oW) pwe = oW;
                acc_t g = 0;
                for (int ph = phs; ph < phe; ++ph)
                    for (int pw = pws; pw < pwe; ++pw)
                        if (ip[ph * oW + pw] - REF_INDEX_BASE == h * W + w) g += (acc_t)gp[ph * oW + pw];
                gx[(size_t)p * H * W + h * W + w] = (real_t)g;
            }
    }
}

/* ------------------------------------------------------------------------ */
/* Support ops of the MobileNetV1 step.                                      */
/* ------------------------------------------------------------------------ */

/* Threshold forward: y = x > th ? x : val (lib/THCUNN/Threshold.cu:6-38). */
void FN(threshold_forward)(const real_t *x, real_t *y, size_t n, real_t th, real_t val)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) y[i] = x[i] > th ? x[i] : val;
}

/* Threshold backward: gx = x > th ? gy : 0 (lib/THCUNN/Threshold.cu:40-72). */
void FN(threshold_backward)(const real_t *x, const real_t *gy, real_t *gx, size_t n, real_t th)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) gx[i] = x[i] > th ? gy[i] : 0.0f;
}

/* Average pooling forward (lib/THCUNN/SpatialAveragePooling.cu:7-39): window
 * clipped to input + pad for the divisor when count_include_pad, else to the
 * input. */
void FN(avgpool_forward)(const real_t *x, real_t *y, int N, int C, int H, int W, int oH, int oW,
                         int kH, int kW, int dH, int dW, int padH, int padW, int count_include_pad)
{
#pragma omp parallel for schedule(static)
    for (long p = 0; p < (long)N * C; ++p)
        for (int ph = 0; ph < oH; ++ph)
            for (int pw = 0; pw < oW; ++pw) {
                int hs = ph * dH - padH, ws = pw * dW - padW;
                int he = hs + kH; if (he > H + padH) he = H + padH;
                int we = ws + kW; if (we > W + padW) we = W + padW;
                const int pool = (he - hs) * (we - ws);
                if (hs < 0) hs = 0;
                if (ws < 0) ws = 0;
                if (he > H) he = H;
                if (we > W) we = W;
                acc_t s = 0;
                for (int h = hs; h < he; ++h)
                    for (int w = ws; w < we; ++w) s += (acc_t)x[(size_t)p * H * W + h * W + w];
                const int div = count_include_pad ? pool : (he - hs) * (we - ws);
                y[(size_t)p * oH * oW + ph * oW + pw] = (real_t)(s / div);
            }
}

/* Average pooling backward (lib/THCUNN/SpatialAveragePooling.cu:42-82). */
void FN(avgpool_backward)(const real_t *gy, real_t *gx, int N, int C, int H, int W, int oH, int oW,
                          int kH, int kW, int dH, int dW, int padH, int padW, int count_include_pad)
{
#pragma omp parallel for schedule(static)
    for (long p = 0; p < (long)N * C; ++p)
        for (int h0 = 0; h0 < H; ++h0)
            for (int w0 = 0; w0 < W; ++w0) {
                const int h = h0 + padH, w = w0 + padW;
                const int phs = (h < kH) ? 0 : (h - kH) / dH + 1;
                int phe = h / dH + 1; if (phe > oH) phe = oH;
                const int pws = (w < kW) ? 0 : (w - kW) / dW + 1;
                int pwe = w / dW + 1; if (pwe > oW) pwe = oW;
                acc_t g = 0;
                for (int ph = phs; ph < phe; ++ph)
                    for (int pw = pws; pw < pwe; ++pw) {
                        int hs = ph * dH - padH, ws = pw * dW - padW;
                        int he = hs + kH; if (he > H + padH) he = H + padH;
                        int we = ws + kW; if (we > W + padW) we = W + padW;
                        const int pool = (he - hs) * (we - ws);
                        if (hs < 0) hs = 0;
                        if (ws < 0) ws = 0;
                        if (he > H) he = H;
                        if (we > W) we = W;
                        const int div = count_include_pad ? pool : (he - hs) * (we - ws);
                        g += (acc_t)gy[(size_t)p * oH * oW + ph * oW + pw] / div;
                    }
                gx[(size_t)p * H * W + h0 * W + w0] = (real_t)g;
            }
}

/* LogSoftMax over the last dimension of [B, D]
 * (lib/THCUNN/LogSoftMax.cu:246-296): x - max - log(sum exp(x - max)). */
void FN(logsoftmax_forward)(const real_t *x, real_t *y, int B, int D)
{
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b) {
        const real_t *xp = x + (size_t)b * D;
        real_t m = REAL_LOWEST;
        for (int i = 0; i < D; ++i) if (xp[i] > m) m = xp[i];
        acc_t s = 0;
        for (int i = 0; i < D; ++i) s += (acc_t)exp((double)xp[i] - (double)m);
        const acc_t l = (acc_t)m + (acc_t)log((double)s);
        for (int i = 0; i < D; ++i) y[(size_t)b * D + i] = (real_t)((acc_t)xp[i] - l);
    }
}

/* LogSoftMax backward (lib/THCUNN/LogSoftMax.cu:298-344):
 * gx = gy - exp(y) * sum(gy). */
void FN(logsoftmax_backward)(const real_t *y, const real_t *gy, real_t *gx, int B, int D)
{
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b) {
        acc_t s = 0;
        for (int i = 0; i < D; ++i) s += (acc_t)gy[(size_t)b * D + i];
        for (int i = 0; i < D; ++i)
            gx[(size_t)b * D + i] = (real_t)((acc_t)gy[(size_t)b * D + i] - (acc_t)exp((double)y[(size_t)b * D + i]) * s);
    }
}

/* ClassNLL forward over log-probabilities [B, D] with targets carrying the
 * index base (lib/THCUNN/ClassNLLCriterion.cu:38-84): loss = -sum w_t lp[t],
 * divided by sum w_t when size_average.  weights may be NULL. */
void FN(classnll_forward)(const real_t *lp, const int64_t *target, const real_t *weights,
                          real_t *loss, real_t *total_weight, int B, int D,
                          int size_average, int64_t ignore_index)
{
    acc_t s = 0, tw = 0;
    for (int b = 0; b < B; ++b) {
        const int64_t t = target[b] - REF_INDEX_BASE;
        if (t == ignore_index - REF_INDEX_BASE) continue;
        const acc_t w = weights ? (acc_t)weights[t] : (acc_t)1;
        s -= w * (acc_t)lp[(size_t)b * D + t];
        tw += w;
    }
    if (size_average && tw > 0) s /= tw;
    *loss = (real_t)s;
    *total_weight = (real_t)tw;
}

/* ClassNLL backward (lib/THCUNN/ClassNLLCriterion.cu:108-132): writes only the
 * target entries of gx; the caller zeroes gx first, as nn.ClassNLLCriterion
 * does. */
void FN(classnll_backward)(const int64_t *target, const real_t *weights, real_t total_weight,
                           real_t *gx, int B, int D, int size_average, int64_t ignore_index)
{
    if (total_weight <= 0) return;
    const acc_t norm = size_average ? (acc_t)1 / (acc_t)total_weight : (acc_t)1;
    for (int b = 0; b < B; ++b) {
        const int64_t t = target[b] - REF_INDEX_BASE;
        if (t == ignore_index - REF_INDEX_BASE) continue;
        const acc_t w = weights ? (acc_t)weights[t] : (acc_t)1;
        gx[(size_t)b * D + t] = (real_t)(-w * norm);
    }
}

/* ------------------------------------------------------------------------ */
/* DataParallelTable shard rule.                                             */
/* ------------------------------------------------------------------------ */

/* ------------------------------------------------------------------------ */
/* SpatialConvolutionLocal: a convolution whose weights are NOT shared       */
/* between output positions (lib/THCUNN/generic/SpatialConvolutionLocal.cu). */
/* weight [oH*oW, K, C*kH*kW] (:58-77), bias [K, oH, oW] (:37-41).           */
/*   y[n,k,p]  = bias[k,p] + sum_r W[p,k,r] col[n,r,p]          (:132-156)   */
/*   gx        = fold over p of W[p]^T gy[n,:,p]                (:232-262)   */
/*   gW[p,k,r] += scale sum_n gy[n,k,p] col[n,r,p]; gb += scale sum_n gy (:366-379) */
/* ------------------------------------------------------------------------ */
void FN(localconv_forward)(const real_t *x, const real_t *w, const real_t *bias, real_t *y,
                           int N, int C, int H, int W, int K, int kH, int kW,
                           int dH, int dW, int padH, int padW, int oH, int oW)
{
    const int P = oH * oW, R = C * kH * kW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            for (int p = 0; p < P; ++p) {
                const int oh = p / oW, ow = p % oW;
                acc_t s = bias ? (acc_t)bias[(size_t)k * P + p] : 0;
                const real_t *wp = w + ((size_t)p * K + k) * R;
                for (int c = 0; c < C; ++c)
                    for (int kh = 0; kh < kH; ++kh) {
                        const int ih = oh * dH - padH + kh;
                        if (ih < 0 || ih >= H) continue;
                        for (int kw_ = 0; kw_ < kW; ++kw_) {
                            const int iw = ow * dW - padW + kw_;
                            if (iw < 0 || iw >= W) continue;
                            s += (acc_t)wp[(c * kH + kh) * kW + kw_] * (acc_t)x[(((size_t)n * C + c) * H + ih) * W + iw];
                        }
                    }
                y[((size_t)n * K + k) * P + p] = (real_t)s;
            }
}

void FN(localconv_grad_input)(const real_t *gy, const real_t *w, real_t *gx,
                              int N, int C, int H, int W, int K, int kH, int kW,
                              int dH, int dW, int padH, int padW, int oH, int oW)
{
    const int P = oH * oW, R = C * kH * kW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
            for (int h = 0; h < H; ++h)
                for (int wi = 0; wi < W; ++wi) {
                    acc_t s = 0;
                    for (int kh = 0; kh < kH; ++kh) {
                        const int a = h + padH - kh;
                        if (a < 0 || a % dH || a / dH >= oH) continue;
                        for (int kw_ = 0; kw_ < kW; ++kw_) {
                            const int b = wi + padW - kw_;
                            if (b < 0 || b % dW || b / dW >= oW) continue;
                            const int p = (a / dH) * oW + b / dW;
                            for (int k = 0; k < K; ++k)
                                s += (acc_t)w[((size_t)p * K + k) * R + (c * kH + kh) * kW + kw_] * (acc_t)gy[((size_t)n * K + k) * P + p];
                        }
                    }
                    gx[(((size_t)n * C + c) * H + h) * W + wi] = (real_t)s;
                }
}

void FN(localconv_acc_grad)(const real_t *x, const real_t *gy, real_t *gw, real_t *gb,
                            int N, int C, int H, int W, int K, int kH, int kW,
                            int dH, int dW, int padH, int padW, int oH, int oW, real_t scale)
{
    const int P = oH * oW, R = C * kH * kW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int p = 0; p < P; ++p)
        for (int k = 0; k < K; ++k) {
            const int oh = p / oW, ow = p % oW;
            for (int c = 0; c < C; ++c)
                for (int kh = 0; kh < kH; ++kh)
                    for (int kw_ = 0; kw_ < kW; ++kw_) {
                        const int ih = oh * dH - padH + kh, iw = ow * dW - padW + kw_;
                        acc_t s = 0;
                        if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                            for (int n = 0; n < N; ++n)
                                s += (acc_t)gy[((size_t)n * K + k) * P + p] * (acc_t)x[(((size_t)n * C + c) * H + ih) * W + iw];
                        real_t *g = gw + ((size_t)p * K + k) * R + (c * kH + kh) * kW + kw_;
                        *g = (real_t)((acc_t)*g + (acc_t)scale * s);
                    }
            if (gb) {
                acc_t s = 0;
                for (int n = 0; n < N; ++n) s += (acc_t)gy[((size_t)n * K + k) * P + p];
                gb[(size_t)k * P + p] = (real_t)((acc_t)gb[(size_t)k * P + p] + (acc_t)scale * s);
            }
        }
}

/* ------------------------------------------------------------------------ */
/* Adaptive pooling to a given output size.  Window of output row i:         */
/*   max:     [floor(float(i) / oH * H), ceil(float(i + 1) / oH * H))   (lib/THCUNN/SpatialAdaptiveMaxPooling.cu:44-52)     */
/*   average: [floor((float)(i * H) / oH), ceil((float)((i + 1) * H) / oH))  (lib/THCUNN/SpatialAdaptiveAveragePooling.cu:6-7) */
/* both in float arithmetic, as the kernels compute them.                    */
/* Max: strict > from the lowest finite value, first maximum wins; indices are stored as two planes,               */
/* ind[0] = row and ind[1] = column of the maximum RELATIVE to the window start, plus the index base              */
/* (:62-78, launch generic/SpatialAdaptiveMaxPooling.cu:48-50: indices_x is the second half).                      */
/* ------------------------------------------------------------------------ */
static int amax_start(int i, int o, int n) { return (int)floorf((float)i / (float)o * (float)n); }
static int amax_end(int i, int o, int n) { return (int)ceilf((float)(i + 1) / (float)o * (float)n); }
static int aavg_start(int i, int o, int n) { return (int)floorf((float)(i * n) / (float)o); }
static int aavg_end(int i, int o, int n) { return (int)ceilf((float)((i + 1) * n) / (float)o); }

void FN(adaptive_maxpool_forward)(const real_t *x, real_t *y, int64_t *ind, int planes, int H, int W, int oH, int oW)
{
    const size_t half = (size_t)planes * oH * oW;
#pragma omp parallel for schedule(static)
    for (int p = 0; p < planes; ++p)
        for (int yy = 0; yy < oH; ++yy)
            for (int xx = 0; xx < oW; ++xx) {
                const int y0 = amax_start(yy, oH, H), y1 = amax_end(yy, oH, H), x0 = amax_start(xx, oW, W), x1 = amax_end(xx, oW, W);
                real_t best = REAL_LOWEST;
                int by = -1, bx = -1;
                for (int h = y0; h < y1; ++h)
                    for (int w = x0; w < x1; ++w) {
                        const real_t v = x[((size_t)p * H + h) * W + w];
                        if (v > best) { best = v; by = h - y0; bx = w - x0; }
                    }
                const size_t o = ((size_t)p * oH + yy) * oW + xx;
                y[o] = best;
                ind[o] = by + REF_INDEX_BASE;
                ind[half + o] = bx + REF_INDEX_BASE;
            }
}

/* gx[window start + stored offset] += gy, summed over the outputs (atomicadaptivemaxgradinput, :133-176). */
void FN(adaptive_maxpool_backward)(const real_t *gy, const int64_t *ind, real_t *gx, int planes, int H, int W, int oH, int oW)
{
    const size_t half = (size_t)planes * oH * oW;
#pragma omp parallel for schedule(static)
    for (int p = 0; p < planes; ++p) {
        acc_t *tmp = (acc_t *)calloc((size_t)H * W, sizeof(acc_t));
        for (int yy = 0; yy < oH; ++yy)
            for (int xx = 0; xx < oW; ++xx) {
                const size_t o = ((size_t)p * oH + yy) * oW + xx;
                const int h = amax_start(yy, oH, H) + (int)(ind[o] - REF_INDEX_BASE), w = amax_start(xx, oW, W) + (int)(ind[half + o] - REF_INDEX_BASE);
                tmp[(size_t)h * W + w] += (acc_t)gy[o];
            }
        for (int i = 0; i < H * W; ++i) gx[(size_t)p * H * W + i] = (real_t)tmp[i];
        free(tmp);
    }
}

void FN(adaptive_avgpool_forward)(const real_t *x, real_t *y, int planes, int H, int W, int oH, int oW)
{
#pragma omp parallel for schedule(static)
    for (int p = 0; p < planes; ++p)
        for (int yy = 0; yy < oH; ++yy)
            for (int xx = 0; xx < oW; ++xx) {
                const int y0 = aavg_start(yy, oH, H), y1 = aavg_end(yy, oH, H), x0 = aavg_start(xx, oW, W), x1 = aavg_end(xx, oW, W);
                acc_t s = 0;
                for (int h = y0; h < y1; ++h)
                    for (int w = x0; w < x1; ++w) s += (acc_t)x[((size_t)p * H + h) * W + w];
                y[((size_t)p * oH + yy) * oW + xx] = (real_t)(s / (y1 - y0) / (x1 - x0));
            }
}

/* every input of a window receives gy / kW / kH (atomicadaptiveaveragegradinput, lib/THCUNN/SpatialAdaptiveAveragePooling.cu:143-190). */
void FN(adaptive_avgpool_backward)(const real_t *gy, real_t *gx, int planes, int H, int W, int oH, int oW)
{
#pragma omp parallel for schedule(static)
    for (int p = 0; p < planes; ++p) {
        acc_t *tmp = (acc_t *)calloc((size_t)H * W, sizeof(acc_t));
        for (int yy = 0; yy < oH; ++yy)
            for (int xx = 0; xx < oW; ++xx) {
                const int y0 = aavg_start(yy, oH, H), y1 = aavg_end(yy, oH, H), x0 = aavg_start(xx, oW, W), x1 = aavg_end(xx, oW, W);
                const acc_t z = (acc_t)gy[((size_t)p * oH + yy) * oW + xx] / (x1 - x0) / (y1 - y0);
                for (int h = y0; h < y1; ++h)
                    for (int w = x0; w < x1; ++w) tmp[(size_t)h * W + w] += z;
            }
        for (int i = 0; i < H * W; ++i) gx[(size_t)p * H * W + i] = (real_t)tmp[i];
        free(tmp);
    }
}

/* Rows [start, start+count) of a batch of `n` rows that replica `i` (0-based)
 * of `g` receives: the first n mod g replicas get one extra row
 * (DataParallelTable.lua:469-479).  Zero-based start. */
void FN(slice_range)(long n, int g, int i, long *start, long *count)
{
    const long base = n / g, extra = n % g;
    *count = base + (i < extra ? 1 : 0);
    *start = (long)i * base + (i < extra ? i : extra);
}
