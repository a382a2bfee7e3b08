/* Test infrastructure: the reference's convolution schedule on the GPU — its OWN unfold / fold
 * kernels (lib/THCUNN/im2col.h:10-121, compiled from where they lie behind ref_shim/) around cuBLAS
 * SGEMM / SGEMV calls, one image at a time for SpatialConvolutionMM and one (image, channel) plane at
 * a time for SpatialDepthWiseConvolution.  The host loops below are this repository's restatement of
 * the reference wrappers' call sequence; each cites the lines it follows.  cuBLAS stands where the
 * reference calls THCudaBlas_Sgemm / Sgemv (cutorch forwards those to cuBLAS); plain fp32 SGEMM, no
 * TF32 math mode.  Everything runs on the legacy default stream; callers synchronise.
 *
 * Matrix roles, in row-major words (the reference states them in cuBLAS's column-major form):
 *   forward   out_n[K, oHW]  = bias[K] 1^T + W[K, CKK] col_n[CKK, oHW]
 *   dgrad     gcol[CKK, oHW] = W^T gy_n[K, oHW];  gx_n = fold(gcol)
 *   wgrad     gW[K, CKK]    += scale * gy_n[K, oHW] col_n^T ;  gb[K] += scale * gy_n 1
 */
#include <cublas_v2.h>

#include "im2col.h"

#define REFK_EXPORT extern "C" __attribute__((visibility("default")))

static cublasHandle_t refk_blas() {
  static cublasHandle_t h = 0;
  if (!h) {
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); std::abort(); }
    cublasSetMathMode(h, CUBLAS_PEDANTIC_MATH);
  }
  return h;
}
#define REFK_BLAS(expr) \
  do { if ((expr) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cuBLAS call failed at %s:%d\n", __FILE__, __LINE__); std::abort(); } } while (0)

__global__ void refk_fill_kernel(float *p, long n, float v) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)blockDim.x * gridDim.x) p[i] = v;
}
static void refk_fill(float *p, long n, float v) {
  if (n > 0) refk_fill_kernel<<<(int)((n + 1023) / 1024 > 4096 ? 4096 : (n + 1023) / 1024), 1024>>>(p, n, v);
}

static inline int out_size(int in, int k, int d, int pad, int dil) { return (in + 2 * pad - (dil * (k - 1) + 1)) / d + 1; }

/* Raw unfold / fold of one image, for pinning index arithmetic (im2col.h:41-61, :105-121). */
REFK_EXPORT void refk_im2col(const float *x, int C, int H, int W, int kH, int kW, int padH, int padW, int dH, int dW,
                             int dilH, int dilW, float *col) {
  im2col<float>(0, x, C, H, W, kH, kW, padH, padW, dH, dW, dilH, dilW, col);
}
REFK_EXPORT void refk_col2im(const float *col, int C, int H, int W, int kH, int kW, int padH, int padW, int dH, int dW,
                             int dilH, int dilW, float *x) {
  col2im<float, float>(0, col, C, H, W, out_size(H, kH, dH, padH, dilH), out_size(W, kW, dW, padW, dilW), kH, kW, padH,
                       padW, dH, dW, dilH, dilW, x);
}

/* Bytes of scratch the schedules below need: the column buffer and the all-ones vector the
 * reference keeps per module (generic/SpatialConvolutionMM.cu:113-122). */
REFK_EXPORT size_t refk_conv_scratch_bytes(int C, int H, int W, int kH, int kW, int dH, int dW, int padH, int padW) {
  long oHW = (long)out_size(H, kH, dH, padH, 1) * out_size(W, kW, dW, padW, 1);
  return (size_t)((long)C * kH * kW * oHW + oHW) * sizeof(float);
}

/* generic/SpatialConvolutionMM.cu:129-194. */
REFK_EXPORT void refk_convmm_forward(const float *x, const float *w, const float *bias, float *y, int N, int C, int H,
                                     int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, CKK = C * kH * kW;
  float *col = scratch, *ones = scratch + (long)CKK * oHW;
  const float one = 1.f, zero = 0.f;
  refk_fill(ones, oHW, 1.f);
  for (int n = 0; n < N; ++n) {
    float *y_n = y + (long)n * K * oHW;
    if (bias)
      REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_T, CUBLAS_OP_N, oHW, K, 1, &one, ones, 1, bias, 1, &zero, y_n, oHW));
    else
      cudaMemsetAsync(y_n, 0, sizeof(float) * K * oHW, 0);
    im2col<float>(0, x + (long)n * C * H * W, C, H, W, kH, kW, padH, padW, dH, dW, 1, 1, col);
    REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_N, CUBLAS_OP_N, oHW, K, CKK, &one, col, oHW, w, CKK, &one, y_n, oHW));
  }
}

/* generic/SpatialConvolutionMM.cu:272-308. */
REFK_EXPORT void refk_convmm_grad_input(const float *gy, const float *w, float *gx, int N, int C, int H, int W, int K,
                                        int kH, int kW, int dH, int dW, int padH, int padW, float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, CKK = C * kH * kW;
  float *gcol = scratch;
  const float one = 1.f, zero = 0.f;
  for (int n = 0; n < N; ++n) {
    REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_N, CUBLAS_OP_T, oHW, CKK, K, &one, gy + (long)n * K * oHW, oHW, w, CKK,
                          &zero, gcol, oHW));
    col2im<float, float>(0, gcol, C, H, W, oH, oW, kH, kW, padH, padW, dH, dW, 1, 1, gx + (long)n * C * H * W);
  }
}

/* generic/SpatialConvolutionMM.cu:396-470 (accumulates into gw / gb). */
REFK_EXPORT void refk_convmm_acc_grad(const float *x, const float *gy, float *gw, float *gb, int N, int C, int H, int W,
                                      int K, int kH, int kW, int dH, int dW, int padH, int padW, float scale,
                                      float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, CKK = C * kH * kW;
  float *col = scratch, *ones = scratch + (long)CKK * oHW;
  const float one = 1.f;
  refk_fill(ones, oHW, 1.f);
  for (int n = 0; n < N; ++n) {
    const float *gy_n = gy + (long)n * K * oHW;
    im2col<float>(0, x + (long)n * C * H * W, C, H, W, kH, kW, padH, padW, dH, dW, 1, 1, col);
    REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_T, CUBLAS_OP_N, CKK, K, oHW, &scale, col, oHW, gy_n, oHW, &one, gw, CKK));
    if (gb) REFK_BLAS(cublasSgemv(refk_blas(), CUBLAS_OP_T, oHW, K, &scale, gy_n, oHW, ones, 1, &one, gb, 1));
  }
}

/* SpatialDepthWiseConvolution.  Weights arrive as the module holds them, [M, C, kH, kW] and bias
 * [M, C]; the reference first makes channel-major contiguous copies (generic/
 * SpatialDepthWiseConvolution.cu:84-99), which `wt` / `bt` (C*M*kH*kW and C*M floats at the head of
 * scratch) hold here.  Scratch = wt | bt | col[kH*kW, oHW] | ones[oHW]. */
REFK_EXPORT size_t refk_dwconv_scratch_bytes(int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH,
                                             int padW) {
  long oHW = (long)out_size(H, kH, dH, padH, 1) * out_size(W, kW, dW, padW, 1);
  return (size_t)((long)C * M * kH * kW + (long)C * M + (long)kH * kW * oHW + oHW) * sizeof(float);
}

__global__ void refk_transpose01_kernel(const float *src, float *dst, int A, int B, int inner) {
  long total = (long)A * B * inner;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)blockDim.x * gridDim.x) {
    int r = (int)(i % inner);
    long ab = i / inner;
    int b = (int)(ab % B), a = (int)(ab / B);          /* dst is [B, A, inner] at (b, a) <- src [A, B, inner] at (a, b) */
    dst[((long)b * A + a) * inner + r] = src[i];
  }
}
static void refk_transpose01(const float *src, float *dst, int A, int B, int inner) {
  long total = (long)A * B * inner;
  if (total > 0) refk_transpose01_kernel<<<(int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256), 256>>>(src, dst, A, B, inner);
}

/* generic/SpatialDepthWiseConvolution.cu:150-226. */
REFK_EXPORT void refk_dwconv_forward(const float *x, const float *w, const float *bias, float *y, int N, int C, int H,
                                     int W, int M, int kH, int kW, int dH, int dW, int padH, int padW, float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, KK = kH * kW;
  float *wt = scratch, *bt = wt + (long)C * M * KK, *col = bt + (long)C * M, *ones = col + (long)KK * oHW;
  const float one = 1.f, zero = 0.f;
  refk_transpose01(w, wt, M, C, KK);
  if (bias) refk_transpose01(bias, bt, M, C, 1);
  refk_fill(ones, oHW, 1.f);
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      float *y_i = y + ((long)n * C + c) * M * oHW;
      if (bias)
        REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_T, CUBLAS_OP_N, oHW, M, 1, &one, ones, 1, bt + (long)c * M, 1, &zero, y_i, oHW));
      else
        cudaMemsetAsync(y_i, 0, sizeof(float) * M * oHW, 0);
      im2col<float>(0, x + ((long)n * C + c) * H * W, 1, H, W, kH, kW, padH, padW, dH, dW, 1, 1, col);
      REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_N, CUBLAS_OP_N, oHW, M, KK, &one, col, oHW, wt + (long)c * M * KK, KK, &one, y_i, oHW));
    }
}

/* generic/SpatialDepthWiseConvolution.cu:343-396. */
REFK_EXPORT void refk_dwconv_grad_input(const float *gy, const float *w, float *gx, int N, int C, int H, int W, int M,
                                        int kH, int kW, int dH, int dW, int padH, int padW, float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, KK = kH * kW;
  float *wt = scratch, *bt = wt + (long)C * M * KK, *gcol = bt + (long)C * M;
  const float one = 1.f, zero = 0.f;
  refk_transpose01(w, wt, M, C, KK);
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_N, CUBLAS_OP_T, oHW, KK, M, &one, gy + ((long)n * C + c) * M * oHW, oHW,
                            wt + (long)c * M * KK, KK, &zero, gcol, oHW));
      col2im<float, float>(0, gcol, 1, H, W, oH, oW, kH, kW, padH, padW, dH, dW, 1, 1, gx + ((long)n * C + c) * H * W);
    }
}

/* generic/SpatialDepthWiseConvolution.cu:520-629: accumulate into channel-major copies of the
 * caller's gradients, then write them back in the caller's [M, C, ...] layout. */
REFK_EXPORT void refk_dwconv_acc_grad(const float *x, const float *gy, float *gw, float *gb, int N, int C, int H, int W,
                                      int M, int kH, int kW, int dH, int dW, int padH, int padW, float scale,
                                      float *scratch) {
  const int oH = out_size(H, kH, dH, padH, 1), oW = out_size(W, kW, dW, padW, 1), oHW = oH * oW, KK = kH * kW;
  float *gwt = scratch, *gbt = gwt + (long)C * M * KK, *col = gbt + (long)C * M, *ones = col + (long)KK * oHW;
  const float one = 1.f;
  refk_transpose01(gw, gwt, M, C, KK);
  if (gb) refk_transpose01(gb, gbt, M, C, 1);
  refk_fill(ones, oHW, 1.f);
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      const float *gy_i = gy + ((long)n * C + c) * M * oHW;
      im2col<float>(0, x + ((long)n * C + c) * H * W, 1, H, W, kH, kW, padH, padW, dH, dW, 1, 1, col);
      REFK_BLAS(cublasSgemm(refk_blas(), CUBLAS_OP_T, CUBLAS_OP_N, KK, M, oHW, &scale, col, oHW, gy_i, oHW, &one,
                            gwt + (long)c * M * KK, KK));
      if (gb) REFK_BLAS(cublasSgemv(refk_blas(), CUBLAS_OP_T, oHW, M, &scale, gy_i, oHW, ones, 1, &one, gbt + (long)c * M, 1));
    }
  refk_transpose01(gwt, gw, C, M, KK);
  if (gb) refk_transpose01(gbt, gb, C, M, 1);
}
