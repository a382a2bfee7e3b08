/* Test infrastructure: launches the reference's OWN pooling kernels, compiled from where they lie
 * in the reference tree (lib/THCUNN/SpatialDilatedMaxPooling.cu:8-80 MaxPoolForward / MaxPoolBackward,
 * lib/THCUNN/SpatialAveragePooling.cu:7-82 AvePoolForward / AvePoolBackward) behind the stand-in
 * headers of ref_shim/.  No reference source is copied here; this file only holds launchers.
 *
 * Launch shapes follow the reference's host wrappers: one thread per output element for the
 * forward kernels, one per input element for the backward kernels, 1024-thread blocks
 * (lib/THCUNN/generic/SpatialDilatedMaxPooling.cu:146-152,219-228,
 *  lib/THCUNN/generic/SpatialAveragePooling.cu:140-160,216-236).
 *
 * Built twice (Makefile target `ref`): by nvcc for the GPU (pointers are device pointers) and by
 * g++ -DREFK_CPU, where the kernel is invoked once per index on the host, as one emulated thread each
 * (pointers are host pointers).  Only tests and the benchmark's reference legs load the result.
 */
#include "SpatialDilatedMaxPooling.cu"
#include "SpatialAveragePooling.cu"

#ifdef REFK_CPU
#define REFK_NAME(n) refk_cpu_##n
#define REFK_LAUNCH(kernel, count, ...) \
  do { gridDim.x = (count); for (blockIdx.x = 0; blockIdx.x < (count); ++blockIdx.x) kernel(__VA_ARGS__); } while (0)
#else
#define REFK_NAME(n) refk_##n
#define REFK_LAUNCH(kernel, count, ...) \
  do { kernel<<<GET_BLOCKS(count), CUDA_NUM_THREADS>>>(__VA_ARGS__); THCudaCheck(cudaGetLastError()); } while (0)
#endif

#define REFK_EXPORT extern "C" __attribute__((visibility("default")))

REFK_EXPORT void REFK_NAME(maxpool_forward)(const float *x, float *y, long *ind, int N, int C, int H, int W, int oH,
                                            int oW, int kH, int kW, int dH, int dW, int padH, int padW, int dilH,
                                            int dilW) {
  int count = N * C * oH * oW;
  if (count == 0) return;
  REFK_LAUNCH((MaxPoolForward<float, float>), count, count, x, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH,
              dilW, y, ind);
}

REFK_EXPORT void REFK_NAME(maxpool_backward)(const float *gy, const long *ind, float *gx, int N, int C, int H, int W,
                                             int oH, int oW, int kH, int kW, int dH, int dW, int padH, int padW,
                                             int dilH, int dilW) {
  int count = N * C * H * W;
  if (count == 0) return;
  REFK_LAUNCH((MaxPoolBackward<float, float>), count, count, gy, ind, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW,
              dilH, dilW, gx);
}

REFK_EXPORT void REFK_NAME(avgpool_forward)(const float *x, float *y, int N, int C, int H, int W, int oH, int oW,
                                            int kH, int kW, int dH, int dW, int padH, int padW, int include_pad) {
  int count = N * C * oH * oW;
  if (count == 0) return;
  if (include_pad)
    REFK_LAUNCH((AvePoolForward<float, float, true>), count, count, x, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, y);
  else
    REFK_LAUNCH((AvePoolForward<float, float, false>), count, count, x, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, y);
}

REFK_EXPORT void REFK_NAME(avgpool_backward)(const float *gy, float *gx, int N, int C, int H, int W, int oH, int oW,
                                             int kH, int kW, int dH, int dW, int padH, int padW, int include_pad) {
  int count = N * C * H * W;
  if (count == 0) return;
  if (include_pad)
    REFK_LAUNCH((AvePoolBackward<float, float, true>), count, count, gy, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, gx);
  else
    REFK_LAUNCH((AvePoolBackward<float, float, false>), count, count, gy, N, C, H, W, oH, oW, kH, kW, dH, dW, padH, padW, gx);
}

REFK_EXPORT int REFK_NAME(index_base)(void) { return TH_INDEX_BASE; }
