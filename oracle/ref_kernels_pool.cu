/* Test infrastructure: launches the reference's OWN pooling kernels, compiled from where they lie
 * in the reference tree (lib/THCUNN/SpatialDilatedMaxPooling.cu:8-80 MaxPoolForward / MaxPoolBackward,
 * lib/THCUNN/SpatialAveragePooling.cu:7-82 AvePoolForward / AvePoolBackward,
 * lib/THCUNN/SpatialAdaptiveMaxPooling.cu:15-176 and SpatialAdaptiveAveragePooling.cu:16-190) behind the stand-in
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
#include "SpatialAdaptiveMaxPooling.cu"
#include "SpatialAdaptiveAveragePooling.cu"

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

/* Adaptive pooling: one block per plane (generic/SpatialAdaptiveMaxPooling.cu:39-50, :121-141; the wrappers always
 * take the atomic backward kernels).  indices: [2, planes, oH, oW], row offsets first (the wrapper passes the second
 * half as indices_x).  gx must be zero on entry, as the wrappers zero gradInput before the launch. */
#ifdef REFK_CPU
#define REFK_LAUNCH_PLANES(kernel, planes, ...) REFK_LAUNCH(kernel, planes, __VA_ARGS__)
#else
#define REFK_LAUNCH_PLANES(kernel, planes, ...) \
  do { int yb = 16 / (planes); if (yb < 1) yb = 1; kernel<<<dim3(planes, yb), dim3(32, 8)>>>(__VA_ARGS__); THCudaCheck(cudaGetLastError()); } while (0)
#endif

REFK_EXPORT void REFK_NAME(adaptive_maxpool_forward)(float *x, float *y, long *ind, int planes, int H, int W, int oH, int oW) {
  if (planes == 0) return;
  REFK_LAUNCH_PLANES((adaptivemaxpool<float>), planes, x, y, ind + (long)planes * oH * oW, ind, planes, H, W, oH, oW, W, 1, H * W);
}
REFK_EXPORT void REFK_NAME(adaptive_maxpool_backward)(float *gx, float *gy, long *ind, int planes, int H, int W, int oH, int oW) {
  if (planes == 0) return;
  REFK_LAUNCH_PLANES((atomicadaptivemaxgradinput<float>), planes, gx, gy, ind + (long)planes * oH * oW, ind, planes, H, W, oH, oW);
}
REFK_EXPORT void REFK_NAME(adaptive_avgpool_forward)(float *x, float *y, int planes, int H, int W, int oH, int oW) {
  if (planes == 0) return;
  REFK_LAUNCH_PLANES((adaptiveaveragepool<float>), planes, x, y, planes, H, W, oH, oW, W, 1, H * W);
}
REFK_EXPORT void REFK_NAME(adaptive_avgpool_backward)(float *gx, float *gy, int planes, int H, int W, int oH, int oW) {
  if (planes == 0) return;
  REFK_LAUNCH_PLANES((atomicadaptiveaveragegradinput<float>), planes, gx, gy, planes, H, W, oH, oW);
}

REFK_EXPORT int REFK_NAME(index_base)(void) { return TH_INDEX_BASE; }
