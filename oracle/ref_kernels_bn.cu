/* Test infrastructure: launches the reference's OWN batch-normalisation kernels
 * (lib/THCUNN/BatchNormalization.cu:141-283), compiled from where they lie in the reference tree
 * behind the stand-in headers of ref_shim/.  GPU only (the kernels use shared memory and shuffles).
 *
 * Launch shape as in the reference's host wrapper (lib/THCUNN/generic/BatchNormalization.cu:
 * 54-63,88-92): one block per channel, getNumThreads(H*W) threads, tensors viewed as [N, C, H*W].
 * Absent optional tensors are passed as NULL and become empty views, as devicetensor<>() does (:10-12).
 */
#include "BatchNormalization.cu"

#define REFK_EXPORT extern "C" __attribute__((visibility("default")))

typedef THCDeviceTensor<float, 3> RefkT3;
typedef THCDeviceTensor<float, 1> RefkT1;

static RefkT3 view3(const float *p, int N, int C, int S) {
  if (!p) return RefkT3();
  int size[3] = {N, C, S};
  return RefkT3(const_cast<float *>(p), size);
}
static RefkT1 view1(const float *p, int C) {
  if (!p) return RefkT1();
  int size[1] = {C};
  return RefkT1(const_cast<float *>(p), size);
}

REFK_EXPORT void refk_bn_forward(const float *x, float *y, const float *weight, const float *bias, float *running_mean,
                                 float *running_var, float *save_mean, float *save_std, int N, int C, int S, int train,
                                 double momentum, double eps) {
  dim3 blocks(C), threads(getNumThreads(S));
  if (!train) {
    BatchNormalizationUpdateOutputInference_kernel<float, float, RefkT1, RefkT3><<<blocks, threads>>>(
        view3(x, N, C, S), view3(y, N, C, S), view1(running_mean, C), view1(running_var, C), view1(weight, C),
        view1(bias, C), (float)eps);
  } else {
    BatchNormalizationUpdateOutput_kernel<float, float, RefkT1, RefkT3><<<blocks, threads>>>(
        view3(x, N, C, S), view3(y, N, C, S), view1(weight, C), view1(bias, C), (float)eps, (float)momentum,
        view1(running_mean, C), view1(running_var, C), view1(save_mean, C), view1(save_std, C));
  }
  THCudaCheck(cudaGetLastError());
}

REFK_EXPORT void refk_bn_backward(const float *x, const float *gy, float *gx, float *gw, float *gb, const float *weight,
                                  const float *running_mean, const float *running_var, const float *save_mean,
                                  const float *save_std, int N, int C, int S, int train, double scale, double eps) {
  dim3 blocks(C), threads(getNumThreads(S));
  BatchNormalizationBackward_kernel<float, float, RefkT1, RefkT3><<<blocks, threads>>>(
      view3(x, N, C, S), view3(gy, N, C, S), view3(gx, N, C, S), view1(gw, C), view1(gb, C), view1(weight, C),
      view1(running_mean, C), view1(running_var, C), view1(save_mean, C), view1(save_std, C), train != 0, (float)scale,
      eps);
  THCudaCheck(cudaGetLastError());
}
