/*
 * cunn_b200 — flat C ABI of the B200 (sm_100a) kernels behind the THCUNN
 * convolutional hot path.
 *
 * Every function takes plain device pointers, sizes and a CUDA stream
 * (`cudaStream_t` passed as `void*`), enqueues its work on that stream and
 * returns without synchronising.  Return value: 0 on success, non-zero on a
 * rejected argument or a failed launch; `cunn_b200_last_error()` then holds
 * the message for the calling thread.  All tensors are contiguous fp32 NCHW
 * unless stated; indices are int64.  There is no CPU fallback: without a
 * CUDA device every compute entry point fails.
 *
 * The `THNN_Cuda*` entry points that the reference's LuaJIT FFI binds
 * (declared in THCUNN_b200.h) are thin tensor-struct wrappers over these.
 */
#ifndef CUNN_B200_H
#define CUNN_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(CUNN_BUILDING)
#define CUNN_API __attribute__((visibility("default")))
#else
#define CUNN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef void *cunn_stream_t; /* a cudaStream_t */

/* Index base added to stored max-pool indices and expected of class targets
 * (TH_INDEX_BASE of the Lua build: lib/THCUNN/SpatialDilatedMaxPooling.cu:40). */
#define CUNN_B200_INDEX_BASE 1

/* Message of the last failure on the calling thread ("" if none). */
CUNN_API const char *cunn_b200_last_error(void);

/* Device-side status word of the current device: 0 = healthy.  Kernels that
 * give up on a bounded wait record a non-zero code here instead of hanging.
 * Synchronises the device. */
CUNN_API int cunn_b200_device_status(void);

/* ---- SpatialDepthWiseConvolution --------------------------------------------
 * x [N,C,H,W]; weight [M,C,kH,kW]; bias [M,C] or NULL; y [N,C*M,oH,oW] with
 * output channel c*M+j; oH = (H+2padH-kH)/dH+1.
 * Replaces THNN_(SpatialDepthWiseConvolution_updateOutput)
 * (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:58-261). */
CUNN_API int cunn_b200_dwconv_forward(const float *x, const float *weight, const float *bias, float *y,
                             int N, int C, int H, int W, int M, int kH, int kW,
                             int dH, int dW, int padH, int padW, cunn_stream_t stream);

/* gx [N,C,H,W] from gy [N,C*M,oH,oW].  Replaces ..._updateGradInput
 * (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:263-416). */
CUNN_API int cunn_b200_dwconv_grad_input(const float *gy, const float *weight, float *gx,
                                int N, int C, int H, int W, int M, int kH, int kW,
                                int dH, int dW, int padH, int padW, cunn_stream_t stream);

/* How parameter gradients are summed across thread blocks, process-wide.  0 (default): fp32 atomic adds — the
 * fastest, but the rounding of the last bits depends on scheduling.  1: a fixed-order reduction through the
 * caller's workspace — bit-reproducible from run to run, a few microseconds slower per call. */
CUNN_API void cunn_b200_set_deterministic(int on);
CUNN_API int cunn_b200_get_deterministic(void);

/* Scratch bytes cunn_b200_dwconv_acc_grad needs for these sizes in deterministic mode (may be 0). */
CUNN_API size_t cunn_b200_dwconv_acc_grad_workspace(int N, int C, int H, int W, int M, int kH, int kW,
                                           int dH, int dW, int padH, int padW);

/* grad_weight [M,C,kH,kW] += scale * dL/dW, grad_bias [M,C] += scale * sum gy
 * (grad_bias may be NULL).  `workspace` (used in deterministic mode only) is caller-owned device scratch
 * of at least the size the query above returns, 16-byte aligned.  Its first 64 KiB hold
 * ticket counters: the buffer must be zero-filled once before its first use
 * (cudaMemset) and every call leaves the counters zero again, so one buffer can
 * serve all later calls that do not overlap on the GPU.  Replaces
 * ..._accGradParameters (lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:418-650). */
CUNN_API int cunn_b200_dwconv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                              int N, int C, int H, int W, int M, int kH, int kW,
                              int dH, int dW, int padH, int padW, float scale,
                              void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* Parameter gradient for callers that cannot supply scratch memory.  It has no counterpart in the
 * reference.  Same arguments and result as cunn_b200_dwconv_acc_grad minus the workspace: the scratch is
 * a fixed 4 MiB array inside the library (resident on every GPU that loads it, until exit), so the call
 * performs no cudaMalloc, cudaFree or other allocation.  It exists for hosts that have no allocator to
 * offer: a program whose own arena already owns all device memory, or a pass-through binding whose
 * signature carries tensors only.  Shapes whose scratch would exceed the array are rejected with an error
 * naming both sizes (cunn_b200_dwconv_acc_grad_static_capacity() returns the limit); shapes outside the
 * 3x3 fast path need no scratch and are accepted.  The first call on each device looks up the array's
 * device address (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls on
 * a device share the one array: calls that may overlap on the GPU (different streams without an ordering
 * between them) race on it and must be serialised by the caller. */
CUNN_API int cunn_b200_dwconv_acc_grad_static(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                              int N, int C, int H, int W, int M, int kH, int kW,
                                              int dH, int dW, int padH, int padW, float scale,
                                              cunn_stream_t stream);
CUNN_API size_t cunn_b200_dwconv_acc_grad_static_capacity(void);

/* ---- SpatialConvolutionMM -----------------------------------------------------
 * x [N,C,H,W]; weight [K, C*kH*kW] (= contiguous [K,C,kH,kW]); bias [K] or NULL; y [N,K,oH,oW].
 * Implicit GEMM on tcgen05 tensor cores with a 3xTF32 split (fp32-class accuracy); no column buffer.
 * Replaces THNN_(SpatialConvolutionMM_updateOutput)
 * (lib/THCUNN/generic/SpatialConvolutionMM.cu:58-209, unfold kernel lib/THCUNN/im2col.h:10-61). */
CUNN_API int cunn_b200_convmm_forward(const float *x, const float *weight, const float *bias, float *y,
                                      int N, int C, int H, int W, int K, int kH, int kW,
                                      int dH, int dW, int padH, int padW, cunn_stream_t stream);

/* gx [N,C,H,W] from gy [N,K,oH,oW].  Replaces ..._updateGradInput
 * (lib/THCUNN/generic/SpatialConvolutionMM.cu:211-325, fold kernel lib/THCUNN/im2col.h:64-121). */
CUNN_API int cunn_b200_convmm_grad_input(const float *gy, const float *weight, float *gx,
                                         int N, int C, int H, int W, int K, int kH, int kW,
                                         int dH, int dW, int padH, int padW, cunn_stream_t stream);

/* grad_weight [K, C*kH*kW] += scale * dL/dW, grad_bias [K] += scale * sum gy (may be NULL).  `workspace`:
 * caller-owned scratch of at least cunn_b200_convmm_acc_grad_workspace(...) bytes, 16-byte aligned,
 * contents irrelevant.  Replaces ..._accGradParameters
 * (lib/THCUNN/generic/SpatialConvolutionMM.cu:327-486). */
CUNN_API size_t cunn_b200_convmm_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW,
                                                    int dH, int dW, int padH, int padW);
CUNN_API int cunn_b200_convmm_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                       int N, int C, int H, int W, int K, int kH, int kW,
                                       int dH, int dW, int padH, int padW, float scale,
                                       void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* 1x1 stride-1 convolutions on 16-byte aligned tensors with H*W and C multiples of 4 fetch their operand tiles with
 * tensor-map (TMA) copies; everything else, and every shape after cunn_b200_convmm_set_tma(0), uses the element-copy
 * loader.  Results are identical; the switch exists so that both loaders can be tested and timed.  No reference
 * counterpart. */
CUNN_API void cunn_b200_convmm_set_tma(int on);
CUNN_API int cunn_b200_convmm_get_tma(void);

/* ---- SpatialDilatedConvolution -------------------------------------------------
 * The same three passes with the kernel taps dilH x dilW apart: output size
 * (in + 2 pad - (dil (k - 1) + 1)) / stride + 1 (lib/THCUNN/generic/SpatialDilatedConvolution.cu:49-50).
 * Kernels of up to 32 taps; dilation 1 is SpatialConvolutionMM.  Replaces
 * THNN_(SpatialDilatedConvolution_updateOutput / _updateGradInput / _accGradParameters)
 * (lib/THCUNN/generic/SpatialDilatedConvolution.cu:88-200, 202-300, 302-450; decl generic/THCUNN.h:727-764). */
CUNN_API int cunn_b200_dilated_conv_forward(const float *x, const float *weight, const float *bias, float *y,
                                            int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                            int padH, int padW, int dilH, int dilW, cunn_stream_t stream);
CUNN_API int cunn_b200_dilated_conv_grad_input(const float *gy, const float *weight, float *gx,
                                               int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                               int padH, int padW, int dilH, int dilW, cunn_stream_t stream);
CUNN_API size_t cunn_b200_dilated_conv_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW,
                                                          int dH, int dW, int padH, int padW, int dilH, int dilW);
CUNN_API int cunn_b200_dilated_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                             int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                             int padH, int padW, int dilH, int dilW, float scale,
                                             void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* ---- SpatialFullDilatedConvolution (transposed convolution) ----------------------
 * x [N,P,H,W], weight [P,Q,kH,kW], bias [Q] or NULL -> y [N,Q,OH,OW] with
 * OH = (H-1)*dH - 2*padH + dilH*(kH-1) + 1 + adjH (adjH < dH required here; the reference also admits
 * adjH < dilH).  Runs on the kernels of the convolution it is the adjoint of: forward = that convolution's
 * input gradient plus bias, input gradient = its forward, parameter gradient = its parameter gradient with
 * activations and output gradient exchanged; dilation 1 is SpatialFullConvolution.  acc_grad accumulates
 * (+= scale * g) and needs cunn_b200_full_conv_acc_grad_workspace(...) bytes of 16-byte aligned scratch.
 * Replaces THNN_(SpatialFullDilatedConvolution_updateOutput / _updateGradInput / _accGradParameters)
 * (lib/THCUNN/generic/SpatialFullDilatedConvolution.cu:68-209, 211-317, 319-461; decl generic/THCUNN.h:766-806)
 * and THNN_(SpatialFullConvolution_*) (lib/THCUNN/generic/SpatialFullConvolution.cu). */
CUNN_API int cunn_b200_full_conv_forward(const float *x, const float *weight, const float *bias, float *y,
                                         int N, int P, int H, int W, int Q, int kH, int kW, int dH, int dW,
                                         int padH, int padW, int dilH, int dilW, int adjH, int adjW,
                                         cunn_stream_t stream);
CUNN_API int cunn_b200_full_conv_grad_input(const float *gy, const float *weight, float *gx,
                                            int N, int P, int H, int W, int Q, int kH, int kW, int dH, int dW,
                                            int padH, int padW, int dilH, int dilW, int adjH, int adjW,
                                            cunn_stream_t stream);
CUNN_API size_t cunn_b200_full_conv_acc_grad_workspace(int N, int P, int H, int W, int Q, int kH, int kW,
                                                       int dH, int dW, int padH, int padW, int dilH, int dilW,
                                                       int adjH, int adjW);
CUNN_API int cunn_b200_full_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                          int N, int P, int H, int W, int Q, int kH, int kW, int dH, int dW,
                                          int padH, int padW, int dilH, int dilW, int adjH, int adjW, float scale,
                                          void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* ---- SpatialMaxPooling --------------------------------------------------------
 * x [N,C,H,W] -> y [N,C,oH,oW] and int64 indices of the same shape holding the flat position h*W + w of
 * the maximum inside its plane plus CUNN_B200_INDEX_BASE.  The window is scanned row-major with a strict
 * "greater than" from -FLT_MAX / index -1, as in the reference, so indices are reproducible bit for bit.
 * oH, oW = cunn_b200_maxpool_out_size(...) (floor or ceil mode with the reference's fix-up that the last
 * window must start inside the padded input).  Requires pad <= k/2.
 * Replaces THNN_(SpatialMaxPooling_updateOutput) -> THNN_(SpatialDilatedMaxPooling_updateOutput)
 * (lib/THCUNN/generic/SpatialMaxPooling.cu:7-21, generic/SpatialDilatedMaxPooling.cu:84-158; kernel
 * lib/THCUNN/SpatialDilatedMaxPooling.cu:8-42). */
CUNN_API int cunn_b200_maxpool_out_size(int in, int k, int d, int pad, int dil, int ceil_mode);
CUNN_API int cunn_b200_maxpool_forward(const float *x, float *y, int64_t *indices, int N, int C, int H, int W,
                                       int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW,
                                       int ceil_mode, cunn_stream_t stream);

/* gx [N,C,H,W]: every input pixel receives the sum of gy over the outputs whose index names it (gather
 * form, deterministic).  Replaces THNN_(SpatialMaxPooling_updateGradInput)
 * (lib/THCUNN/generic/SpatialMaxPooling.cu:23-38, generic/SpatialDilatedMaxPooling.cu:160-235; kernel
 * lib/THCUNN/SpatialDilatedMaxPooling.cu:46-80). */
CUNN_API int cunn_b200_maxpool_backward(const float *gy, const int64_t *indices, float *gx, int N, int C, int H, int W,
                                        int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW,
                                        int ceil_mode, cunn_stream_t stream);

/* ---- BatchNormalization over [N, C, S] (S = product of the trailing dimensions) ----------------
 * Training (train != 0): per-channel batch mean and biased variance; y = gamma (x - mean) invstd + beta;
 * save_mean = mean, save_std = invstd = 1/sqrt(var + eps); running_mean/var updated with `momentum`,
 * running_var from the UNBIASED variance.  Inference: uses the running statistics and leaves them alone.
 * weight / bias may be NULL (gamma = 1, beta = 0).  `workspace`: caller-owned scratch of at least
 * cunn_b200_batchnorm_workspace(N, C) bytes, 16-byte aligned.  Its first cunn_b200_batchnorm_counter_bytes()
 * bytes hold per-channel ticket counters and ready flags (the CTA that hands in a channel's last partial sum
 * finishes the channel; large tensors are reduced and normalised group by group inside one launch so that the
 * second read comes from L2): they must be zero when a call is enqueued and every call leaves them zero, so zero
 * the buffer once and let no other operator write there; the rest of the buffer needs no initialisation.  If
 * cunn_b200_device_status() ever reports a wait that ran out, zero the counters again before the next call.
 * Replaces THNN_(BatchNormalization_updateOutput) (lib/THCUNN/generic/BatchNormalization.cu:34-66,
 * kernels lib/THCUNN/BatchNormalization.cu:141-212). */
CUNN_API size_t cunn_b200_batchnorm_workspace(int N, int C);
CUNN_API size_t cunn_b200_batchnorm_counter_bytes(void);
/* Which shapes take the one-launch, group-by-group kernels (statistics and normalisation of a group of channels
 * back to back, so that the second read of the group comes from L2).  0: none; 1 (default): the training forward
 * pass when a channel's N planes are at least 6 MB and two such slabs fit the L2 window; 2: every shape they
 * apply to, forward and backward.  Results do not depend on the mode beyond rounding.  Process-wide. */
CUNN_API void cunn_b200_batchnorm_set_grouped(int mode);
CUNN_API int cunn_b200_batchnorm_get_grouped(void);
CUNN_API int cunn_b200_batchnorm_forward(const float *x, float *y, const float *weight, const float *bias,
                                         float *running_mean, float *running_var, float *save_mean, float *save_std,
                                         int N, int C, int S, int train, double momentum, double eps,
                                         void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* Backward: gx (may be NULL), grad_weight += scale * sum gy (x - mean) invstd, grad_bias += scale * sum gy
 * (either may be NULL).  Training mode uses save_mean / save_std, inference mode the running statistics.
 * Replaces THNN_(BatchNormalization_backward) (lib/THCUNN/generic/BatchNormalization.cu:68-94, kernel
 * lib/THCUNN/BatchNormalization.cu:215-283). */
CUNN_API int cunn_b200_batchnorm_backward(const float *x, const float *gy, float *gx, float *grad_weight,
                                          float *grad_bias, const float *weight, const float *running_mean,
                                          const float *running_var, const float *save_mean, const float *save_std,
                                          int N, int C, int S, int train, double scale, double eps,
                                          void *workspace, size_t workspace_bytes, cunn_stream_t stream);

/* BatchNormalization followed by ReLU in one pass (y = max(0, BN(x))), and its backward: the caller-side
 * fusion of nn.SpatialBatchNormalization + nn.ReLU, which saves two full activation passes per layer in each
 * direction.  The backward needs x, the affine parameters and the statistics only: it recomputes the sign of
 * BN(x) with the forward's exact arithmetic instead of reading y.  No counterpart in the reference (it runs
 * BatchNormalization.cu and Threshold.cu as separate kernels); results equal the two separate calls exactly. */
CUNN_API int cunn_b200_batchnorm_relu_forward(const float *x, float *y, const float *weight, const float *bias,
                                              float *running_mean, float *running_var, float *save_mean, float *save_std,
                                              int N, int C, int S, int train, double momentum, double eps,
                                              void *workspace, size_t workspace_bytes, cunn_stream_t stream);
CUNN_API int cunn_b200_batchnorm_relu_backward(const float *x, const float *gy, float *gx, float *grad_weight,
                                               float *grad_bias, const float *weight, const float *bias,
                                               const float *running_mean, const float *running_var,
                                               const float *save_mean, const float *save_std, int N, int C, int S,
                                               int train, double scale, double eps, void *workspace,
                                               size_t workspace_bytes, cunn_stream_t stream);

/* ---- Support operators of the MobileNetV1 step ---------------------------------------------
 * Threshold (ReLU is threshold 0, value 0; y may alias x, gx may alias gy):
 * THNN_(Threshold_updateOutput / _updateGradInput), lib/THCUNN/generic/Threshold.cu:7-67. */
CUNN_API int cunn_b200_threshold_forward(const float *x, float *y, long long n, float threshold, float value,
                                         cunn_stream_t stream);
CUNN_API int cunn_b200_threshold_backward(const float *x, const float *gy, float *gx, long long n, float threshold,
                                          cunn_stream_t stream);

/* SpatialAveragePooling with caller-computed output size (cunn_b200_maxpool_out_size with dil = 1 gives it):
 * THNN_(SpatialAveragePooling_updateOutput / _updateGradInput), lib/THCUNN/generic/SpatialAveragePooling.cu:72-235. */
CUNN_API int cunn_b200_avgpool_forward(const float *x, float *y, int N, int C, int H, int W, int oH, int oW,
                                       int kH, int kW, int dH, int dW, int padH, int padW, int count_include_pad,
                                       cunn_stream_t stream);
CUNN_API int cunn_b200_avgpool_backward(const float *gy, float *gx, int N, int C, int H, int W, int oH, int oW,
                                        int kH, int kW, int dH, int dW, int padH, int padW, int count_include_pad,
                                        cunn_stream_t stream);

/* LogSoftMax over the last dimension of [B, D]:
 * THNN_(LogSoftMax_updateOutput / _updateGradInput), lib/THCUNN/generic/LogSoftMax.cu:7-237. */
CUNN_API int cunn_b200_logsoftmax_forward(const float *x, float *y, int B, int D, cunn_stream_t stream);
CUNN_API int cunn_b200_logsoftmax_backward(const float *y, const float *gy, float *gx, int B, int D, cunn_stream_t stream);

/* ClassNLLCriterion on log-probabilities [B, D]; targets are int64 and carry CUNN_B200_INDEX_BASE;
 * loss_and_total_weight[0] = loss, [1] = total weight (device memory).  Backward writes only the target
 * entries of gx: zero gx first, as nn.ClassNLLCriterion does.
 * THNN_(ClassNLLCriterion_updateOutput / _updateGradInput), lib/THCUNN/generic/ClassNLLCriterion.cu:5-177. */
CUNN_API int cunn_b200_classnll_forward(const float *logprob, const int64_t *target, const float *weights,
                                        float *loss_and_total_weight, int B, int D, int size_average,
                                        long long ignore_index, cunn_stream_t stream);
CUNN_API int cunn_b200_classnll_backward(const int64_t *target, const float *weights, const float *total_weight,
                                         float *gx, int B, int D, int size_average, long long ignore_index,
                                         cunn_stream_t stream);

/* params -= lr * grads: the update DataParallelTable:updateParameters applies (DataParallelTable.lua:315-321). */
CUNN_API int cunn_b200_sgd_update(float *params, const float *grads, long long n, float lr, cunn_stream_t stream);

CUNN_API int cunn_b200_fill(float *p, long long n, float value, cunn_stream_t stream);

/* ---- MobileNetV1 replica step (the module a batch-sharded DataParallelTable replicates) ----------
 * image_hw: input resolution (224), width_div: channel divisor (1 = full width; 2, 4, 8 ... for tests),
 * num_classes: classifier outputs.  Parameters and gradients are flat fp32 buffers of
 * cunn_b200_mobilenet_param_count() floats in module order (DataParallelTable.lua:104-128 flattenParameters);
 * cunn_b200_mobilenet_layer_info() gives every tensor's offset.  bn_running holds running mean | var per
 * layer (cunn_b200_mobilenet_bn_stat_count() floats) and stays per replica.  One call runs forward, loss
 * and backward on `batch` local images and ACCUMULATES parameter gradients of
 * (1 / global batch) * sum of the local rows' NLL into `grads`; *loss (device) receives that scaled sum, so
 * replica losses and gradients simply add up (the data-parallel step all-reduces `grads`).  The arena is
 * caller-owned device memory of cunn_b200_mobilenet_arena_bytes() bytes, 256-byte aligned. */
typedef struct cunn_b200_mobilenet_config {
    int image_hw;
    int width_div;
    int num_classes;
} cunn_b200_mobilenet_config;
CUNN_API long long cunn_b200_mobilenet_param_count(const cunn_b200_mobilenet_config *cfg);
CUNN_API long long cunn_b200_mobilenet_bn_stat_count(const cunn_b200_mobilenet_config *cfg);
CUNN_API int cunn_b200_mobilenet_num_layers(const cunn_b200_mobilenet_config *cfg);
CUNN_API int cunn_b200_mobilenet_layer_info(const cunn_b200_mobilenet_config *cfg, int layer, long long *info12);
CUNN_API size_t cunn_b200_mobilenet_arena_bytes(const cunn_b200_mobilenet_config *cfg, int batch);
CUNN_API int cunn_b200_mobilenet_step(const cunn_b200_mobilenet_config *cfg, const float *images, const int64_t *labels,
                                      int batch, float inv_global_batch, const float *params, float *grads,
                                      float *bn_running, void *arena, size_t arena_bytes, float *loss,
                                      double momentum, double eps, cunn_stream_t stream);

/* ---- SpatialConvolutionLocal: convolution with weights that are not shared between output positions ----------
 * weight [oH*oW, K, C*kH*kW] (the reference's 3-D view of its 6-D [oH, oW, K, C, kH, kW] weight,
 * lib/THCUNN/generic/SpatialConvolutionLocal.cu:58-77), bias [K, oH, oW] or NULL, x [N, C, H, W], y [N, K, oH, oW];
 * oH, oW must be the sizes that follow from H, W, kernel, stride and padding.  acc_grad accumulates with `scale`.
 * Replace THNN_(SpatialConvolutionLocal_updateOutput / _updateGradInput / _accGradParameters) (:79-407). */
CUNN_API int cunn_b200_local_conv_forward(const float *x, const float *weight, const float *bias, float *y, int N, int C, int H, int W,
                                          int K, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW,
                                          cunn_stream_t stream);
CUNN_API int cunn_b200_local_conv_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H, int W, int K, int kH,
                                             int kW, int dH, int dW, int padH, int padW, int oH, int oW, cunn_stream_t stream);
CUNN_API int cunn_b200_local_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias, int N, int C, int H,
                                           int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW,
                                           float scale, cunn_stream_t stream);

/* ---- SpatialAdaptiveMaxPooling / SpatialAdaptiveAveragePooling over `planes` = N*C planes of H x W --------------
 * Output size oH x oW is given; the window of output row i is [floor(i/oH*H), ceil((i+1)/oH*H)) in the float
 * arithmetic of the reference kernels.  Max pooling stores TWO index planes, indices [2, planes, oH, oW]: first the
 * row, then the column of the maximum RELATIVE to the window start, plus CUNN_B200_INDEX_BASE (first maximum wins,
 * strict compare from -FLT_MAX).  The backward passes are gathers (deterministic; the reference adds atomically).
 * Replace THNN_(SpatialAdaptiveMaxPooling_*) (lib/THCUNN/SpatialAdaptiveMaxPooling.cu:15-176, generic/...:7-190) and
 * THNN_(SpatialAdaptiveAveragePooling_*) (lib/THCUNN/SpatialAdaptiveAveragePooling.cu:6-190, generic/...:7-170). */
CUNN_API int cunn_b200_adaptive_maxpool_forward(const float *x, float *y, int64_t *indices, int planes, int H, int W, int oH, int oW,
                                                cunn_stream_t stream);
CUNN_API int cunn_b200_adaptive_maxpool_backward(const float *gy, const int64_t *indices, float *gx, int planes, int H, int W, int oH,
                                                 int oW, cunn_stream_t stream);
CUNN_API int cunn_b200_adaptive_avgpool_forward(const float *x, float *y, int planes, int H, int W, int oH, int oW, cunn_stream_t stream);
CUNN_API int cunn_b200_adaptive_avgpool_backward(const float *gy, float *gx, int planes, int H, int W, int oH, int oW,
                                                 cunn_stream_t stream);

/* ---- fp64 twins of the hot path -----------------------------------------------------------------------
 * The operators above for double tensors, behind THNN_CudaDouble* (the reference instantiates every entry point
 * for float and double: lib/THCUNN/SpatialDepthWiseConvolution.cu:9, SpatialConvolutionMM.cu:9,
 * BatchNormalization.cu:285-286, SpatialDilatedMaxPooling.cu:82-83 include THCGenerateFloatTypes.h; `accreal`
 * is double, THCUNN.lua:54).  Same argument meaning, layouts, accumulate semantics and error behaviour; plain fp64
 * CUDA-core kernels of any shape (the convolution is an implicit GEMM on the fp64 FMA pipes).  The
 * parameter-gradient calls need no scratch (their workspace queries return 0 and the arguments are ignored);
 * batch norm needs cunn_b200_double_batchnorm_workspace(N, C) bytes whose contents are irrelevant. */
CUNN_API int cunn_b200_double_dwconv_forward(const double *x, const double *weight, const double *bias, double *y, int N, int C,
                                             int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                             cunn_stream_t stream);
CUNN_API int cunn_b200_double_dwconv_grad_input(const double *gy, const double *weight, double *gx, int N, int C, int H, int W,
                                                int M, int kH, int kW, int dH, int dW, int padH, int padW, cunn_stream_t stream);
CUNN_API size_t cunn_b200_double_dwconv_acc_grad_workspace(int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW,
                                                           int padH, int padW);
CUNN_API int cunn_b200_double_dwconv_acc_grad(const double *x, const double *gy, double *grad_weight, double *grad_bias, int N,
                                              int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                              double scale, void *workspace, size_t workspace_bytes, cunn_stream_t stream);
CUNN_API int cunn_b200_double_convmm_forward(const double *x, const double *weight, const double *bias, double *y, int N, int C,
                                             int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                             cunn_stream_t stream);
CUNN_API int cunn_b200_double_convmm_grad_input(const double *gy, const double *weight, double *gx, int N, int C, int H, int W,
                                                int K, int kH, int kW, int dH, int dW, int padH, int padW, cunn_stream_t stream);
CUNN_API size_t cunn_b200_double_convmm_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                                           int padH, int padW);
CUNN_API int cunn_b200_double_convmm_acc_grad(const double *x, const double *gy, double *grad_weight, double *grad_bias, int N,
                                              int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                              double scale, void *workspace, size_t workspace_bytes, cunn_stream_t stream);
CUNN_API size_t cunn_b200_double_batchnorm_workspace(int N, int C);
CUNN_API int cunn_b200_double_batchnorm_forward(const double *x, double *y, const double *weight, const double *bias,
                                                double *running_mean, double *running_var, double *save_mean, double *save_std,
                                                int N, int C, int S, int train, double momentum, double eps, void *workspace,
                                                size_t workspace_bytes, cunn_stream_t stream);
CUNN_API int cunn_b200_double_batchnorm_backward(const double *x, const double *gy, double *gx, double *grad_weight,
                                                 double *grad_bias, const double *weight, const double *running_mean,
                                                 const double *running_var, const double *save_mean, const double *save_std, int N,
                                                 int C, int S, int train, double scale, double eps, void *workspace,
                                                 size_t workspace_bytes, cunn_stream_t stream);
CUNN_API int cunn_b200_double_maxpool_forward(const double *x, double *y, int64_t *indices, int N, int C, int H, int W, int kH,
                                              int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int ceil_mode,
                                              cunn_stream_t stream);
CUNN_API int cunn_b200_double_maxpool_backward(const double *gy, const int64_t *indices, double *gx, int N, int C, int H, int W,
                                               int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int ceil_mode,
                                               cunn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CUNN_B200_H */
