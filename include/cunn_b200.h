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

/* Scratch bytes cunn_b200_dwconv_acc_grad needs for these sizes (may be 0). */
CUNN_API size_t cunn_b200_dwconv_acc_grad_workspace(int N, int C, int H, int W, int M, int kH, int kW,
                                           int dH, int dW, int padH, int padW);

/* grad_weight [M,C,kH,kW] += scale * dL/dW, grad_bias [M,C] += scale * sum gy
 * (grad_bias may be NULL).  `workspace` is caller-owned device scratch of at
 * least the size the query above returns, 16-byte aligned.  Its first 64 KiB hold
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

/* Tuning hook for sweeps and tests: overrides the tile plan of the 3x3 fast path for the calling
 * thread.  values[0..count) = {planes_per_tile, rows_per_tile, rows_per_strip, stages, ctas_per_sm,
 * force_generic, stage_budget_kb, vec, staged_stores(-1 auto)}; 0 keeps the automatic choice, missing
 * entries are reset.  force_generic != 0 routes every call to the shape-generic kernels. */
CUNN_API void cunn_b200_dwconv_tuning(const int *values, int count);

/* Writes a one-line description of the tile plan the fast path picks (mode 0 forward, 1 stride-2
 * input gradient, 2 parameter gradient) for a 3x3/pad-1 layer; returns 0 if the fast path applies. */
CUNN_API int cunn_b200_dwconv_describe_plan(int mode, int N, int C, int H, int W, int stride, char *buf, int buflen);

#ifdef __cplusplus
}
#endif
#endif /* CUNN_B200_H */
