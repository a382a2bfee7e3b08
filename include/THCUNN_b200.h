/*
 * THNN_Cuda* entry points of libTHCUNN.so — the symbols the reference's LuaJIT FFI binding looks up
 * (THCUNN.lua:129-138) — for the convolutional hot path, with the reference's signatures
 * (lib/THCUNN/generic/THCUNN.h).  `accreal` is `float` for the Cuda type (THCUNN.lua:48).
 *
 * The tensor and storage structs restate the public layout of cutorch 1.0's THCTensor.h / THCStorage.h.
 * cutorch is not part of the reference tree and is absent from this image, so binary compatibility with
 * a real Lua-Torch install could not be verified; inside a cutorch build compile the library with
 * -DCUNN_B200_USE_REAL_THC: this header then includes cutorch's <THC/THC.h> and the entry points reach
 * the state and the tensors through libTHC (csrc/thc_backend_real.inc) instead of the structs below.
 *
 * The small THCudaTensor_* / THCState_* helper set below is what a C harness needs to drive the entry
 * points without cutorch; it is not a reimplementation of libTHC.
 */
#ifndef THCUNN_B200_H
#define THCUNN_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "cunn_b200.h"

#ifdef CUNN_B200_USE_REAL_THC
#include <THC/THC.h>   /* cutorch's THCState, THCudaTensor, THCudaLongTensor */
#endif

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CUNN_B200_USE_REAL_THC
typedef struct THCudaStorage {
    void *data;                 /* float* (THCudaStorage) or long* (THCudaLongStorage) */
    ptrdiff_t size;             /* elements */
    int refcount;
    char flag;
    void *allocator;
    void *allocatorContext;
    struct THCudaStorage *view;
    int device;
} THCudaStorage;

typedef struct THCudaTensor {
    long *size;
    long *stride;
    int nDimension;
    THCudaStorage *storage;
    ptrdiff_t storageOffset;
    int refcount;
    char flag;
} THCudaTensor;

typedef THCudaTensor THCudaLongTensor;   /* same layout, 8-byte elements */
typedef THCudaTensor THCudaDoubleTensor; /* same layout, 8-byte elements */
typedef struct THCState THCState;        /* opaque here: current stream, error hook, scratch */
#endif

/* ---- harness helpers (built-in tensor layer only) ------------------------------------------------- */
#ifndef CUNN_B200_USE_REAL_THC
CUNN_API THCState *THCState_b200_new(void);
CUNN_API void THCState_b200_free(THCState *state);
CUNN_API void THCState_b200_setStream(THCState *state, cunn_stream_t stream);
/* Error hook, the counterpart of TH's THError handler.  Argument and launch errors are reported through it
 * (under Lua it raises a Lua error and does not return).  If it returns, the entry point returns at once.
 * The default hook prints the message to stderr. */
typedef void (*THCUNN_b200_error_fn)(const char *msg, void *ctx);
CUNN_API void THCState_b200_setErrorHandler(THCState *state, THCUNN_b200_error_fn fn, void *ctx);
CUNN_API const char *THCState_b200_lastError(THCState *state);

CUNN_API THCudaTensor *THCudaTensor_b200_new(THCState *state);                    /* empty, 0 dimensions */
CUNN_API THCudaLongTensor *THCudaLongTensor_b200_new(THCState *state);
/* A tensor over caller-owned device memory (never freed or reallocated by the library; a resize that does
 * not fit raises an error).  sizes/strides in elements; strides == NULL means contiguous; `data` is the
 * start of the storage and the view begins storage_offset_elems elements into it. */
CUNN_API THCudaTensor *THCudaTensor_b200_wrap(THCState *state, void *data, ptrdiff_t capacity_elems, int ndim,
                                              const long *sizes, const long *strides, int elem_size,
                                              ptrdiff_t storage_offset_elems);
CUNN_API void THCudaTensor_b200_free(THCState *state, THCudaTensor *t);
/* Device address of the view's first element (storage data + storageOffset * elem_size bytes). */
CUNN_API void *THCudaTensor_b200_data(THCState *state, THCudaTensor *t, int elem_size);
#endif

/* ---- hot path (float) ---------------------------------------------------------------------------- */
CUNN_API void THNN_CudaSpatialDepthWiseConvolution_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaSpatialDepthWiseConvolution_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaSpatialDepthWiseConvolution_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, float scale);

CUNN_API void THNN_CudaSpatialConvolutionMM_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaSpatialConvolutionMM_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaSpatialConvolutionMM_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, float scale);

CUNN_API void THNN_CudaSpatialDilatedConvolution_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW,
    int dilationH);
CUNN_API void THNN_CudaSpatialDilatedConvolution_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH);
CUNN_API void THNN_CudaSpatialDilatedConvolution_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW,
    int dilationH, float scale);

/* lib/THCUNN/generic/THCUNN.h:766-806 (SpatialFullDilatedConvolution) and :849-886 (SpatialFullConvolution) */
CUNN_API void THNN_CudaSpatialFullDilatedConvolution_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW,
    int dilationH, int adjW, int adjH);
CUNN_API void THNN_CudaSpatialFullDilatedConvolution_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH,
    int adjW, int adjH);
CUNN_API void THNN_CudaSpatialFullDilatedConvolution_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW,
    int dilationH, int adjW, int adjH, float scale);
CUNN_API void THNN_CudaSpatialFullConvolution_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH);
CUNN_API void THNN_CudaSpatialFullConvolution_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH);
CUNN_API void THNN_CudaSpatialFullConvolution_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH,
    float scale);

CUNN_API void THNN_CudaBatchNormalization_updateOutput(
    THCState *state, THCudaTensor *input_, THCudaTensor *output_, THCudaTensor *weight_, THCudaTensor *bias_,
    THCudaTensor *runningMean_, THCudaTensor *runningVar_, THCudaTensor *saveMean_, THCudaTensor *saveStd_,
    bool train, double momentum, double eps);
CUNN_API void THNN_CudaBatchNormalization_backward(
    THCState *state, THCudaTensor *input_, THCudaTensor *gradOutput_, THCudaTensor *gradInput_,
    THCudaTensor *gradWeight_, THCudaTensor *gradBias_, THCudaTensor *weight_, THCudaTensor *runningMean_,
    THCudaTensor *runningVar_, THCudaTensor *saveMean_, THCudaTensor *saveStd_, bool train, double scale, double eps);

CUNN_API void THNN_CudaSpatialMaxPooling_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaLongTensor *indices, int kW, int kH, int dW,
    int dH, int padW, int padH, bool ceil_mode);
CUNN_API void THNN_CudaSpatialMaxPooling_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaLongTensor *indices,
    int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode);

/* lib/THCUNN/generic/THCUNN.h:587-628 (SpatialConvolutionLocal), :520-546 (adaptive pooling) */
CUNN_API void THNN_CudaSpatialConvolutionLocal_updateOutput(
    THCState *state, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *finput,
    THCudaTensor *fgradInput, int kW, int kH, int dW, int dH, int padW, int padH, long inputWidth, long inputHeight,
    long outputWidth, long outputHeight);
CUNN_API void THNN_CudaSpatialConvolutionLocal_updateGradInput(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *finput, THCudaTensor *fgradInput, int kW, int kH, int dW, int dH, int padW, int padH, long inputWidth,
    long inputHeight, long outputWidth, long outputHeight);
CUNN_API void THNN_CudaSpatialConvolutionLocal_accGradParameters(
    THCState *state, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *finput, THCudaTensor *fgradInput, int kW, int kH, int dW, int dH, int padW, int padH, long inputWidth,
    long inputHeight, long outputWidth, long outputHeight, float scale);
CUNN_API void THNN_CudaSpatialAdaptiveMaxPooling_updateOutput(THCState *state, THCudaTensor *input, THCudaTensor *output,
                                                              THCudaLongTensor *indices, int nOutputCols, int nOutputRows);
CUNN_API void THNN_CudaSpatialAdaptiveMaxPooling_updateGradInput(THCState *state, THCudaTensor *input, THCudaTensor *gradOutput,
                                                                 THCudaTensor *gradInput, THCudaLongTensor *indices);
CUNN_API void THNN_CudaSpatialAdaptiveAveragePooling_updateOutput(THCState *state, THCudaTensor *input, THCudaTensor *output,
                                                                  int nOutputCols, int nOutputRows);
CUNN_API void THNN_CudaSpatialAdaptiveAveragePooling_updateGradInput(THCState *state, THCudaTensor *input, THCudaTensor *gradOutput,
                                                                     THCudaTensor *gradInput);

/* ---- hot path (double): the same ten entry points for THCudaDoubleTensor, accreal = double (THCUNN.lua:54) ---- */
CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_updateOutput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaDoubleTensor *weight, THCudaDoubleTensor *bias,
    THCudaDoubleTensor *columns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_updateGradInput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaDoubleTensor *weight,
    THCudaDoubleTensor *gradColumns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_accGradParameters(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradWeight, THCudaDoubleTensor *gradBias,
    THCudaDoubleTensor *columns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, double scale);
CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_updateOutput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaDoubleTensor *weight, THCudaDoubleTensor *bias,
    THCudaDoubleTensor *columns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_updateGradInput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaDoubleTensor *weight,
    THCudaDoubleTensor *gradColumns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH);
CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_accGradParameters(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradWeight, THCudaDoubleTensor *gradBias,
    THCudaDoubleTensor *columns, THCudaDoubleTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, double scale);
CUNN_API void THNN_CudaDoubleBatchNormalization_updateOutput(
    THCState *state, THCudaDoubleTensor *input_, THCudaDoubleTensor *output_, THCudaDoubleTensor *weight_, THCudaDoubleTensor *bias_,
    THCudaDoubleTensor *runningMean_, THCudaDoubleTensor *runningVar_, THCudaDoubleTensor *saveMean_, THCudaDoubleTensor *saveStd_,
    bool train, double momentum, double eps);
CUNN_API void THNN_CudaDoubleBatchNormalization_backward(
    THCState *state, THCudaDoubleTensor *input_, THCudaDoubleTensor *gradOutput_, THCudaDoubleTensor *gradInput_,
    THCudaDoubleTensor *gradWeight_, THCudaDoubleTensor *gradBias_, THCudaDoubleTensor *weight_, THCudaDoubleTensor *runningMean_,
    THCudaDoubleTensor *runningVar_, THCudaDoubleTensor *saveMean_, THCudaDoubleTensor *saveStd_, bool train, double scale, double eps);
CUNN_API void THNN_CudaDoubleSpatialMaxPooling_updateOutput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaLongTensor *indices, int kW, int kH, int dW,
    int dH, int padW, int padH, bool ceil_mode);
CUNN_API void THNN_CudaDoubleSpatialMaxPooling_updateGradInput(
    THCState *state, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaLongTensor *indices,
    int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode);

/* ---- support operators (float) --------------------------------------------------------------------- */
CUNN_API void THNN_CudaThreshold_updateOutput(THCState *state, THCudaTensor *input, THCudaTensor *output,
                                              float threshold, float val, bool inplace);
CUNN_API void THNN_CudaThreshold_updateGradInput(THCState *state, THCudaTensor *input, THCudaTensor *gradOutput,
                                                 THCudaTensor *gradInput, float threshold, float val, bool inplace);
CUNN_API void THNN_CudaSpatialAveragePooling_updateOutput(THCState *state, THCudaTensor *input, THCudaTensor *output,
                                                          int kW, int kH, int dW, int dH, int padW, int padH,
                                                          bool ceil_mode, bool count_include_pad);
CUNN_API void THNN_CudaSpatialAveragePooling_updateGradInput(THCState *state, THCudaTensor *input,
                                                             THCudaTensor *gradOutput, THCudaTensor *gradInput, int kW,
                                                             int kH, int dW, int dH, int padW, int padH, bool ceil_mode,
                                                             bool count_include_pad);
CUNN_API void THNN_CudaLogSoftMax_updateOutput(THCState *state, THCudaTensor *input, THCudaTensor *output);
CUNN_API void THNN_CudaLogSoftMax_updateGradInput(THCState *state, THCudaTensor *input, THCudaTensor *gradOutput,
                                                  THCudaTensor *gradInput, THCudaTensor *output);
CUNN_API void THNN_CudaClassNLLCriterion_updateOutput(THCState *state, THCudaTensor *input, THCudaLongTensor *target,
                                                      THCudaTensor *output, bool sizeAverage, THCudaTensor *weights,
                                                      THCudaTensor *total_weight, long ignore_index);
CUNN_API void THNN_CudaClassNLLCriterion_updateGradInput(THCState *state, THCudaTensor *input, THCudaLongTensor *target,
                                                         THCudaTensor *gradInput, bool sizeAverage,
                                                         THCudaTensor *weights, THCudaTensor *total_weight,
                                                         long ignore_index);

/* Every other THNN_Cuda<Op>_<method> and THNN_CudaDouble<Op>_<method> name of the reference header is
 * exported too, so the binding's symbol lookup cannot fail, but only reports "not implemented in this
 * build" through the error hook of the state it is given. */

#ifdef __cplusplus
}
#endif
#endif /* THCUNN_B200_H */
