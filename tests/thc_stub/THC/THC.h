/* Declaration-only stand-in for cutorch's <THC/THC.h>, used by the tests to compile-check the cutorch
 * back-end of the THNN entry points (cunn_b200/csrc/thc_backend_real.inc) where cutorch is absent.  It
 * declares the structs with the public fields the reference's wrappers dereference (size, stride,
 * nDimension, storage, storageOffset — e.g. lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:76-77,100)
 * and the libTHC functions that back-end calls, and defines nothing: an object built against it has
 * those functions as undefined symbols, which the test lists. */
#ifndef THC_STUB_THC_H
#define THC_STUB_THC_H

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct THCState THCState;

typedef struct THCudaStorage { float *data; ptrdiff_t size; int refcount; char flag; void *allocator; void *allocatorContext; struct THCudaStorage *view; int device; } THCudaStorage;
typedef struct THCudaLongStorage { long *data; ptrdiff_t size; int refcount; char flag; void *allocator; void *allocatorContext; struct THCudaLongStorage *view; int device; } THCudaLongStorage;
typedef struct THCudaDoubleStorage { double *data; ptrdiff_t size; int refcount; char flag; void *allocator; void *allocatorContext; struct THCudaDoubleStorage *view; int device; } THCudaDoubleStorage;
typedef struct THCudaDoubleTensor { long *size; long *stride; int nDimension; THCudaDoubleStorage *storage; ptrdiff_t storageOffset; int refcount; char flag; } THCudaDoubleTensor;
typedef struct THCudaTensor { long *size; long *stride; int nDimension; THCudaStorage *storage; ptrdiff_t storageOffset; int refcount; char flag; } THCudaTensor;
typedef struct THCudaLongTensor { long *size; long *stride; int nDimension; THCudaLongStorage *storage; ptrdiff_t storageOffset; int refcount; char flag; } THCudaLongTensor;

cudaStream_t THCState_getCurrentStream(THCState *state);
cudaError_t THCudaMalloc(THCState *state, void **ptr, size_t size);
cudaError_t THCudaFree(THCState *state, void *ptr);

THCudaTensor *THCudaTensor_new(THCState *state);
void THCudaTensor_free(THCState *state, THCudaTensor *self);
THCudaTensor *THCudaTensor_newContiguous(THCState *state, THCudaTensor *tensor);
void THCudaTensor_resizeNd(THCState *state, THCudaTensor *tensor, int nDimension, long *size, long *stride);
void THCudaDoubleTensor_free(THCState *state, THCudaDoubleTensor *self);
THCudaDoubleTensor *THCudaDoubleTensor_newContiguous(THCState *state, THCudaDoubleTensor *tensor);
void THCudaDoubleTensor_resizeNd(THCState *state, THCudaDoubleTensor *tensor, int nDimension, long *size, long *stride);
void THCudaLongTensor_resizeNd(THCState *state, THCudaLongTensor *tensor, int nDimension, long *size, long *stride);

void _THError(const char *file, const int line, const char *fmt, ...);
#define THError(...) _THError(__FILE__, __LINE__, __VA_ARGS__)

#ifdef __cplusplus
}
#endif
#endif
