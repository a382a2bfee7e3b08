/* Stand-in for cutorch's <THC/THC.h>, written for this repository (test infrastructure).
 *
 * The reference's kernel files (lib/THCUNN/*.cu, im2col.h) include cutorch headers that are not
 * part of the reference tree.  This folder supplies just enough of those names for the __global__
 * kernel templates in those files to compile unchanged, from where they lie, with the host
 * wrappers (lib/THCUNN/generic/*.cu) left out: THCGenerateFloatTypes.h here expands to nothing.
 * Nothing in this folder is taken from cutorch; each definition restates the public meaning of the
 * name (THCNumerics<T>::min() is the lowest finite value, ScalarConvert a static_cast, ...).
 *
 * Two build modes (see ../Makefile):
 *   nvcc          the kernels run on the GPU as the reference wrote them;
 *   g++ -DREFK_CPU the kernels that are a plain CUDA_KERNEL_LOOP over independent indices (pooling)
 *                 run on the host, one kernel invocation per index (one emulated thread per block).
 */
#ifndef REFK_SHIM_THC_H
#define REFK_SHIM_THC_H

#include <cfloat>
#include <cmath>
#include <cstdio>
#include <cstdlib>

#ifdef REFK_CPU
#include <algorithm>
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
struct refk_dim3 { int x, y, z; };
/* One emulated thread per block; the launcher sets gridDim.x to the element count and steps blockIdx.x,
 * so each kernel invocation handles exactly one index, as each CUDA thread does in the reference's launch. */
static refk_dim3 blockIdx = {0, 0, 0}, gridDim = {1, 1, 1};
static const refk_dim3 threadIdx = {0, 0, 0}, blockDim = {1, 1, 1};
using std::max;
using std::min;
#else
#include <cuda_runtime.h>
#endif

/* Lua-Torch builds libTH with 1-based indices; the pooling kernels add this to stored indices. */
#ifndef TH_INDEX_BASE
#define TH_INDEX_BASE 1
#endif

#define TH_CONCAT_3(x, y, z) TH_CONCAT_3_EXPAND(x, y, z)
#define TH_CONCAT_3_EXPAND(x, y, z) x##y##z
#define TH_API extern "C"

typedef struct THCState THCState;

#ifndef REFK_CPU
static inline void refk_cuda_check(cudaError_t e, const char *file, int line) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "reference kernel launch failed at %s:%d: %s\n", file, line, cudaGetErrorString(e));
    std::abort();
  }
}
#define THCudaCheck(expr) refk_cuda_check((expr), __FILE__, __LINE__)
#endif

#include "../THCNumerics.cuh"

#endif
