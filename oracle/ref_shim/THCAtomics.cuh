/* Stand-in for cutorch's THCAtomics.cuh: float / double atomicAdd are CUDA built-ins; on the host build an
 * "atomic" add is a plain add (one emulated thread at a time). */
#ifndef REFK_SHIM_THCATOMICS_CUH
#define REFK_SHIM_THCATOMICS_CUH
#ifdef REFK_CPU
template <typename T> static inline T atomicAdd(T *address, T val) { T old = *address; *address = old + val; return old; }
#endif
#endif
