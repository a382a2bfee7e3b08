/* Stand-in for cutorch's THCNumerics.cuh: the two helpers the reference kernels on this path use. */
#ifndef REFK_SHIM_THCNUMERICS_CUH
#define REFK_SHIM_THCNUMERICS_CUH
#include "THC/THC.h"

template <typename T> struct THCNumerics;
template <> struct THCNumerics<float> {
  static inline __host__ __device__ float min() { return -FLT_MAX; }
  static inline __host__ __device__ float max() { return FLT_MAX; }
};
template <> struct THCNumerics<double> {
  static inline __host__ __device__ double min() { return -DBL_MAX; }
  static inline __host__ __device__ double max() { return DBL_MAX; }
};

template <typename In, typename Out> struct ScalarConvert {
  static inline __host__ __device__ Out to(const In v) { return (Out)v; }
};
#endif
