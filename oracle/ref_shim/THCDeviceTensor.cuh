/* Stand-in for cutorch's THCDeviceTensor.cuh: a contiguous Dim-dimensional view of device memory
 * with the member names the reference's batch-norm kernels use (getSize, numElements, chained
 * operator[] ending in a reference-like proxy with ldg()). */
#ifndef REFK_SHIM_THCDEVICETENSOR_CUH
#define REFK_SHIM_THCDEVICETENSOR_CUH
#include "THC/THC.h"

template <typename T> struct RefkElem {
  T *p;
  __device__ RefkElem(T *q) : p(q) {}
  __device__ operator T() const { return *p; }
  __device__ T ldg() const { return __ldg(p); }
  __device__ RefkElem &operator=(T v) { *p = v; return *this; }
  __device__ RefkElem &operator+=(T v) { *p += v; return *this; }
};

template <typename T, int Dim, int Sub> struct RefkSub {
  T *p;
  const int *size;
  __device__ RefkSub(T *q, const int *s) : p(q), size(s) {}
  __device__ RefkSub<T, Dim, Sub - 1> operator[](int i) const {
    long stride = 1;
    for (int d = Dim - Sub + 1; d < Dim; ++d) stride *= size[d];
    return RefkSub<T, Dim, Sub - 1>(p + i * stride, size);
  }
};
template <typename T, int Dim> struct RefkSub<T, Dim, 1> {
  T *p;
  const int *size;
  __device__ RefkSub(T *q, const int *s) : p(q), size(s) {}
  __device__ RefkElem<T> operator[](int i) const { return RefkElem<T>(p + i); }
};

template <typename T, int Dim> class THCDeviceTensor {
 public:
  __host__ __device__ THCDeviceTensor() : data_(0) { for (int i = 0; i < Dim; ++i) size_[i] = 0; }
  __host__ __device__ THCDeviceTensor(T *data, const int size[Dim]) : data_(data) {
    for (int i = 0; i < Dim; ++i) size_[i] = size[i];
  }
  __host__ __device__ int getSize(int i) const { return size_[i]; }
  __host__ __device__ long numElements() const {
    if (!data_) return 0;
    long n = 1;
    for (int i = 0; i < Dim; ++i) n *= size_[i];
    return n;
  }
  __device__ auto operator[](int i) const { return RefkSub<T, Dim, Dim>(data_, size_)[i]; }

 private:
  T *data_;
  int size_[Dim];
};
#endif
