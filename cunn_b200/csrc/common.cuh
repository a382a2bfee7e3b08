// Shared host/device helpers of the cunn_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/cunn_b200.h"

namespace cunn {

// ---- host-side error reporting ---------------------------------------------
// Thread-local message buffer behind cunn_b200_last_error().
int fail(const char *fmt, ...);
void clear_error();

#define CUNN_CHECK_ARG(cond, ...)                 \
    do {                                          \
        if (!(cond)) return cunn::fail(__VA_ARGS__); \
    } while (0)

#define CUNN_CUDA(call)                                                                  \
    do {                                                                                 \
        cudaError_t e_ = (call);                                                         \
        if (e_ != cudaSuccess)                                                           \
            return cunn::fail("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

#define CUNN_LAUNCH_CHECK(name)                                                         \
    do {                                                                                \
        cudaError_t e_ = cudaGetLastError();                                            \
        if (e_ != cudaSuccess) return cunn::fail("launch of %s failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Device status word (one per device, zero-initialised).  Kernels record a
// non-zero code here when a bounded wait runs out; see cunn_b200_device_status().
int *device_status_ptr();

enum StatusCode : int {
    STATUS_OK = 0,
    STATUS_MBARRIER_TIMEOUT = 1,
    STATUS_TMEM_TIMEOUT = 2,
    STATUS_FLAG_TIMEOUT = 3,      // a CTA gave up waiting for another CTA of its own grid
};

#ifdef __CUDACC__
// ---- device-side PTX wrappers ----------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

// Makes freshly initialised barriers visible to the async (bulk copy) proxy.
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One poll of the barrier phase.  The suspend-time hint lets the hardware park the thread until the
// phase completes (or the hint, in nanoseconds, runs out) instead of burning issue slots on polling.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000000u)
        : "memory");
    return ok != 0;
}

// Waits for the given phase parity with a cycle limit (about a second).  On
// expiry records STATUS_MBARRIER_TIMEOUT in *status and returns false so the
// caller can leave the kernel instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 2000000000LL) {
            if (status) atomicExch(status, (int)STATUS_MBARRIER_TIMEOUT);
            return false;
        }
    }
    return true;
}

// 1-D bulk copy global -> shared through the TMA unit, completion counted in
// bytes on an mbarrier.  dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// The same copy with an L2 eviction-priority policy (createpolicy) attached to the global read.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

// Programmatic dependent launch (PDL).  launch_dependents: the next kernel in the stream, if it was launched
// as a programmatic dependent, may be scheduled once every CTA of this grid has passed this point or exited.
// wait: blocks until the grids this one depends on have completed and their memory is visible; a no-op
// when the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
#endif  // __CUDACC__

}  // namespace cunn
