// Error reporting, device properties and the per-device status word.
#include "common.cuh"

#include <string.h>

namespace cunn {

static thread_local char g_err[512] = "";

int fail(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return 1;
}

void clear_error() { g_err[0] = 0; }

static const int kMaxDevices = 64;

int sm_count() {
    static int cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// One status word per device that loads this module; zero at load.
__device__ int g_device_status = 0;

int *device_status_ptr() {
    static int *cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!cached[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cached[dev] = (int *)p;
    }
    return cached[dev];
}

}  // namespace cunn

extern "C" const char *cunn_b200_last_error(void) { return cunn::g_err; }

extern "C" int cunn_b200_device_status(void) {
    int *p = cunn::device_status_ptr();
    if (!p) {
        cunn::fail("no CUDA device: %s", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        cunn::fail("device status read failed: %s", cudaGetErrorString(e));
        return -1;
    }
    return v;
}
