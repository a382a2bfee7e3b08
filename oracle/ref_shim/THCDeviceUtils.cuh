/* Stand-in for cutorch's THCDeviceUtils.cuh: warp shuffle spelling for CUDA 9+. */
#ifndef REFK_SHIM_THCDEVICEUTILS_CUH
#define REFK_SHIM_THCDEVICEUTILS_CUH
#define WARP_SHFL_XOR(value, mask, width) __shfl_xor_sync(0xffffffffu, (value), (mask), (width))
#endif
