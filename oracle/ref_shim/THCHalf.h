/* Stand-in for cutorch's THCHalf.h: no half type in this build (CUDA_HALF_TENSOR stays undefined). */
#ifndef REFK_SHIM_THCHALF_H
#define REFK_SHIM_THCHALF_H
#include "THC/THC.h"
#endif
