// First-layer (3 channels, 3x3, 32 filters) direct convolution kernels; see stemconv.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace cunn {
namespace stem {

bool applies(int C, int K, int kH, int kW);
int wgrad_ctas();                    // CTAs of the weight-gradient kernel = partial sums per output
size_t wgrad_workspace_bytes();      // [ctas][864] weight partials, then [32][ctas] bias partials
int forward(const float *x, const float *w, const float *bias, float *y, int N, int H, int W, int oH, int oW, int dH, int dW,
            int padH, int padW, cudaStream_t stream);
int weight_grad_partials(const float *x, const float *gy, float *partial, float *bias_part, int N, int H, int W, int oH,
                         int oW, int dH, int dW, int padH, int padW, cudaStream_t stream);

}  // namespace stem
}  // namespace cunn
