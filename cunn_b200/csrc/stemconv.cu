// Direct convolution for the first layer of an image network: 3 input channels, 3x3 kernel, 32 filters
// (SpatialConvolutionMM with C * kH * kW = 27).  The reduction length of 27 fills less than one k-block of
// the tensor-core path and both passes are bound by the 2 GB of activations they stream, so they run on the
// fp32 pipes with the operands staged once:
//   forward          one thread per output pixel: its 27 input values in registers, the 864 weights in
//                    shared memory read as 16-byte broadcasts (4 filters per load), 32 coalesced stores;
//   weight gradient  tiles of 256 pixels: the unfolded inputs [pixel][27 (+5 zero) taps] and the output
//                    gradients [pixel][32 filters] are written to shared memory in 16-byte chunks (chunk index
//                    XOR pixel, so neither the row-wise writes nor the reads conflict); each warp then walks 32
//                    pixels with a 4-filter x 8-tap register tile per lane.  Per-CTA sums go to the workspace
//                    and are added up in CTA order by the same reduction kernels as the GEMM path.
#include "common.cuh"
#include "stemconv.h"

#include <algorithm>

namespace cunn {
namespace stem {

constexpr int CIN = 3, KS = 3, TAPS = CIN * KS * KS, KOUT = 32;
constexpr int TILE_PIX = 256;

__global__ void __launch_bounds__(256)
fwd_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y,
           int H, int W, int oH, int oW, int dH, int dW, int padH, int padW, long long total)
{
    __shared__ __align__(16) float ws[TAPS * KOUT];      // [tap][filter]
    for (int i = threadIdx.x; i < TAPS * KOUT; i += blockDim.x) {
        const int k = i % KOUT, tap = i / KOUT;
        ws[i] = __ldg(w + k * TAPS + tap);
    }
    __syncthreads();
    const long long pix = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= total) return;
    const int oHW = oH * oW;
    const int n = (int)(pix / oHW), r = (int)(pix - (long long)n * oHW);
    const int oh = r / oW, ow = r - oh * oW;
    const int ih0 = oh * dH - padH, iw0 = ow * dW - padW;
    float xv[TAPS];
    const float *xi = x + (size_t)n * CIN * H * W;
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int kh = 0; kh < KS; ++kh)
#pragma unroll
            for (int kw = 0; kw < KS; ++kw) {
                const int ih = ih0 + kh, iw = iw0 + kw;
                xv[(c * KS + kh) * KS + kw] =
                    ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) ? __ldg(xi + ((size_t)c * H + ih) * W + iw) : 0.f;
            }
    float acc[KOUT];
#pragma unroll
    for (int k = 0; k < KOUT; ++k) acc[k] = bias ? __ldg(bias + k) : 0.f;
    const float4 *ws4 = reinterpret_cast<const float4 *>(ws);
#pragma unroll
    for (int tap = 0; tap < TAPS; ++tap) {
#pragma unroll
        for (int q = 0; q < KOUT / 4; ++q) {
            const float4 w4 = ws4[tap * (KOUT / 4) + q];
            acc[4 * q + 0] = fmaf(xv[tap], w4.x, acc[4 * q + 0]);
            acc[4 * q + 1] = fmaf(xv[tap], w4.y, acc[4 * q + 1]);
            acc[4 * q + 2] = fmaf(xv[tap], w4.z, acc[4 * q + 2]);
            acc[4 * q + 3] = fmaf(xv[tap], w4.w, acc[4 * q + 3]);
        }
    }
    float *yo = y + (size_t)n * KOUT * oHW + r;
#pragma unroll
    for (int k = 0; k < KOUT; ++k) yo[(size_t)k * oHW] = acc[k];
}

// partial: [gridDim.x][TAPS * KOUT] in gradWeight order; bias_part: [KOUT][gridDim.x].
__global__ void __launch_bounds__(256)
wgrad_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ partial,
             float *__restrict__ bias_part, int H, int W, int oH, int oW, int dH, int dW, int padH, int padW, long long total)
{
    extern __shared__ __align__(16) float sm[];
    float4 *xt = reinterpret_cast<float4 *>(sm);                       // [pixel][8 chunks of 4 taps], chunk ^ (pixel & 7)
    float4 *gt = reinterpret_cast<float4 *>(sm) + TILE_PIX * 8;        // [pixel][8 chunks of 4 filters], same swizzle
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kq = lane & 7, tg = lane >> 3;                           // this lane's 4 filters and 8 taps
    const int oHW = oH * oW;
    float acc[4][8];
    float bsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;

    const long long tiles = (total + TILE_PIX - 1) / TILE_PIX;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        // ---- build: one thread per pixel ----
        const long long pix = tile * TILE_PIX + tid;
        float v[32], g[KOUT];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll
        for (int k = 0; k < KOUT; ++k) g[k] = 0.f;
        if (pix < total) {
            const int n = (int)(pix / oHW), r = (int)(pix - (long long)n * oHW);
            const int oh = r / oW, ow = r - oh * oW;
            const int ih0 = oh * dH - padH, iw0 = ow * dW - padW;
            const float *xi = x + (size_t)n * CIN * H * W;
#pragma unroll
            for (int c = 0; c < CIN; ++c)
#pragma unroll
                for (int kh = 0; kh < KS; ++kh)
#pragma unroll
                    for (int kw = 0; kw < KS; ++kw) {
                        const int ih = ih0 + kh, iw = iw0 + kw;
                        if ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W)
                            v[(c * KS + kh) * KS + kw] = __ldg(xi + ((size_t)c * H + ih) * W + iw);
                    }
            const float *gi = gy + (size_t)n * KOUT * oHW + r;
#pragma unroll
            for (int k = 0; k < KOUT; ++k) g[k] = __ldg(gi + (size_t)k * oHW);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            xt[tid * 8 + (c ^ (tid & 7))] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
            gt[tid * 8 + (c ^ (tid & 7))] = make_float4(g[4 * c], g[4 * c + 1], g[4 * c + 2], g[4 * c + 3]);
        }
        __syncthreads();
        // ---- accumulate: each warp takes 32 pixels of the tile ----
#pragma unroll 4
        for (int pp = 0; pp < 32; ++pp) {
            const int p = warp * 32 + pp;
            const float4 g4 = gt[p * 8 + (kq ^ (p & 7))];
            const float4 xa = xt[p * 8 + ((2 * tg) ^ (p & 7))];
            const float4 xb = xt[p * 8 + ((2 * tg + 1) ^ (p & 7))];
            const float gv[4] = {g4.x, g4.y, g4.z, g4.w};
            const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                bsum[a] += gv[a];
#pragma unroll
                for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(gv[a], xs[b], acc[a][b]);
            }
        }
        __syncthreads();
    }
    // ---- add the eight warps' tiles in warp order; thread t finishes outputs t, t + 256, ... ----
    float *scratch = sm;                                               // [8 warps][KOUT * 32 padded taps] + [8][KOUT]
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) scratch[warp * 1024 + (kq * 4 + a) * 32 + tg * 8 + b] = acc[a][b];
    if (tg == 0) {
#pragma unroll
        for (int a = 0; a < 4; ++a) scratch[8 * 1024 + warp * KOUT + kq * 4 + a] = bsum[a];
    }
    __syncthreads();
    for (int i = tid; i < KOUT * TAPS; i += blockDim.x) {
        const int k = i / TAPS, tap = i - k * TAPS;
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) s += scratch[wv * 1024 + k * 32 + tap];
        partial[(size_t)blockIdx.x * (KOUT * TAPS) + i] = s;
    }
    if (bias_part && tid < KOUT) {
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) s += scratch[8 * 1024 + wv * KOUT + tid];
        bias_part[(size_t)tid * gridDim.x + blockIdx.x] = s;
    }
}

constexpr size_t WGRAD_SMEM = (size_t)(8 * 1024 + 8 * KOUT) * sizeof(float) > (size_t)2 * TILE_PIX * 8 * sizeof(float4)
                                  ? (size_t)(8 * 1024 + 8 * KOUT) * sizeof(float)
                                  : (size_t)2 * TILE_PIX * 8 * sizeof(float4);

bool applies(int C, int K, int kH, int kW)
{
    return C == CIN && K == KOUT && kH == KS && kW == KS;
}

int wgrad_ctas() { return sm_count() * 2; }

size_t wgrad_workspace_bytes()
{
    return (size_t)wgrad_ctas() * (KOUT * TAPS + KOUT) * sizeof(float) + 256;
}

int forward(const float *x, const float *w, const float *bias, float *y, int N, int H, int W, int oH, int oW, int dH, int dW,
            int padH, int padW, cudaStream_t stream)
{
    const long long total = (long long)N * oH * oW;
    const long long blocks = (total + 255) / 256;
    CUNN_CHECK_ARG(blocks < (1LL << 31), "too many output pixels");
    fwd_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, w, bias, y, H, W, oH, oW, dH, dW, padH, padW, total);
    CUNN_LAUNCH_CHECK("first-layer convolution forward");
    return 0;
}

int weight_grad_partials(const float *x, const float *gy, float *partial, float *bias_part, int N, int H, int W, int oH,
                         int oW, int dH, int dW, int padH, int padW, cudaStream_t stream)
{
    const long long total = (long long)N * oH * oW;
    CUNN_CUDA(cudaFuncSetAttribute((const void *)wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WGRAD_SMEM));
    wgrad_kernel<<<wgrad_ctas(), 256, WGRAD_SMEM, stream>>>(x, gy, partial, bias_part, H, W, oH, oW, dH, dW, padH, padW, total);
    CUNN_LAUNCH_CHECK("first-layer convolution weight gradient");
    return 0;
}

}  // namespace stem
}  // namespace cunn
