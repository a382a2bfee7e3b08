// Spatial max pooling with argmax for sm_100a: forward (values + int64 indices) and backward.
//
// Semantics follow the reference kernels exactly (bit-exact indices): the window is scanned row-major,
// a candidate replaces the running maximum only if it is strictly greater, the scan starts from
// -FLT_MAX with index -1, so NaN and -inf never win and the first of equal maxima is kept.  The stored
// index is the flat position h*W + w inside the plane plus CUNN_B200_INDEX_BASE.  Backward is the
// gather form: every input pixel adds the gradients of the outputs whose stored index names it, so it
// needs no atomics and is deterministic.
//
// Both directions are HBM-bound.  The 3x3 / stride 2 / pad 1 case (ResNet, MobileNet stems) has
// dedicated kernels with 16-byte loads and stores; everything else runs shape-generic kernels.
#include "common.cuh"
#include "pool_generic.cuh"

#include <float.h>
#include <algorithm>

namespace cunn {
namespace pool {

// ---------------------------------------------------------------------------
// 3x3, stride 2, pad 1, even W with W % 8 == 0 (so oW == W / 2 and oW % 4 == 0)
// ---------------------------------------------------------------------------

// Forward.  A thread owns four adjacent outputs of RS consecutive output rows; per input row it loads
// columns 8g-1 .. 8g+7 (one scalar + two 16-byte loads) and keeps row 2o+1 for the next window.
// Out-of-range rows and the left pad column read as -FLT_MAX, which can never win the strict compare.
template <int RS>
__global__ void __launch_bounds__(256)
fwd_k3s2p1_kernel(const float *__restrict__ x, float *__restrict__ y, long long *__restrict__ ind, int H, int W,
                  int oH, int oW, long long planes)
{
    const int CG = oW >> 2;
    const int strips = (oH + RS - 1) / RS;
    const long long items = planes * strips * CG;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const int g = (int)(it % CG);
        const long long t = it / CG;
        const int strip = (int)(t % strips);
        const long long plane = t / strips;
        const float *xp = x + plane * (long long)H * W + 8 * g;
        float *yp = y + plane * (long long)oH * oW + 4 * g;
        long long *ip = ind + plane * (long long)oH * oW + 4 * g;
        const int o0 = strip * RS, o1 = min(oH, o0 + RS);
        const bool has_left = g > 0;
        const int colbase = 8 * g - 1;  // column of r[0]

        auto load_row = [&](int row, float (&r)[9]) {
            if ((unsigned)row >= (unsigned)H) {
#pragma unroll
                for (int i = 0; i < 9; ++i) r[i] = -FLT_MAX;
                return;
            }
            const float *p = xp + (long long)row * W;
            r[0] = has_left ? __ldg(p - 1) : -FLT_MAX;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(p + 4));
            r[1] = a.x; r[2] = a.y; r[3] = a.z; r[4] = a.w;
            r[5] = b.x; r[6] = b.y; r[7] = b.z; r[8] = b.w;
        };
        auto emit = [&](int o, const float (&ra)[9], const float (&rb)[9], const float (&rc)[9]) {
            float bv[4];
            long long bi[4];
            const int rowoff0 = (2 * o - 1) * W + colbase;  // flat index of ra[0]
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                float best = -FLT_MAX;
                int idx = -1;
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    const float c = ra[2 * v + kw];
                    if (c > best) { best = c; idx = rowoff0 + 2 * v + kw; }
                }
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    const float c = rb[2 * v + kw];
                    if (c > best) { best = c; idx = rowoff0 + W + 2 * v + kw; }
                }
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
                    const float c = rc[2 * v + kw];
                    if (c > best) { best = c; idx = rowoff0 + 2 * W + 2 * v + kw; }
                }
                bv[v] = best;
                bi[v] = (long long)idx + CUNN_B200_INDEX_BASE;
            }
            *reinterpret_cast<float4 *>(yp + (long long)o * oW) = make_float4(bv[0], bv[1], bv[2], bv[3]);
            longlong2 *ipo = reinterpret_cast<longlong2 *>(ip + (long long)o * oW);
            ipo[0] = make_longlong2(bi[0], bi[1]);
            ipo[1] = make_longlong2(bi[2], bi[3]);
        };
        float r0[9], r1[9], r2[9];
        load_row(2 * o0 - 1, r0);
        for (int o = o0; o < o1; o += 2) {
            load_row(2 * o, r1);
            load_row(2 * o + 1, r2);
            emit(o, r0, r1, r2);
            if (o + 1 >= o1) break;
            load_row(2 * o + 2, r1);
            load_row(2 * o + 3, r0);
            emit(o + 1, r2, r1, r0);
        }
    }
}

// Backward.  Input rows 2a and 2a+1 only receive from output rows a and a+1 (even rows only from a),
// input columns 2b and 2b+1 only from output columns b and b+1 (even columns only from b).  A thread
// owns an 2-row x 8-column block of gx: it loads five (index, gradient) pairs from each of the two
// output rows and writes two 16-byte vectors per row.
__global__ void __launch_bounds__(256)
bwd_k3s2p1_kernel(const float *__restrict__ gy, const long long *__restrict__ ind, float *__restrict__ gx, int H,
                  int W, int oH, int oW, long long planes)
{
    const int CG = W >> 3;            // blocks of 8 input columns = 4 output columns
    const int RB = (H + 1) >> 1;      // blocks of 2 input rows
    const long long items = planes * RB * CG;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const int g = (int)(it % CG);
        const long long t = it / CG;
        const int a = (int)(t % RB);
        const long long plane = t / RB;
        const float *gp = gy + plane * (long long)oH * oW + 4 * g;
        const long long *ip = ind + plane * (long long)oH * oW + 4 * g;
        float *xp = gx + plane * (long long)H * W + (long long)(2 * a) * W + 8 * g;
        const bool has_right = 4 * g + 4 < oW;

        // outputs (a, 4g .. 4g+4) and (a+1, 4g .. 4g+4); missing ones get an index that matches nothing
        long long i0[5], i1[5];
        float g0[5], g1[5];
        auto load_out = [&](int row, long long (&ii)[5], float (&gg)[5]) {
            if (row >= oH) {
#pragma unroll
                for (int j = 0; j < 5; ++j) { ii[j] = -1; gg[j] = 0.f; }
                return;
            }
            const longlong2 *q = reinterpret_cast<const longlong2 *>(ip + (long long)row * oW);
            const longlong2 q0 = __ldg(q), q1 = __ldg(q + 1);
            const float4 f = __ldg(reinterpret_cast<const float4 *>(gp + (long long)row * oW));
            ii[0] = q0.x; ii[1] = q0.y; ii[2] = q1.x; ii[3] = q1.y;
            gg[0] = f.x; gg[1] = f.y; gg[2] = f.z; gg[3] = f.w;
            if (has_right) {
                ii[4] = __ldg(ip + (long long)row * oW + 4);
                gg[4] = __ldg(gp + (long long)row * oW + 4);
            } else {
                ii[4] = -1;
                gg[4] = 0.f;
            }
        };
        load_out(a, i0, g0);
        load_out(a + 1, i1, g1);
        const long long base = (long long)(2 * a) * W + 8 * g + CUNN_B200_INDEX_BASE;  // index of block's (0,0)
        float e[8], o[8];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const long long pe0 = base + 2 * v, pe1 = pe0 + 1;          // row 2a, columns 2b and 2b+1
            const long long po0 = pe0 + W, po1 = po0 + 1;               // row 2a+1
            // accumulate in the reference's order: output rows ascending, columns ascending
            e[2 * v] = (i0[v] == pe0) ? g0[v] : 0.f;
            float s = (i0[v] == pe1) ? g0[v] : 0.f;
            if (i0[v + 1] == pe1) s += g0[v + 1];
            e[2 * v + 1] = s;
            s = (i0[v] == po0) ? g0[v] : 0.f;
            if (i1[v] == po0) s += g1[v];
            o[2 * v] = s;
            s = (i0[v] == po1) ? g0[v] : 0.f;
            if (i0[v + 1] == po1) s += g0[v + 1];
            if (i1[v] == po1) s += g1[v];
            if (i1[v + 1] == po1) s += g1[v + 1];
            o[2 * v + 1] = s;
        }
        *reinterpret_cast<float4 *>(xp) = make_float4(e[0], e[1], e[2], e[3]);
        *reinterpret_cast<float4 *>(xp + 4) = make_float4(e[4], e[5], e[6], e[7]);
        if (2 * a + 1 < H) {
            *reinterpret_cast<float4 *>(xp + W) = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4 *>(xp + W + 4) = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
}

static int out_size(int in, int k, int d, int pad, int dil, int ceil_mode)
{
    // floor / ceil of (in - (dil*(k-1)+1) + 2 pad) / d in integers, then the reference's fix-up:
    // the last window must start inside the input or its left/top padding
    const int num = in - (dil * (k - 1) + 1) + 2 * pad;
    int o;
    if (ceil_mode) o = (num >= 0 ? (num + d - 1) / d : -((-num) / d)) + 1;
    else           o = (num >= 0 ? num / d : -((-num + d - 1) / d)) + 1;
    if (pad && (o - 1) * d >= in + pad) --o;
    return o;
}

static int check(int N, int C, int H, int W, int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW,
                 int ceil_mode, int *oH, int *oW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(dilH > 0 && dilW > 0, "dilation should be greater than zero, but got dilationH: %d dilationW: %d",
                   dilH, dilW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && H > 0 && W > 0 && padH >= 0 && padW >= 0, "bad pooling sizes N=%d C=%d H=%d W=%d",
                   N, C, H, W);
    CUNN_CHECK_ARG(kW / 2 >= padW && kH / 2 >= padH,
                   "pad should be smaller than half of kernel size, but got padW = %d, padH = %d, kW = %d, kH = %d", padW,
                   padH, kW, kH);
    *oH = out_size(H, kH, dH, padH, dilH, ceil_mode);
    *oW = out_size(W, kW, dW, padW, dilW, ceil_mode);
    CUNN_CHECK_ARG(*oH >= 1 && *oW >= 1,
                   "Given input size: (%dx%dx%d). Calculated output size: (%dx%dx%d). Output size is too small", C, H, W,
                   C, *oH, *oW);
    CUNN_CHECK_ARG((long long)N * C * (long long)H * W < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    return 0;
}

static int grid_for(long long work_items)
{
    const long long want = ceil_div_ll(work_items, 256);
    const long long cap = (long long)sm_count() * 32;
    return (int)std::max(1LL, std::min(want, cap));
}

static bool fast_shape(const void *a, const void *b, const void *c, int H, int W, int oH, int oW, int kH, int kW,
                       int dH, int dW, int padH, int padW, int dilH, int dilW)
{
    const uintptr_t al = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c;
    return kH == 3 && kW == 3 && dH == 2 && dW == 2 && padH == 1 && padW == 1 && dilH == 1 && dilW == 1 && W % 8 == 0 &&
           oW * 2 == W && (al & 15) == 0 && (oH == H / 2 || oH == (H + 1) / 2) && oH * 2 + 1 >= H;
}

}  // namespace pool
}  // namespace cunn

using namespace cunn;
using namespace cunn::pool;

extern "C" CUNN_API int cunn_b200_maxpool_out_size(int in, int k, int d, int pad, int dil, int ceil_mode)
{
    return out_size(in, k, d, pad, dil, ceil_mode);
}

extern "C" CUNN_API int cunn_b200_maxpool_forward(const float *x, float *y, int64_t *indices, int N, int C, int H,
                                                  int W, int kH, int kW, int dH, int dW, int padH, int padW, int dilH,
                                                  int dilW, int ceil_mode, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, ceil_mode, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && y && indices, "null tensor pointer");
    const long long planes = (long long)N * C;
    if (fast_shape(x, y, indices, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)) {
        constexpr int RS = 4;
        const long long items = planes * ceil_div(oH, RS) * (oW / 4);
        fwd_k3s2p1_kernel<RS><<<grid_for(items), 256, 0, stream>>>(x, y, (long long *)indices, H, W, oH, oW, planes);
        CUNN_LAUNCH_CHECK("maxpool forward (3x3 s2 p1)");
        return 0;
    }
    const long long total = planes * oH * oW;
    forward_taps_kernel<float><<<grid_for(total), 256, 0, stream>>>(x, y, (long long *)indices, H, W, oH, oW, kH, kW, dH, dW,
                                                           padH, padW, dilH, dilW, total);
    CUNN_LAUNCH_CHECK("maxpool forward (generic)");
    return 0;
}

extern "C" CUNN_API int cunn_b200_maxpool_backward(const float *gy, const int64_t *indices, float *gx, int N, int C,
                                                   int H, int W, int kH, int kW, int dH, int dW, int padH, int padW,
                                                   int dilH, int dilW, int ceil_mode, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, kH, kW, dH, dW, padH, padW, dilH, dilW, ceil_mode, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && gx && indices, "null tensor pointer");
    const long long planes = (long long)N * C;
    if (fast_shape(gy, gx, indices, H, W, oH, oW, kH, kW, dH, dW, padH, padW, dilH, dilW)) {
        const long long items = planes * ((H + 1) / 2) * (W / 8);
        bwd_k3s2p1_kernel<<<grid_for(items), 256, 0, stream>>>(gy, (const long long *)indices, gx, H, W, oH, oW, planes);
        CUNN_LAUNCH_CHECK("maxpool backward (3x3 s2 p1)");
        return 0;
    }
    const long long total = planes * H * W;
    backward_taps_kernel<float><<<grid_for(total), 256, 0, stream>>>(gy, (const long long *)indices, gx, H, W, oH, oW, kH, kW, dH,
                                                           dW, padH, padW, dilH, dilW, total);
    CUNN_LAUNCH_CHECK("maxpool backward (generic)");
    return 0;
}
