// Depthwise convolution for sm_100a: forward, input gradient, parameter gradient.
//
// Two families of kernels:
//  * shape-generic kernels (any kernel size, stride, padding, depth multiplier):
//    one thread per output element / input element, plain coalesced loads;
//  * the 3x3 / pad 1 / stride 1|2 / multiplier 1 fast path that MobileNet-style
//    networks use: each CTA owns a group of channels and a range of images, and
//    streams whole planes (or row bands of one plane) through a ring of shared
//    memory stages filled by 1-D TMA bulk copies (cp.async.bulk + mbarrier).
//    Threads slide a 3-row register window down a strip of output rows, so each
//    staged input row is read from shared memory about once, and write results
//    with 16-byte stores.  The parameter-gradient kernel keeps its ten running
//    sums (nine taps and the bias) in registers across all tiles of the CTA and
//    writes one partial per (CTA, channel); a second tiny kernel adds the
//    partials in a fixed order in fp64, so results do not depend on scheduling.
//
// All three operations are HBM-bound: per element of x and y they move 4 bytes
// each way and do nine FMAs.
#include "common.cuh"

#include <algorithm>

namespace cunn {
namespace dw {

// ---------------------------------------------------------------------------
// Shape-generic kernels
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
fwd_generic_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                   float *__restrict__ y, int C, int H, int W, int M, int kH, int kW, int dH, int dW,
                   int padH, int padW, int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(idx % oW);
        long long t = idx / oW;
        const int oh = (int)(t % oH);
        t /= oH;
        const int j = (int)(t % M);
        t /= M;
        const int c = (int)(t % C);
        const long long n = t / C;
        const float *xp = x + (n * C + c) * (long long)H * W;
        const float *wp = w + ((long long)j * C + c) * kH * kW;
        float s = bias ? __ldg(bias + (long long)j * C + c) : 0.f;
        const int ih0 = oh * dH - padH, iw0 = ow * dW - padW;
        for (int kh = 0; kh < kH; ++kh) {
            const int ih = ih0 + kh;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < kW; ++kw) {
                const int iw = iw0 + kw;
                if (iw < 0 || iw >= W) continue;
                s = fmaf(__ldg(wp + kh * kW + kw), __ldg(xp + ih * W + iw), s);
            }
        }
        y[idx] = s;
    }
}

__global__ void __launch_bounds__(256)
dgrad_generic_kernel(const float *__restrict__ gy, const float *__restrict__ w, float *__restrict__ gx,
                     int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                     int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int wi = (int)(idx % W);
        long long t = idx / W;
        const int h = (int)(t % H);
        t /= H;
        const int c = (int)(t % C);
        const long long n = t / C;
        float s = 0.f;
        for (int j = 0; j < M; ++j) {
            const float *wp = w + ((long long)j * C + c) * kH * kW;
            const float *gp = gy + ((n * C + c) * M + j) * (long long)oH * oW;
            for (int kh = 0; kh < kH; ++kh) {
                const int a = h + padH - kh;
                if (a < 0 || a % dH) continue;
                const int oh = a / dH;
                if (oh >= oH) continue;
                for (int kw = 0; kw < kW; ++kw) {
                    const int b = wi + padW - kw;
                    if (b < 0 || b % dW) continue;
                    const int ow = b / dW;
                    if (ow >= oW) continue;
                    s = fmaf(__ldg(wp + kh * kW + kw), __ldg(gp + oh * oW + ow), s);
                }
            }
        }
        gx[idx] = s;
    }
}

// One CTA per (j, c, tap) with tap == kH*kW meaning the bias sum.  Reduces over
// all images and output positions in fp32 per thread, fp64 across threads.
__global__ void __launch_bounds__(256)
wgrad_generic_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ gw,
                     float *__restrict__ gb, int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW,
                     int padH, int padW, int oH, int oW, float scale)
{
    const int kk = kH * kW;
    const int tap = blockIdx.x % (kk + 1);
    const int jc = blockIdx.x / (kk + 1);
    const int j = jc / C, c = jc % C;
    if (tap == kk && gb == nullptr) return;
    const int kh = tap / kW, kw = tap % kW;
    const int ohw = oH * oW;
    double acc = 0.0;
    for (int n = 0; n < N; ++n) {
        const float *xp = x + ((long long)n * C + c) * H * W;
        const float *gp = gy + (((long long)n * C + c) * M + j) * ohw;
        float part = 0.f;
        for (int i = threadIdx.x; i < ohw; i += blockDim.x) {
            const float g = __ldg(gp + i);
            if (tap == kk) {
                part += g;
            } else {
                const int ih = (i / oW) * dH - padH + kh, iw = (i % oW) * dW - padW + kw;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) part = fmaf(g, __ldg(xp + ih * W + iw), part);
            }
        }
        acc += (double)part;
    }
    __shared__ double red[8];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
        if (tap == kk) gb[(long long)j * C + c] = (float)((double)gb[(long long)j * C + c] + (double)scale * s);
        else           gw[((long long)j * C + c) * kk + tap] = (float)((double)gw[((long long)j * C + c) * kk + tap] + (double)scale * s);
    }
}

// ---------------------------------------------------------------------------
// 3x3 fast path
// ---------------------------------------------------------------------------
//
// Work decomposition.  A tile is P whole planes (consecutive channels of one image) or, for planes
// too large for a stage, a band of R output rows of one plane.  Tiles are numbered group-major
// (group = P consecutive channels), then image, then band; every CTA of the persistent grid takes a
// contiguous, equal share of that sequence.  Inside a tile each thread owns one work item
// (plane, strip of RS output rows, group of VEC output columns) and slides a three-row register
// window down its strip.
//
// Data movement.  Input tiles are contiguous in NCHW memory, so one thread fetches each with a single
// 1-D TMA bulk copy into a ring of shared-memory stages (mbarrier completion, bounded waits).
// Results go out either as 16-byte global stores straight from registers (VEC == 4) or, for row
// lengths that cannot be vectorised (7, 14, ...), through a shared-memory copy of the output tile
// that one thread writes back with a TMA bulk store, so global writes are always full sectors.
//
// Parameter gradient.  Each thread keeps ten sums (nine taps, bias) in registers across all tiles of
// a channel group.  When the CTA leaves a group it reduces them per plane in shared memory, writes one
// partial per plane to the workspace and takes a ticket on the group's counter; the CTA that draws
// the last ticket adds all partials of the group in CTA order in fp64 and updates grad_weight /
// grad_bias.  The order is fixed, so results are bit-reproducible; no second kernel is needed.

enum Mode : int { MODE_FWD = 0, MODE_DGRAD_S2 = 1, MODE_WGRAD = 2 };

struct FastParams {
    const float *in;    // FWD: x (or gy when used as the stride-1 input gradient); DGRAD_S2: gy; WGRAD: x
    const float *in2;   // WGRAD: gy
    const float *w;     // [C][9]
    const float *bias;  // FWD only; may be null
    float *out;         // FWD: y; DGRAD_S2: gx
    float *gw, *gb;     // WGRAD: accumulated outputs (gb may be null)
    float *partials;    // WGRAD: [grid][maxseg][P][10]
    unsigned int *counters;  // WGRAD: one ticket counter per channel group, zero on entry and exit
    int *status;
    float scale;
    int N, C;
    int H, W;           // extent of the convolution's input side (x, gx)
    int oH, oW;         // extent of its output side (y, gy)
    int P;              // channels per tile (bands == 1 when P > 1)
    int bands;          // row bands per plane
    int R;              // driver rows (rows of y / gy) per band
    int RS;             // driver rows per thread strip
    int strips;         // ceil(R / RS)
    int CG;             // column groups per row = oW / VEC
    int items;          // P * strips * CG  (<= blockDim.x)
    int maxseg;         // WGRAD: partial slots per CTA (channel groups one CTA's tile range can touch)
    int tiles_base;     // every CTA takes tiles_base tiles of the sequence, the first tiles_rem CTAs one more
    int tiles_rem;
    int stages;
    int stage_floats;   // floats per stage for `in`
    int stage2_floats;  // floats per stage for `in2`
    int out_floats;     // floats per output staging buffer (two buffers), 0 when stores are direct
    int flip;           // FWD: use the 180-degree rotated kernel (stride-1 input gradient)
    int atomic_flush;   // WGRAD: add each CTA's per-plane sums to gw / gb with fp32 atomics (fast, order-dependent
                        // rounding) instead of the ticketed fixed-order reduction (bit-reproducible)
};

template <int S, int VEC>
struct Win {
    static constexpr int NV = (VEC - 1) * S + 3;  // input columns a thread needs per row
};

// Shared-memory loads on 32-bit shared-window addresses (cheaper address arithmetic than generic
// pointers).  volatile + memory clobber keeps them ordered with the mbarrier waits and barriers.
__device__ __forceinline__ float lds32(uint32_t a)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float2 lds64(uint32_t a)
{
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float4 lds128(uint32_t a)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}

// Loads the NV input values of one row that a column group needs; r is the shared address of the group's
// first interior column (column col0 of the row, or of the all-zero row for rows outside the plane).
// v[0] is column col0-1, v[NV-1] the last one; those two may lie outside the row and then read as zero.
template <int S, int VEC>
__device__ __forceinline__ void load_row(uint32_t r, bool has_left, bool has_right, float (&v)[Win<S, VEC>::NV])
{
    constexpr int NV = Win<S, VEC>::NV;
    v[0] = 0.f;
    if (has_left) v[0] = lds32(r - 4);
    if (VEC == 4 && S == 1) {
        const float4 q = lds128(r);
        v[1] = q.x; v[2] = q.y; v[3] = q.z; v[4] = q.w;
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = lds32(r + 16);
    } else if (VEC == 4 && S == 2) {
        const float4 q0 = lds128(r);
        const float4 q1 = lds128(r + 16);
        v[1] = q0.x; v[2] = q0.y; v[3] = q0.z; v[4] = q0.w;
        v[5] = q1.x; v[6] = q1.y; v[7] = q1.z; v[NV - 1] = q1.w;
    } else if (VEC == 2 && S == 1) {
        const float2 q = lds64(r);
        v[1] = q.x; v[2] = q.y;
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = lds32(r + 8);
    } else if (VEC == 2 && S == 2) {
        const float4 q = lds128(r);
        v[1] = q.x; v[2] = q.y; v[3] = q.z; v[NV - 1] = q.w;
    } else {
#pragma unroll
        for (int i = 1; i < NV - 1; ++i) v[i] = lds32(r + 4 * (i - 1));
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = lds32(r + 4 * (NV - 2));
    }
}

template <int VEC>
__device__ __forceinline__ void load_vec(uint32_t a, float (&g)[VEC])
{
    if (VEC == 4) {
        const float4 q = lds128(a);
        g[0] = q.x; g[1] = q.y; g[2] = q.z; g[3] = q.w;
    } else if (VEC == 2) {
        const float2 q = lds64(a);
        g[0] = q.x; g[1] = q.y;
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) g[i] = lds32(a + 4 * i);
    }
}

// The same two loaders on global memory (read-only path), for the variant that skips shared memory.
template <int S, int VEC>
__device__ __forceinline__ void load_row_g(const float *r, bool valid, bool has_left, bool has_right,
                                           float (&v)[Win<S, VEC>::NV])
{
    constexpr int NV = Win<S, VEC>::NV;
    if (!valid) {
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = 0.f;
        return;
    }
    v[0] = 0.f;
    if (has_left) v[0] = __ldg(r - 1);
    if (VEC == 4 && S == 1) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(r));
        v[1] = q.x; v[2] = q.y; v[3] = q.z; v[4] = q.w;
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = __ldg(r + 4);
    } else if (VEC == 4 && S == 2) {
        const float4 q0 = __ldg(reinterpret_cast<const float4 *>(r));
        const float4 q1 = __ldg(reinterpret_cast<const float4 *>(r + 4));
        v[1] = q0.x; v[2] = q0.y; v[3] = q0.z; v[4] = q0.w;
        v[5] = q1.x; v[6] = q1.y; v[7] = q1.z; v[NV - 1] = q1.w;
    } else if (VEC == 2 && S == 1) {
        const float2 q = __ldg(reinterpret_cast<const float2 *>(r));
        v[1] = q.x; v[2] = q.y;
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = __ldg(r + 2);
    } else if (VEC == 2 && S == 2) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(r));
        v[1] = q.x; v[2] = q.y; v[3] = q.z; v[NV - 1] = q.w;
    } else {
#pragma unroll
        for (int i = 1; i < NV - 1; ++i) v[i] = __ldg(r + i - 1);
        v[NV - 1] = 0.f;
        if (has_right) v[NV - 1] = __ldg(r + NV - 2);
    }
}

template <int VEC>
__device__ __forceinline__ void load_vec_g(const float *p, float (&g)[VEC])
{
    if (VEC == 4) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(p));
        g[0] = q.x; g[1] = q.y; g[2] = q.z; g[3] = q.w;
    } else if (VEC == 2) {
        const float2 q = __ldg(reinterpret_cast<const float2 *>(p));
        g[0] = q.x; g[1] = q.y;
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) g[i] = __ldg(p + i);
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float *p, const float (&o)[VEC])
{
    if (VEC == 4) *reinterpret_cast<float4 *>(p) = make_float4(o[0], o[1], o[2], o[3]);
    else if (VEC == 2) *reinterpret_cast<float2 *>(p) = make_float2(o[0], o[1]);
    else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) p[i] = o[i];
    }
}

// Geometry of a tile: which channel group and image, which rows are staged.
struct Tile {
    int g;              // channel group
    int n, d0, d1;      // image, driver-row range [d0, d1)
    int r0, r1;         // staged rows of `in` [r0, r1)
};

// Position in the tile sequence, which runs group-major, then image, then band:
// t = (g * N + n) * bands + band.  Advanced incrementally; divisions happen once per CTA.
struct Cursor {
    int g, n, band;
};

__device__ __forceinline__ Cursor cursor_at(const FastParams &p, int t)
{
    Cursor c;
    const int tpg = p.N * p.bands;
    c.g = t / tpg;
    const int r = t - c.g * tpg;
    c.n = r / p.bands;
    c.band = r - c.n * p.bands;
    return c;
}

__device__ __forceinline__ void cursor_next(const FastParams &p, Cursor &c)
{
    if (++c.band == p.bands) {
        c.band = 0;
        if (++c.n == p.N) {
            c.n = 0;
            ++c.g;
        }
    }
}

template <int MODE, int S>
__device__ __forceinline__ Tile tile_of(const FastParams &p, const Cursor &c)
{
    Tile tl;
    tl.g = c.g;
    tl.n = c.n;
    tl.d0 = c.band * p.R;
    tl.d1 = min(p.oH, tl.d0 + p.R);
    if (p.bands == 1) {  // whole planes
        tl.r0 = 0;
        tl.r1 = (MODE == MODE_DGRAD_S2) ? p.oH : p.H;
    } else if (MODE == MODE_DGRAD_S2) {
        tl.r0 = tl.d0;
        tl.r1 = min(p.oH, tl.d1 + 1);
    } else {
        tl.r0 = max(0, tl.d0 * S - 1);
        tl.r1 = min(p.H, (tl.d1 - 1) * S + 2);
    }
    return tl;
}

template <int MODE, int S>
__device__ __forceinline__ void issue_tile(const FastParams &p, const Tile &tl, float *stage_in, float *stage_in2,
                                           uint32_t bar)
{
    const int c0 = tl.g * p.P;
    const int rows = (MODE == MODE_DGRAD_S2) ? p.oH : p.H;
    const int cols = (MODE == MODE_DGRAD_S2) ? p.oW : p.W;
    const long long plane0 = (long long)tl.n * p.C + c0;
    const float *src = p.in + (plane0 * rows + tl.r0) * cols;
    const uint32_t bytes = (uint32_t)((p.bands == 1 ? p.P * rows * cols : (tl.r1 - tl.r0) * cols) * 4);
    uint32_t total = bytes;
    const float *src2 = nullptr;
    uint32_t bytes2 = 0;
    if (MODE == MODE_WGRAD) {
        src2 = p.in2 + (plane0 * p.oH + tl.d0) * p.oW;
        bytes2 = (uint32_t)((p.bands == 1 ? p.P * p.oH * p.oW : (tl.d1 - tl.d0) * p.oW) * 4);
        total += bytes2;
    }
    mbar_arrive_expect_tx(bar, total);
    bulk_g2s(smem_u32(stage_in), src, bytes, bar);
    if (MODE == MODE_WGRAD) bulk_g2s(smem_u32(stage_in2), src2, bytes2, bar);
}

// The tile sequence is split evenly: CTA b owns tiles [cta_begin(b), cta_begin(b + 1)).
__device__ __forceinline__ int cta_begin(const FastParams &p, int b) { return b * p.tiles_base + min(b, p.tiles_rem); }
__device__ __forceinline__ int cta_of_tile(const FastParams &p, int t)
{
    const int big = p.tiles_rem * (p.tiles_base + 1);  // tiles owned by the CTAs that hold one extra
    return t < big ? t / (p.tiles_base + 1) : p.tiles_rem + (t - big) / p.tiles_base;
}

// Hands in the ten running sums of the channel group `g` this CTA just finished: per-plane reduction
// in shared memory -> partial slot of (this CTA, g) -> ticket; the last ticket holder of the group
// folds every CTA's partial into gw / gb in CTA order.
__device__ __forceinline__ void wgrad_flush(const FastParams &p, const float (&acc)[10], float *red, int *flag,
                                            bool active, int per_plane, int g, int g_first)
{
    const int tid = threadIdx.x;
    __syncthreads();
    if (active) {
#pragma unroll
        for (int k = 0; k < 10; ++k) red[tid * 10 + k] = acc[k];
    }
    __syncthreads();
    // One thread per (plane, sum) pair adding the plane's items serially, or (long planes, few pairs) one
    // warp per pair with a shuffle reduction.
    const int npairs = p.P * 10;
    const bool serial = per_plane <= 16 || ((npairs + (int)blockDim.x - 1) / (int)blockDim.x) * per_plane <= 96;
    if (p.atomic_flush) {
        // fire-and-forget: scale * (sum over this CTA's items of the plane) straight into gw / gb
        const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
        if (serial) {
            for (int pair = tid; pair < p.P * 10; pair += blockDim.x) {
                const int ppl = pair / 10, k = pair - ppl * 10;
                const float *r = red + ppl * per_plane * 10 + k;
                float s0 = 0.f, s1 = 0.f;
                int i = 0;
                for (; i + 1 < per_plane; i += 2) { s0 += r[i * 10]; s1 += r[i * 10 + 10]; }
                if (i < per_plane) s0 += r[i * 10];
                const float s = s0 + s1;
                const int c = g * p.P + ppl;
                if (k < 9) atomicAdd(p.gw + (size_t)c * 9 + k, p.scale * s);
                else if (p.gb) atomicAdd(p.gb + c, p.scale * s);
            }
        } else {
            for (int pair = warp; pair < p.P * 10; pair += nwarps) {
                const int ppl = pair / 10, k = pair - ppl * 10;
                float s = 0.f;
                for (int i = lane; i < per_plane; i += 32) s += red[(ppl * per_plane + i) * 10 + k];
                s = warp_sum(s);
                const int c = g * p.P + ppl;
                if (lane == 0) {
                    if (k < 9) atomicAdd(p.gw + (size_t)c * 9 + k, p.scale * s);
                    else if (p.gb) atomicAdd(p.gb + c, p.scale * s);
                }
            }
        }
        return;
    }
    float *slot = p.partials + ((size_t)blockIdx.x * p.maxseg + (g - g_first)) * p.P * 10;
    if (serial) {
        for (int pair = tid; pair < p.P * 10; pair += blockDim.x) {
            const int ppl = pair / 10, k = pair - ppl * 10;
            const float *r = red + ppl * per_plane * 10 + k;
            float s = 0.f;
            for (int i = 0; i < per_plane; ++i) s += r[i * 10];
            __stcg(slot + pair, s);
        }
    } else {
        const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
        for (int pair = warp; pair < p.P * 10; pair += nwarps) {
            const int ppl = pair / 10, k = pair - ppl * 10;
            float s = 0.f;
            for (int i = lane; i < per_plane; i += 32) s += red[(ppl * per_plane + i) * 10 + k];
            s = warp_sum(s);
            if (lane == 0) __stcg(slot + pair, s);
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        // CTAs whose tile range meets this group's tiles [lo, lo + tpg)
        const int tpg = p.N * p.bands;
        const int lo = g * tpg;
        const int b_lo = cta_of_tile(p, lo), b_hi = cta_of_tile(p, lo + tpg - 1);
        const unsigned int ticket = atomicAdd(p.counters + g, 1u);
        flag[0] = (ticket == (unsigned int)(b_hi - b_lo)) ? 1 : 0;
        flag[1] = b_lo;
        flag[2] = b_hi;
        flag[3] = g - cta_begin(p, b_lo) / tpg;  // slot of group g inside CTA b_lo; every later CTA starts in g
    }
    __syncthreads();
    if (flag[0]) {
        __threadfence();
        const int b_lo = flag[1], b_hi = flag[2], seg_lo = flag[3];
        const size_t stride = (size_t)p.maxseg * p.P * 10;
        const int n10 = p.P * 10;
        const float *first = p.partials + b_lo * stride + (size_t)seg_lo * n10;   // CTA b_lo's slot of group g
        const float *rest = p.partials + (size_t)(b_lo + 1) * stride;             // later CTAs start inside g
        const int nrest = b_hi - b_lo;
        if ((n10 & 3) == 0) {
            // four sums per thread, 16-byte loads, several CTAs' partials in flight at once
            for (int q = tid * 4; q < n10; q += blockDim.x * 4) {
                const float4 f = __ldcg(reinterpret_cast<const float4 *>(first + q));
                double s0 = f.x, s1 = f.y, s2 = f.z, s3 = f.w;
#pragma unroll 8
                for (int b = 0; b < nrest; ++b) {
                    const float4 v = __ldcg(reinterpret_cast<const float4 *>(rest + b * stride + q));
                    s0 += (double)v.x; s1 += (double)v.y; s2 += (double)v.z; s3 += (double)v.w;
                }
                const double sv[4] = {s0, s1, s2, s3};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int idx = q + j, ppl = idx / 10, k = idx - ppl * 10;
                    const int c = g * p.P + ppl;
                    if (k < 9) p.gw[(size_t)c * 9 + k] = (float)((double)p.gw[(size_t)c * 9 + k] + (double)p.scale * sv[j]);
                    else if (p.gb) p.gb[c] = (float)((double)p.gb[c] + (double)p.scale * sv[j]);
                }
            }
        } else {
            for (int idx = tid; idx < n10; idx += blockDim.x) {
                const int ppl = idx / 10, k = idx - ppl * 10;
                const int c = g * p.P + ppl;
                double s = (double)__ldcg(first + idx);
#pragma unroll 8
                for (int b = 0; b < nrest; ++b) s += (double)__ldcg(rest + b * stride + idx);
                if (k < 9) p.gw[(size_t)c * 9 + k] = (float)((double)p.gw[(size_t)c * 9 + k] + (double)p.scale * s);
                else if (p.gb) p.gb[c] = (float)((double)p.gb[c] + (double)p.scale * s);
            }
        }
        if (tid == 0) p.counters[g] = 0u;  // leave the control words zero for the next call
    }
}

__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src_smem, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// DIRECT = true skips the shared-memory ring: rows are read straight from global memory through the
// read-only path (L1 absorbs the halo re-reads) and nothing in the tile loop synchronises the CTA.
template <int MODE, int S, int VEC, bool STAGE_OUT, bool DIRECT>
__global__ void __launch_bounds__(256)
fast_kernel(const FastParams p)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NV = Win<S, VEC>::NV;

    // smem: in stages | in2 stages | out buffers (2) | zero row | barriers | flag | reduction scratch (WGRAD)
    float *in_s = reinterpret_cast<float *>(smem_raw);
    float *in2_s = in_s + (size_t)p.stages * p.stage_floats;
    float *out_s = in2_s + (size_t)p.stages * p.stage2_floats;
    float *zrow_base = out_s + 2 * (size_t)p.out_floats;
    const int zlen = ((MODE == MODE_DGRAD_S2 ? p.oW : p.W) + 8 + 31) & ~31;
    uint64_t *bars = reinterpret_cast<uint64_t *>(zrow_base + zlen);
    int *flag = reinterpret_cast<int *>(bars + p.stages);
    float *red = reinterpret_cast<float *>(flag + 4);

    // Persistent CTA: a contiguous, balanced range of the global tile sequence.
    const int t_begin = cta_begin(p, blockIdx.x);
    const int T = p.tiles_base + ((int)blockIdx.x < p.tiles_rem ? 1 : 0);
    Cursor cur = cursor_at(p, t_begin);
    const int g_first = cur.g;

    const int tid = threadIdx.x;
    // Programmatic dependent launch: let the next kernel in the stream start its prologue while this grid
    // drains, and do this kernel's own shared-memory set-up before waiting for the previous grid.  Nothing
    // before pdl_wait() touches global memory.
    pdl_launch_dependents();
    for (int i = tid; i < zlen; i += blockDim.x) zrow_base[i] = 0.f;
    if (!DIRECT && tid == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();
    Cursor pre = cur;  // thread 0: cursor of the next tile to fetch
    if (!DIRECT && tid == 0) {
        const int npre = min(T, p.stages);
        for (int i = 0; i < npre; ++i) {
            const Tile tl = tile_of<MODE, S>(p, pre);
            issue_tile<MODE, S>(p, tl, in_s + (size_t)i * p.stage_floats, in2_s + (size_t)i * p.stage2_floats,
                                smem_u32(bars + i));
            cursor_next(p, pre);
        }
    }

    // static work item of this thread
    const bool active = tid < p.items;
    const int per_plane = p.strips * p.CG;
    const int pl = active ? tid / per_plane : 0;
    const int rem = active ? tid - pl * per_plane : 0;
    const int strip = rem / p.CG;
    const int cg = rem - strip * p.CG;
    const float *zrow = zrow_base + 4;  // one spare float on the left for the (never selected) halo read

    float wk[9];
    float bias = 0.f;
    float acc[10];
#pragma unroll
    for (int i = 0; i < 10; ++i) acc[i] = 0.f;
    int cur_g = -1;
    int c = 0;
    int st = 0;            // stage of the current tile and the parity of its barrier phase
    uint32_t phase = 0;

    for (int t = 0; t < T; ++t) {
        const Tile tl = tile_of<MODE, S>(p, cur);
        if (tl.g != cur_g) {
            // entering a new channel group: fetch its weights, or (WGRAD) hand in the sums of the last one
            if (MODE == MODE_WGRAD && cur_g >= 0) {
                wgrad_flush(p, acc, red, flag, active, per_plane, cur_g, g_first);
#pragma unroll
                for (int i = 0; i < 10; ++i) acc[i] = 0.f;
            }
            cur_g = tl.g;
            c = cur_g * p.P + pl;
            if (MODE != MODE_WGRAD) {
#pragma unroll
                for (int i = 0; i < 9; ++i)
                    wk[i] = __ldg(p.w + (size_t)c * 9 + ((MODE == MODE_FWD && p.flip) ? 8 - i : i));
                if (MODE == MODE_FWD && p.bias) bias = __ldg(p.bias + c);
            }
        }
        if (!DIRECT) {
            if (!mbar_wait(smem_u32(bars + st), phase, p.status)) return;
        }
        const int dbeg = tl.d0 + strip * p.RS;
        const int dend = min(tl.d1, dbeg + p.RS);
        float *os = out_s + (size_t)(t & 1) * p.out_floats;

        if (active && dbeg < dend) {
            if (MODE == MODE_FWD || MODE == MODE_WGRAD) {
                const int W = p.W, H = p.H, oW = p.oW;
                const int col0 = cg * VEC * S;
                const bool has_left = col0 > 0;
                const bool has_right = col0 + NV - 2 < W;
                // shared address of column col0 of plane row `row` is row_base + row * 4W
                const uint32_t row_base = smem_u32(in_s + (size_t)st * p.stage_floats) + (uint32_t)(((pl * H - tl.r0) * W + col0) * 4);
                const uint32_t zr = smem_u32(zrow) + (uint32_t)(col0 * 4);
                const uint32_t W4 = (uint32_t)W * 4u;
                const float *gbase = nullptr;   // DIRECT: column col0 of row 0 of this thread's plane
                const float *gyg = nullptr;     // DIRECT, WGRAD: this thread's gy columns of row dbeg
                if (DIRECT) {
                    gbase = p.in + (((size_t)tl.n * p.C + c) * H) * W + col0;
                    if (MODE == MODE_WGRAD) gyg = p.in2 + (((size_t)tl.n * p.C + c) * p.oH + dbeg) * oW + cg * VEC;
                }
                auto ldrow = [&](int row, uint32_t saddr, float (&r)[NV]) {
                    if (DIRECT) load_row_g<S, VEC>(gbase + (ptrdiff_t)row * W, (unsigned)row < (unsigned)H, has_left, has_right, r);
                    else load_row<S, VEC>(saddr, has_left, has_right, r);
                };
                float *yp = nullptr;
                float *osp = nullptr;
                uint32_t gp = 0;
                if (MODE == MODE_FWD) {
                    if (STAGE_OUT) osp = os + (pl * p.oH - tl.d0 + dbeg) * oW + cg * VEC;
                    else yp = p.out + (((size_t)tl.n * p.C + c) * p.oH + dbeg) * oW + cg * VEC;
                } else {
                    gp = smem_u32(in2_s + (size_t)st * p.stage2_floats) + (uint32_t)((((pl * p.oH - tl.d0 + dbeg) * oW) + cg * VEC) * 4);
                }
                // one output row from the three window rows; advances the output / gy cursor by one row
                auto compute = [&](const float (&ra)[NV], const float (&rb)[NV], const float (&rc)[NV]) {
                    if (MODE == MODE_FWD) {
                        float ov[VEC];
#pragma unroll
                        for (int v = 0; v < VEC; ++v) {
                            float s = bias;
#pragma unroll
                            for (int kw = 0; kw < 3; ++kw) {
                                s = fmaf(wk[kw], ra[v * S + kw], s);
                                s = fmaf(wk[3 + kw], rb[v * S + kw], s);
                                s = fmaf(wk[6 + kw], rc[v * S + kw], s);
                            }
                            ov[v] = s;
                        }
                        if (STAGE_OUT) {
#pragma unroll
                            for (int v = 0; v < VEC; ++v) osp[v] = ov[v];
                            osp += oW;
                        } else {
                            store_vec<VEC>(yp, ov);
                            yp += oW;
                        }
                    } else {
                        float g[VEC];
                        if (DIRECT) {
                            load_vec_g<VEC>(gyg, g);
                            gyg += oW;
                        } else {
                            load_vec<VEC>(gp, g);
                            gp += (uint32_t)oW * 4u;
                        }
#pragma unroll
                        for (int v = 0; v < VEC; ++v) {
#pragma unroll
                            for (int kw = 0; kw < 3; ++kw) {
                                acc[kw] = fmaf(g[v], ra[v * S + kw], acc[kw]);
                                acc[3 + kw] = fmaf(g[v], rb[v * S + kw], acc[3 + kw]);
                                acc[6 + kw] = fmaf(g[v], rc[v * S + kw], acc[6 + kw]);
                            }
                            acc[9] += g[v];
                        }
                    }
                };
                float r0[NV], r1[NV], r2[NV];
                const int n_out = dend - dbeg;
                if (S == 1) {
                    // window rows (o-1, o, o+1); roles rotate so no register copies are needed.  Only the
                    // first row (above the plane) and the last one (below it) can be outside.
                    uint32_t rp = row_base + (uint32_t)(dbeg - 1) * W4;
                    ldrow(dbeg - 1, dbeg > 0 ? rp : zr, r0);
                    rp += W4;
                    ldrow(dbeg, rp, r1);
                    const bool bottom_out = dend >= H;   // row `dend` is below the plane
                    for (int i = 0; i < n_out; i += 3) {
                        rp += W4;
                        ldrow(dbeg + i + 1, (i + 1 == n_out && bottom_out) ? zr : rp, r2);
                        compute(r0, r1, r2);
                        if (i + 1 >= n_out) break;
                        rp += W4;
                        ldrow(dbeg + i + 2, (i + 2 == n_out && bottom_out) ? zr : rp, r0);
                        compute(r1, r2, r0);
                        if (i + 2 >= n_out) break;
                        rp += W4;
                        ldrow(dbeg + i + 3, (i + 3 == n_out && bottom_out) ? zr : rp, r1);
                        compute(r2, r0, r1);
                    }
                } else {
                    // window rows (2o-1, 2o, 2o+1); the last row is the next window's first.  Row 2o+1 of the
                    // last output row is below the plane when H is odd.
                    uint32_t rp = row_base + (uint32_t)(dbeg * 2 - 1) * W4;
                    ldrow(dbeg * 2 - 1, dbeg > 0 ? rp : zr, r0);
                    const bool bottom_out = 2 * dend - 1 >= H;
                    for (int i = 0; i < n_out; i += 2) {
                        ldrow((dbeg + i) * 2, rp + W4, r1);
                        rp += 2 * W4;
                        ldrow((dbeg + i) * 2 + 1, (i + 1 == n_out && bottom_out) ? zr : rp, r2);
                        compute(r0, r1, r2);
                        if (i + 1 >= n_out) break;
                        ldrow((dbeg + i) * 2 + 2, rp + W4, r1);
                        rp += 2 * W4;
                        ldrow((dbeg + i) * 2 + 3, (i + 2 == n_out && bottom_out) ? zr : rp, r0);
                        compute(r2, r1, r0);
                    }
                }
            } else {
                // Stride-2 input gradient: gy row a feeds gx rows 2a and 2a+1.
                // gx[2a  ][2b  ] = w11 G0[b]
                // gx[2a  ][2b+1] = w10 G0[b+1] + w12 G0[b]
                // gx[2a+1][2b  ] = w01 G1[b]   + w21 G0[b]
                // gx[2a+1][2b+1] = w00 G1[b+1] + w02 G1[b] + w20 G0[b+1] + w22 G0[b]
                // with G0 = gy row a, G1 = gy row a+1 (zero beyond the plane).
                const int oW = p.oW, oH = p.oH, W = p.W, H = p.H;
                const int b0 = cg * VEC;
                const bool has_right = b0 + VEC < oW;
                const uint32_t row_base = smem_u32(in_s + (size_t)st * p.stage_floats) + (uint32_t)(((pl * oH - tl.r0) * oW + b0) * 4);
                const uint32_t zr = smem_u32(zrow) + (uint32_t)(b0 * 4);
                float *xp = nullptr;
                float *osp = nullptr;
                if (STAGE_OUT) osp = os + pl * H * W + 2 * b0;
                else xp = p.out + (((size_t)tl.n * p.C + c) * H) * W + 2 * b0;
                const float *gbase = DIRECT ? p.in + (((size_t)tl.n * p.C + c) * oH) * oW + b0 : nullptr;
                auto load_g = [&](int a, float (&G)[VEC + 1]) {
                    float tmp[VEC];
                    if (DIRECT) {
                        if (a < oH) {
                            const float *r = gbase + (ptrdiff_t)a * oW;
                            load_vec_g<VEC>(r, tmp);
                            G[VEC] = 0.f;
                            if (has_right) G[VEC] = __ldg(r + VEC);
                        } else {
#pragma unroll
                            for (int v = 0; v < VEC; ++v) tmp[v] = 0.f;
                            G[VEC] = 0.f;
                        }
                    } else {
                        const uint32_t r = (a < oH) ? row_base + (uint32_t)(a * oW * 4) : zr;
                        load_vec<VEC>(r, tmp);
                        G[VEC] = 0.f;
                        if (has_right) G[VEC] = lds32(r + 4 * VEC);
                    }
#pragma unroll
                    for (int v = 0; v < VEC; ++v) G[v] = tmp[v];
                };
                auto emit = [&](int a, const float (&G0)[VEC + 1], const float (&G1)[VEC + 1]) {
                    float e[2 * VEC], o2[2 * VEC];
#pragma unroll
                    for (int v = 0; v < VEC; ++v) {
                        e[2 * v] = wk[4] * G0[v];
                        e[2 * v + 1] = fmaf(wk[3], G0[v + 1], wk[5] * G0[v]);
                        o2[2 * v] = fmaf(wk[1], G1[v], wk[7] * G0[v]);
                        o2[2 * v + 1] = fmaf(wk[0], G1[v + 1], fmaf(wk[2], G1[v], fmaf(wk[6], G0[v + 1], wk[8] * G0[v])));
                    }
                    // W is even on this path, so all 2*VEC columns exist; row 2a+1 may not (odd H)
                    float *dst = STAGE_OUT ? osp + 2 * a * W : xp + (size_t)(2 * a) * W;
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        if (2 * a + rr < H) {
                            const float *src = rr ? o2 : e;
                            float *d = dst + rr * W;
                            if (STAGE_OUT) {
#pragma unroll
                                for (int q = 0; q < 2 * VEC; ++q) d[q] = src[q];
                            } else if ((2 * VEC) % 4 == 0) {
#pragma unroll
                                for (int q = 0; q < 2 * VEC; q += 4)
                                    *reinterpret_cast<float4 *>(d + q) = make_float4(src[q], src[q + 1], src[q + 2], src[q + 3]);
                            } else {
#pragma unroll
                                for (int q = 0; q < 2 * VEC; q += 2)
                                    *reinterpret_cast<float2 *>(d + q) = make_float2(src[q], src[q + 1]);
                            }
                        }
                    }
                };
                float GA[VEC + 1], GB[VEC + 1];
                load_g(dbeg, GA);
                for (int a = dbeg; a < dend; a += 2) {
                    load_g(a + 1, GB);
                    emit(a, GA, GB);
                    if (a + 1 >= dend) break;
                    load_g(a + 2, GA);
                    emit(a + 1, GB, GA);
                }
            }
        }
        if (STAGE_OUT) {
            fence_async_smem();               // make this thread's staged outputs visible to the TMA unit
            if (tid == 0) bulk_wait_read0();  // the store issued one tile ago has left its buffer
        }
        if (!DIRECT) __syncthreads();  // every thread is done with stage st (and with the output buffer)
        if (!DIRECT && tid == 0) {
            if (STAGE_OUT) {
                const int rows_o = (MODE == MODE_DGRAD_S2) ? p.H : p.oH;
                const int cols_o = (MODE == MODE_DGRAD_S2) ? p.W : p.oW;
                float *dst = p.out + ((size_t)tl.n * p.C + (size_t)tl.g * p.P) * rows_o * cols_o;
                bulk_s2g(dst, smem_u32(os), (uint32_t)(p.P * rows_o * cols_o * 4));
            }
            if (t + p.stages < T) {
                const Tile nt = tile_of<MODE, S>(p, pre);
                issue_tile<MODE, S>(p, nt, in_s + (size_t)st * p.stage_floats, in2_s + (size_t)st * p.stage2_floats,
                                    smem_u32(bars + st));
                cursor_next(p, pre);
            }
        }
        cursor_next(p, cur);
        if (++st == p.stages) {
            st = 0;
            phase ^= 1u;
        }
    }
    if (STAGE_OUT && tid == 0) bulk_wait_read0();  // shared memory must outlive the last store's reads
    if (MODE == MODE_WGRAD && cur_g >= 0) wgrad_flush(p, acc, red, flag, active, per_plane, cur_g, g_first);
}

// ---------------------------------------------------------------------------
// Host side: tile planning and dispatch
// ---------------------------------------------------------------------------

static const int kMaxGroups = 16384;  // ticket counters in the parameter-gradient workspace

// Process-wide switch (cunn_b200_set_deterministic): 0 = parameter gradients are summed across CTAs with fp32
// atomics (default), 1 = with the ticketed fixed-order reduction, whose results are bit-reproducible.
static int g_deterministic = 0;

struct Tuning {
    int P = 0, R = 0, RS = 0, stages = 0, ctas_per_sm = 0, force_generic = 0, budget_kb = 0, vec = 0, stage_out = -1, direct = -1;
};
static thread_local Tuning g_tuning;

struct Plan {
    bool ok = false;
    int S = 1, VEC = 1;
    bool stage_out = false;
    bool direct = false;      // read rows straight from global memory instead of through the TMA ring
    int P = 1, bands = 1, R = 0, RS = 0, strips = 0, CG = 0, items = 0, threads = 0, stages = 0, grid = 1, maxseg = 1;
    int stage_floats = 0, stage2_floats = 0, out_floats = 0;
    size_t smem = 0;
    int mode = 0;
    long long tiles = 0;      // tiles in the whole problem
    int tiles_per_group = 0;  // tiles of one channel group
};

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

static bool vec_ok(int mode, int S, int VEC, int W, int oW)
{
    if (oW % VEC) return false;
    if (mode == MODE_DGRAD_S2) {
        // gy rows are read VEC at a time, gx rows written 2*VEC at a time
        if (VEC == 4) return false;  // 8 columns per thread would split every 32-byte sector over two stores
        if (VEC == 2) return oW % 2 == 0 && W % 4 == 0;
        return true;
    }
    if (S == 1) {
        if (VEC == 4) return W % 4 == 0;
        if (VEC == 2) return W % 2 == 0;
        return true;
    }
    if (VEC == 4 || VEC == 2) return W % 4 == 0 && W == 2 * oW;
    return true;
}

// Chooses VEC, the tile shape and the grid for the fast path, or returns ok = false when the
// shape cannot use it (then the generic kernels run).
static Plan make_plan(int mode, int N, int C, int H, int W, int oH, int oW, int S)
{
    Plan pl;
    pl.S = S;
    if (N <= 0 || C <= 0) return pl;
    if (mode == MODE_DGRAD_S2 && (W % 2)) return pl;  // paired column stores need an even row length

    const int in_rows = (mode == MODE_DGRAD_S2) ? oH : H;
    const int in_cols = (mode == MODE_DGRAD_S2) ? oW : W;
    const int out_rows = (mode == MODE_DGRAD_S2) ? H : oH;   // rows/cols of the tensor the kernel writes
    const int out_cols = (mode == MODE_DGRAD_S2) ? W : oW;
    const long long plane_in = (long long)in_rows * in_cols;  // floats
    const long long plane_in2 = (mode == MODE_WGRAD) ? (long long)oH * oW : 0;
    const long long plane_out = (mode == MODE_WGRAD) ? 0 : (long long)out_rows * out_cols;
    const long long budget = (g_tuning.budget_kb > 0 ? g_tuning.budget_kb : (mode == MODE_WGRAD ? 20 : 16)) * 1024 / 4;

    // Candidate column-group widths.  16-byte vectors are used whenever the row length allows them;
    // otherwise the widths that divide the row compete on estimated cost.
    int kVecs[4] = {0, 0, 0, 0};
    if (mode == MODE_DGRAD_S2) {
        if (vec_ok(mode, S, 2, W, oW)) kVecs[0] = 2;
        else { kVecs[0] = 7; kVecs[1] = 1; }
    } else {
        if (vec_ok(mode, S, 4, W, oW)) kVecs[0] = 4;
        else { kVecs[0] = 7; kVecs[1] = 2; kVecs[2] = 1; }
    }
    double best = -1.0;
    int bestVEC = 0, bestP = 0, bestRS = 0, bestR = 0;
    bool bestStage = false;
    for (int vi = 0; vi < 4; ++vi) {
        const int VEC = kVecs[vi];
        if (VEC == 0) continue;
        if (g_tuning.vec > 0 && VEC != g_tuning.vec) continue;
        if (!vec_ok(mode, S, VEC, W, oW)) continue;
        const int CG = oW / VEC;
        if (CG > 256) continue;
        const int NV = (mode == MODE_DGRAD_S2) ? VEC + 1 : (VEC - 1) * S + 3;
        // load instructions and shared-memory wavefronts (per warp) of one staged row
        int ld = NV, wf = NV * (S == 1 ? 1 : 2);
        if (mode != MODE_DGRAD_S2) {
            if (VEC == 4) { ld = 3; wf = (S == 1) ? 12 : 20; }
            else if (VEC == 2) { ld = (S == 1) ? 3 : 2; wf = (S == 1) ? 6 : 8; }
            else if (VEC == 1) { wf = (S == 1) ? 3 : 6; }
        } else {
            wf = VEC + 1;
            if (VEC == 2) { ld = 2; wf = 4; }
        }
        auto score = [&](int P, int R, int RS, bool staged) {
            const int strips = ceil_div(R, RS);
            const int items = P * strips * CG;
            if (items > 256) return -1.0;
            const int threads = std::max(64, round_up(items, 32));
            const double util = (double)items / threads * (double)R / (strips * RS);
            double rows_per_out, fma, st;
            if (mode == MODE_DGRAD_S2) {
                rows_per_out = (double)(RS + 1) / RS;
                fma = 9.0 * VEC;
                st = staged ? 4.0 * VEC : (VEC == 2 ? 2.0 : 2.0 * VEC);
            } else {
                rows_per_out = (double)(RS * S + 3 - S) / RS;
                fma = (mode == MODE_WGRAD ? 10.0 : 9.0) * VEC;
                const double vst = (VEC == 4 || VEC == 2) ? 1.0 : VEC;
                st = (mode == MODE_WGRAD) ? vst : (staged ? VEC : vst);
            }
            const double outs = (mode == MODE_DGRAD_S2) ? 4.0 * VEC : VEC;
            // issue slots and shared-memory wavefronts per output element
            const double instr = (ld * rows_per_out + fma + st + 8.0) / outs;
            const double waves = wf * rows_per_out / (32.0 * outs);
            // scalar and 8-byte shared loads weigh more than the 16-byte ones (measured on 14x14 and 7x7 planes)
            double cost = instr + (VEC == 4 ? 40.0 : 80.0) * waves;
            if (mode != MODE_WGRAD && !staged && VEC != 4 && !(mode == MODE_DGRAD_S2 && VEC == 2))
                cost *= 2.0;  // narrow direct stores fill sectors piecemeal
            const double size = std::min(1.0, items / 128.0);
            return util * (0.6 + 0.4 * size) / cost;
        };
        const bool want_stage = (mode != MODE_WGRAD) && (g_tuning.stage_out >= 0 ? g_tuning.stage_out != 0 : VEC != 4 && !(mode == MODE_DGRAD_S2 && VEC == 2));
        if (g_tuning.P > 0 && g_tuning.RS > 0) {
            const int R = (g_tuning.P > 1 || g_tuning.R <= 0) ? oH : g_tuning.R;
            const bool staged = want_stage && R >= oH;
            const double sc = score(g_tuning.P, R, g_tuning.RS, staged);
            if (sc > best) { best = sc; bestVEC = VEC; bestP = g_tuning.P; bestRS = g_tuning.RS; bestR = R; bestStage = staged; }
            continue;
        }
        const long long plane_all = plane_in + plane_in2 + (want_stage ? plane_out : 0);
        if (plane_all <= budget) {
            // whole planes, several channels per tile
            for (int P = 1; P <= C && P * plane_all <= budget; ++P) {
                if (C % P) continue;
                if ((P * plane_in) % 4 || (P * plane_in2) % 4) continue;
                bool staged = want_stage;
                if (staged && ((P * plane_out) % 4 || ((long long)C * plane_out) % 4)) staged = false;
                for (int RS = 1; RS <= std::min(oH, 16); ++RS) {
                    const double sc = score(P, oH, RS, staged);
                    if (sc > best) { best = sc; bestVEC = VEC; bestP = P; bestRS = RS; bestR = oH; bestStage = staged; }
                }
            }
        } else {
            // one plane in row bands (direct stores only)
            if (in_cols % 4 || (mode == MODE_WGRAD && oW % 4)) continue;
            for (int R = 2; R <= oH; ++R) {
                const long long rows_in = (mode == MODE_DGRAD_S2) ? R + 1 : (long long)(R - 1) * S + 3;
                if (rows_in * in_cols + (long long)R * (mode == MODE_WGRAD ? oW : 0) > budget) break;
                const int bands = ceil_div(oH, R);
                const double fill = (double)oH / (bands * R);
                // halo rows are fetched by both neighbouring bands
                const double halo = (double)(R * S) / (R * S + (mode == MODE_DGRAD_S2 ? 1 : 3 - S));
                for (int RS = 1; RS <= std::min(R, 16); ++RS) {
                    const double sc = score(1, R, RS, false) * fill * (0.5 + 0.5 * halo);
                    if (sc > best) { best = sc; bestVEC = VEC; bestP = 1; bestRS = RS; bestR = R; bestStage = false; }
                }
            }
        }
    }
    if (bestVEC <= 0 || bestP <= 0 || bestRS <= 0 || bestR <= 0) return pl;
    if (C % bestP) return pl;
    const bool direct_ok = (mode == MODE_DGRAD_S2) ? bestVEC == 2 : bestVEC == 4;
    pl.VEC = bestVEC;
    pl.CG = oW / pl.VEC;
    pl.P = bestP;
    pl.R = std::min(bestR, oH);
    pl.RS = bestRS;
    pl.bands = ceil_div(oH, pl.R);
    if (pl.P > 1 && pl.bands != 1) return pl;
    pl.stage_out = bestStage && pl.bands == 1;
    pl.strips = ceil_div(pl.R, pl.RS);
    pl.items = pl.P * pl.strips * pl.CG;
    if (pl.items > 256 || pl.items <= 0) return pl;
    pl.threads = std::max(64, round_up(pl.items, 32));
    // alignment of every bulk copy: plane-group base and band offsets multiples of 16 bytes
    if ((pl.P * plane_in) % 4 || (pl.P * plane_in2) % 4) return pl;
    if (((long long)C * plane_in) % 4 || ((long long)C * plane_in2) % 4) return pl;
    if (pl.bands > 1 && (in_cols % 4 || (mode == MODE_WGRAD && oW % 4))) return pl;
    if (pl.stage_out && ((pl.P * plane_out) % 4 || ((long long)C * plane_out) % 4)) return pl;
    if (!vec_ok(mode, S, pl.VEC, W, oW)) return pl;

    long long rows_in = (pl.bands == 1) ? in_rows : ((mode == MODE_DGRAD_S2) ? pl.R + 1 : (long long)(pl.R - 1) * S + 3);
    rows_in = std::min<long long>(rows_in, in_rows);
    pl.stage_floats = round_up((int)(pl.P * rows_in * in_cols), 32);
    pl.stage2_floats = (mode == MODE_WGRAD) ? round_up(pl.P * std::min(pl.R, oH) * oW, 32) : 0;
    pl.out_floats = pl.stage_out ? round_up((int)(pl.P * plane_out), 32) : 0;

    if (mode == MODE_WGRAD && C / pl.P > kMaxGroups) return pl;
    pl.mode = mode;
    pl.tiles = (long long)(C / pl.P) * N * pl.bands;
    if (pl.tiles >= (1LL << 30)) return pl;
    pl.tiles_per_group = N * pl.bands;
    pl.stages = g_tuning.stages > 0 ? g_tuning.stages : 4;
    pl.direct = direct_ok && !pl.stage_out && (g_tuning.direct >= 0 ? g_tuning.direct != 0 : false);
    if (pl.direct) {
        pl.stages = 0;
        pl.stage_floats = pl.stage2_floats = pl.out_floats = 0;
    }
    const size_t fixed = (size_t)2 * pl.out_floats * 4 + (size_t)round_up(in_cols + 8, 32) * 4 + 64 +
                         ((mode == MODE_WGRAD) ? (size_t)pl.items * 10 * 4 : 0);
    const size_t per_stage = (size_t)(pl.stage_floats + pl.stage2_floats) * 4 + 8;
    pl.smem = (size_t)pl.stages * per_stage + fixed;
    if (pl.smem > 200 * 1024) return pl;
    pl.ok = true;
    return pl;
}

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

typedef void (*FastKernel)(const FastParams);

template <int MODE, int S>
static FastKernel pick_kernel_s(int VEC, bool staged, bool direct)
{
    constexpr bool kCanStage = MODE != MODE_WGRAD;
    constexpr int kDirectVec = (MODE == MODE_DGRAD_S2) ? 2 : 4;
    if (direct) return VEC == kDirectVec ? (FastKernel)fast_kernel<MODE, S, kDirectVec, false, true> : nullptr;
    if (kCanStage && staged) {
        switch (VEC) {
            case 7: return fast_kernel<MODE, S, 7, kCanStage, false>;
            case 2: return fast_kernel<MODE, S, 2, kCanStage, false>;
            case 1: return fast_kernel<MODE, S, 1, kCanStage, false>;
            case 4: return MODE == MODE_DGRAD_S2 ? nullptr : (FastKernel)fast_kernel<MODE, S, kDirectVec, kCanStage, false>;
            default: return nullptr;
        }
    }
    switch (VEC) {
        case 7: return fast_kernel<MODE, S, 7, false, false>;
        case 2: return fast_kernel<MODE, S, 2, false, false>;
        case 1: return fast_kernel<MODE, S, 1, false, false>;
        case 4: return MODE == MODE_DGRAD_S2 ? nullptr : (FastKernel)fast_kernel<MODE, S, kDirectVec, false, false>;
        default: return nullptr;
    }
}

static FastKernel pick_kernel(const Plan &pl)
{
    switch (pl.mode) {
        case MODE_FWD: return pl.S == 2 ? pick_kernel_s<MODE_FWD, 2>(pl.VEC, pl.stage_out, pl.direct) : pick_kernel_s<MODE_FWD, 1>(pl.VEC, pl.stage_out, pl.direct);
        case MODE_DGRAD_S2: return pick_kernel_s<MODE_DGRAD_S2, 2>(pl.VEC, pl.stage_out, pl.direct);
        default: return pl.S == 2 ? pick_kernel_s<MODE_WGRAD, 2>(pl.VEC, false, pl.direct) : pick_kernel_s<MODE_WGRAD, 1>(pl.VEC, false, pl.direct);
    }
}

// Sizes the persistent grid: one wave of CTAs, as many per SM as the kernel's registers, threads and
// shared memory allow (asked of the runtime; estimated when no device is present), each taking an equal
// share of the tile sequence.
static int finalize_plan(Plan &pl)
{
    FastKernel kern = pick_kernel(pl);
    if (!kern) return fail("dwconv: no kernel for VEC=%d", pl.VEC);
    int occ = g_tuning.ctas_per_sm;
    if (occ <= 0) {
        bool asked = false;
        if (pl.smem <= 48 * 1024 ||
            cudaFuncSetAttribute((const void *)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) == cudaSuccess) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, (const void *)kern, pl.threads, pl.smem) == cudaSuccess && n > 0) {
                occ = n;
                asked = true;
            }
        }
        if (!asked) {
            (void)cudaGetLastError();
            const int by_smem = (int)((220 * 1024) / (pl.smem + 1024));
            occ = std::max(1, std::min(std::min(by_smem, 2048 / pl.threads), 65536 / (80 * pl.threads)));
        }
        occ = std::min(occ, 8);
    } else if (pl.smem > 48 * 1024) {
        (void)cudaFuncSetAttribute((const void *)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        (void)cudaGetLastError();
    }
    long long grid = (long long)sm_count() * occ;
    if (grid > pl.tiles) grid = pl.tiles;
    pl.grid = (int)std::max(1LL, grid);
    const long long range = ceil_div_ll(pl.tiles, pl.grid);
    pl.maxseg = (int)(ceil_div_ll(range, pl.tiles_per_group) + 1);
    return 0;
}

static int launch_fast(FastParams &fp, const Plan &pl, cudaStream_t stream, const char *name)
{
    FastKernel kern = pick_kernel(pl);
    if (!kern) return fail("dwconv: no kernel for VEC=%d", pl.VEC);
    fp.maxseg = pl.maxseg;
    fp.tiles_base = (int)(pl.tiles / pl.grid);
    fp.tiles_rem = (int)(pl.tiles % pl.grid);
    void *args[] = {(void *)&fp};
    // launched as a programmatic dependent of whatever precedes it in the stream: its prologue may overlap
    // the tail of the previous kernel; the kernel itself waits (pdl_wait) before touching global memory
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(pl.threads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CUNN_CUDA(cudaLaunchKernelExC(&cfg, (const void *)kern, args));
    (void)name;
    return 0;
}

static void fill_params(FastParams &fp, const Plan &pl, int N, int C, int H, int W, int oH, int oW)
{
    fp.N = N; fp.C = C; fp.H = H; fp.W = W; fp.oH = oH; fp.oW = oW;
    fp.P = pl.P; fp.bands = pl.bands; fp.R = pl.R; fp.RS = pl.RS; fp.strips = pl.strips; fp.CG = pl.CG;
    fp.items = pl.items; fp.maxseg = pl.maxseg; fp.stages = pl.stages;
    fp.stage_floats = pl.stage_floats; fp.stage2_floats = pl.stage2_floats; fp.out_floats = pl.out_floats;
    fp.status = device_status_ptr();
    fp.flip = 0;
    fp.scale = 1.f;
}

// Workspace of the parameter-gradient kernel: a control region of fixed size holding one ticket counter
// per channel group, followed by the partial sums.  The control region never moves or resizes, so the
// "zero on entry, zero on exit" rule holds across calls with different shapes on one buffer.
static size_t wgrad_counter_bytes(int, const Plan &) { return (size_t)kMaxGroups * 4; }
static size_t wgrad_workspace_bytes(int C, const Plan &pl)
{
    return wgrad_counter_bytes(C, pl) + (size_t)pl.grid * pl.maxseg * pl.P * 10 * sizeof(float);
}

static bool fast_shape(int M, int kH, int kW, int dH, int dW, int padH, int padW)
{
    return !g_tuning.force_generic && M == 1 && kH == 3 && kW == 3 && dH == dW && (dH == 1 || dH == 2) && padH == 1 &&
           padW == 1;
}

static int check_common(int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                        int *oH, int *oW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && H > 0 && W > 0 && M > 0 && padH >= 0 && padW >= 0,
                   "bad depthwise sizes N=%d C=%d H=%d W=%d M=%d pad=%d,%d", N, C, H, W, M, padH, padW);
    *oH = (H + 2 * padH - kH) / dH + 1;
    *oW = (W + 2 * padW - kW) / dW + 1;
    CUNN_CHECK_ARG(H + 2 * padH >= kH && W + 2 * padW >= kW && *oH >= 1 && *oW >= 1,
                   "Given input size: (%d x %d x %d). Calculated output size: (%d x %d x %d). Output size is too small",
                   C, H, W, C * M, *oH, *oW);
    CUNN_CHECK_ARG((long long)N * C * M * (long long)(*oH) * (*oW) < (1LL << 31) && (long long)N * C * (long long)H * W < (1LL << 31),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

static int grid_for(long long total)
{
    const long long want = ceil_div_ll(total, 256);
    const long long cap = (long long)sm_count() * 16;
    return (int)std::max(1LL, std::min(want, cap));
}

}  // namespace dw
}  // namespace cunn

using namespace cunn;
using namespace cunn::dw;

// Developer hooks for tile-plan sweeps; not part of the library's interface and absent from the
// default build (compile with -DCUNN_B200_DEV_HOOKS).
#ifdef CUNN_B200_DEV_HOOKS
extern "C" CUNN_API void cunn_b200_dwconv_tuning(const int *values, int count)
{
    int v[10] = {0, 0, 0, 0, 0, 0, 0, 0, -1, -1};
    for (int i = 0; i < count && i < 10; ++i) v[i] = values[i];
    g_tuning.P = v[0];
    g_tuning.R = v[1];
    g_tuning.RS = v[2];
    g_tuning.stages = v[3];
    g_tuning.ctas_per_sm = v[4];
    g_tuning.force_generic = v[5];
    g_tuning.budget_kb = v[6];
    g_tuning.vec = v[7];
    g_tuning.stage_out = v[8];
    g_tuning.direct = v[9];
}
#endif  // CUNN_B200_DEV_HOOKS

extern "C" int cunn_b200_dwconv_forward(const float *x, const float *weight, const float *bias, float *y, int N, int C,
                                        int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                        cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check_common(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    if (fast_shape(M, kH, kW, dH, dW, padH, padW) && aligned16(x) && aligned16(y)) {
        Plan pl = make_plan(MODE_FWD, N, C, H, W, oH, oW, dH);
        if (pl.ok && finalize_plan(pl) == 0) {
            FastParams fp{};
            fill_params(fp, pl, N, C, H, W, oH, oW);
            fp.in = x; fp.w = weight; fp.bias = bias; fp.out = y;
            return launch_fast(fp, pl, stream, "dwconv forward (3x3)");
        }
    }
    const long long total = (long long)N * C * M * oH * oW;
    fwd_generic_kernel<<<grid_for(total), 256, 0, stream>>>(x, weight, bias, y, C, H, W, M, kH, kW, dH, dW, padH, padW,
                                                           oH, oW, total);
    CUNN_LAUNCH_CHECK("dwconv forward (generic)");
    return 0;
}

extern "C" int cunn_b200_dwconv_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H, int W,
                                           int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                           cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check_common(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    if (fast_shape(M, kH, kW, dH, dW, padH, padW) && aligned16(gy) && aligned16(gx)) {
        if (dH == 1) {
            // stride 1: the input gradient is the forward stencil with the kernel rotated by 180 degrees
            Plan pl = make_plan(MODE_FWD, N, C, oH, oW, H, W, 1);
            if (pl.ok && finalize_plan(pl) == 0) {
                FastParams fp{};
                fill_params(fp, pl, N, C, oH, oW, H, W);
                fp.in = gy; fp.w = weight; fp.bias = nullptr; fp.out = gx; fp.flip = 1;
                return launch_fast(fp, pl, stream, "dwconv grad input (3x3 s1)");
            }
        } else {
            Plan pl = make_plan(MODE_DGRAD_S2, N, C, H, W, oH, oW, 2);
            if (pl.ok && finalize_plan(pl) == 0) {
                FastParams fp{};
                fill_params(fp, pl, N, C, H, W, oH, oW);
                fp.in = gy; fp.w = weight; fp.out = gx;
                return launch_fast(fp, pl, stream, "dwconv grad input (3x3 s2)");
            }
        }
    }
    const long long total = (long long)N * C * H * W;
    dgrad_generic_kernel<<<grid_for(total), 256, 0, stream>>>(gy, weight, gx, C, H, W, M, kH, kW, dH, dW, padH, padW, oH,
                                                             oW, total);
    CUNN_LAUNCH_CHECK("dwconv grad input (generic)");
    return 0;
}

extern "C" CUNN_API void cunn_b200_set_deterministic(int on) { g_deterministic = on ? 1 : 0; }
extern "C" CUNN_API int cunn_b200_get_deterministic(void) { return g_deterministic; }

extern "C" size_t cunn_b200_dwconv_acc_grad_workspace(int N, int C, int H, int W, int M, int kH, int kW, int dH, int dW,
                                                      int padH, int padW)
{
    int oH, oW;
    if (check_common(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 0;
    if (!fast_shape(M, kH, kW, dH, dW, padH, padW) || N == 0) return 0;
    Plan pl = make_plan(MODE_WGRAD, N, C, H, W, oH, oW, dH);
    if (!pl.ok || finalize_plan(pl)) return 0;
    return wgrad_workspace_bytes(C, pl);
}

extern "C" int cunn_b200_dwconv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias, int N,
                                         int C, int H, int W, int M, int kH, int kW, int dH, int dW, int padH, int padW,
                                         float scale, void *workspace, size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check_common(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    if (fast_shape(M, kH, kW, dH, dW, padH, padW) && aligned16(x) && aligned16(gy)) {
        Plan pl = make_plan(MODE_WGRAD, N, C, H, W, oH, oW, dH);
        if (pl.ok && finalize_plan(pl) == 0) {
            FastParams fp{};
            fill_params(fp, pl, N, C, H, W, oH, oW);
            fp.in = x; fp.in2 = gy; fp.w = nullptr; fp.out = nullptr;
            fp.gw = grad_weight; fp.gb = grad_bias; fp.scale = scale;
            if (!g_deterministic) {
                fp.atomic_flush = 1;   // no scratch needed: the workspace argument is ignored
                return launch_fast(fp, pl, stream, "dwconv acc grad (3x3)");
            }
            const size_t need = wgrad_workspace_bytes(C, pl);
            CUNN_CHECK_ARG(workspace && workspace_bytes >= need && aligned16(workspace),
                           "dwconv acc_grad needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                           workspace ? workspace_bytes : (size_t)0);
            // The ticket counters return to zero when every CTA hands in its partials; a CTA that gave up on a
            // bounded wait does not, so they are cleared here rather than trusted to be zero on entry.
            CUNN_CUDA(cudaMemsetAsync(workspace, 0, (size_t)(C / pl.P) * sizeof(unsigned int), stream));
            fp.counters = (unsigned int *)workspace;
            fp.partials = (float *)((char *)workspace + wgrad_counter_bytes(C, pl));
            return launch_fast(fp, pl, stream, "dwconv acc grad (3x3)");
        }
    }
    const int blocks = M * C * (kH * kW + 1);
    wgrad_generic_kernel<<<blocks, 256, 0, stream>>>(x, gy, grad_weight, grad_bias, N, C, H, W, M, kH, kW, dH, dW, padH,
                                                    padW, oH, oW, scale);
    CUNN_LAUNCH_CHECK("dwconv acc grad (generic)");
    return 0;
}

#ifdef CUNN_B200_DEV_HOOKS
// Writes the tile plan the 3x3 fast path would use into buf (for tests, tuning and documentation).
// mode: 0 forward, 1 stride-2 input gradient, 2 parameter gradient.
extern "C" CUNN_API int cunn_b200_dwconv_describe_plan(int mode, int N, int C, int H, int W, int stride, char *buf, int buflen)
{
    const int oH = (H + 2 - 3) / stride + 1, oW = (W + 2 - 3) / stride + 1;
    Plan pl = make_plan(mode, N, C, H, W, oH, oW, stride);
    if (pl.ok) finalize_plan(pl);
    snprintf(buf, buflen,
             "ok=%d S=%d VEC=%d staged_out=%d direct=%d P=%d bands=%d R=%d RS=%d strips=%d CG=%d items=%d threads=%d stages=%d "
             "maxseg=%d grid=%d stage_bytes=%d+%d out_bytes=2x%d smem=%zu",
             (int)pl.ok, pl.S, pl.VEC, (int)pl.stage_out, (int)pl.direct, pl.P, pl.bands, pl.R, pl.RS, pl.strips, pl.CG, pl.items,
             pl.threads, pl.stages, pl.maxseg, pl.ok ? pl.grid : 0, pl.stage_floats * 4, pl.stage2_floats * 4,
             pl.out_floats * 4, pl.smem);
    return pl.ok ? 0 : 1;
}
#endif  // CUNN_B200_DEV_HOOKS

// ---------------------------------------------------------------------------
// Parameter gradient without caller-provided scratch
// ---------------------------------------------------------------------------
//
// Some hosts cannot hand this library a workspace: a program that has given all device memory to an
// arena of its own has nothing left to cudaMalloc from, and a binding that only passes tensors through
// (the LuaJIT FFI signature of accGradParameters has no workspace argument) has no allocator to ask.
// For them the scratch of the 3x3 parameter-gradient kernel lives in a fixed array inside this module.
// Every GPU that loads the library holds these bytes until the process exits.
static const size_t kStaticScratchBytes = (size_t)4 << 20;  // 4 MiB: 64 KiB of ticket counters + partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// Device address of g_static_scratch per device.  In host code the array's name only stands for the
// symbol; the address a kernel can use comes from cudaGetSymbolAddress with that device current.
unsigned char *g_static_scratch_ptr[64];
}

extern "C" CUNN_API size_t cunn_b200_dwconv_acc_grad_static_capacity(void) { return kStaticScratchBytes; }

extern "C" CUNN_API int cunn_b200_dwconv_acc_grad_static(const float *x, const float *gy, float *grad_weight,
                                                         float *grad_bias, int N, int C, int H, int W, int M, int kH,
                                                         int kW, int dH, int dW, int padH, int padW, float scale,
                                                         cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check_common(N, C, H, W, M, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    if (fast_shape(M, kH, kW, dH, dW, padH, padW) && aligned16(x) && aligned16(gy)) {
        Plan pl = make_plan(MODE_WGRAD, N, C, H, W, oH, oW, dH);
        if (pl.ok && finalize_plan(pl) == 0) {
            const size_t need = wgrad_workspace_bytes(C, pl);
            CUNN_CHECK_ARG(need <= kStaticScratchBytes,
                           "dwconv acc_grad (static scratch): this shape needs %zu bytes of scratch, the built-in array "
                           "holds %zu; use cunn_b200_dwconv_acc_grad with a caller-provided workspace",
                           need, kStaticScratchBytes);
            int dev = 0;
            CUNN_CUDA(cudaGetDevice(&dev));
            CUNN_CHECK_ARG(dev >= 0 && dev < 64, "device index %d out of range", dev);
            if (!g_static_scratch_ptr[dev]) {
                // one-time set-up for this device (it is the current one)
                void *ptr = nullptr;
                CUNN_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
                g_static_scratch_ptr[dev] = (unsigned char *)ptr;
            }
            unsigned char *scratch = g_static_scratch_ptr[dev];
            // The array keeps whatever the previous call left.  The ticket counters must start at zero;
            // the partial sums are fully written before they are read.
            CUNN_CUDA(cudaMemsetAsync(scratch, 0, (size_t)(C / pl.P) * sizeof(unsigned int), stream));
            FastParams fp{};
            fill_params(fp, pl, N, C, H, W, oH, oW);
            fp.in = x; fp.in2 = gy; fp.w = nullptr; fp.out = nullptr;
            fp.gw = grad_weight; fp.gb = grad_bias; fp.scale = scale;
            fp.counters = (unsigned int *)scratch;
            fp.partials = (float *)(scratch + wgrad_counter_bytes(C, pl));
            return launch_fast(fp, pl, stream, "dwconv acc grad (3x3, static scratch)");
        }
    }
    // shapes outside the 3x3 fast path use the generic kernel, which needs no scratch at all
    const int blocks = M * C * (kH * kW + 1);
    wgrad_generic_kernel<<<blocks, 256, 0, stream>>>(x, gy, grad_weight, grad_bias, N, C, H, W, M, kH, kW, dH, dW, padH,
                                                    padW, oH, oW, scale);
    CUNN_LAUNCH_CHECK("dwconv acc grad (generic)");
    return 0;
}
