// Batch normalisation over [N, C, S] (S = H*W) for sm_100a: forward (training and inference) and backward.
//
// The reference runs one 512-thread CTA per channel, which leaves most of a 148-SM GPU idle when C is
// small and reads the input three times.  Here every pass is spread over (channel x chunk) CTAs:
//   * statistics: each CTA reduces a contiguous run of planes of one channel with 16-byte loads.  Sums
//     are taken of (x - K) and (x - K)^2 with K the mean of the chunk's first elements, which keeps fp32
//     accumulation accurate even when |mean| >> std; chunks are merged in fp64 (Chan's formula) by a
//     small second kernel that also writes save_mean / save_std and updates the running statistics;
//   * normalisation / gradient: one grid-stride pass with 16-byte loads and stores.
// Formulas (lib/THCUNN/BatchNormalization.cu:141-283): save_std holds 1/sqrt(biased var + eps) (0 when
// var == 0 and eps == 0), running_var is updated with the unbiased variance n/(n-1).
#include "common.cuh"

#include <algorithm>

namespace cunn {
namespace bn {

struct ChunkStat {
    float k;      // shift
    float s1;     // sum (x - k)
    float s2;     // sum (x - k)^2
    float n;      // element count
};

__device__ __forceinline__ float block_sum(float v, float *sh)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = 0.f;
    if (warp == 0) {
        r = (lane < (int)(blockDim.x >> 5)) ? sh[lane] : 0.f;
        r = warp_sum(r);
        if (lane == 0) sh[0] = r;
    }
    __syncthreads();
    return sh[0];
}

// Planes of channel c: image n at x + (n*C + c)*S.  Chunk j of `chunks` covers images [n0, n1).
__device__ __forceinline__ void chunk_range(int N, int chunks, int j, int *n0, int *n1)
{
    const int per = N / chunks, extra = N % chunks;
    *n0 = j * per + min(j, extra);
    *n1 = *n0 + per + (j < extra ? 1 : 0);
}

// Merges the chunk statistics of channel c in fp64 (Chan's formula), publishes mean / inverse std and updates
// the running statistics.
__device__ __forceinline__ void finish_stats_channel(const ChunkStat *part, int c, int chunks, float *running_mean,
                                                     float *running_var, float *save_mean, float *save_std,
                                                     double momentum, double eps)
{
    double n = 0.0, mean = 0.0, m2 = 0.0;
    for (int j = 0; j < chunks; ++j) {
        const float4 raw = __ldcg(reinterpret_cast<const float4 *>(part + c * chunks + j));   // written by other CTAs
        const ChunkStat p{raw.x, raw.y, raw.z, raw.w};
        if (p.n <= 0.f) continue;
        const double nb = p.n;
        const double mb = (double)p.k + (double)p.s1 / nb;
        const double m2b = (double)p.s2 - (double)p.s1 * (double)p.s1 / nb;
        const double delta = mb - mean, nt = n + nb;
        mean += delta * nb / nt;
        m2 += m2b + delta * delta * n * nb / nt;
        n = nt;
    }
    if (m2 < 0.0) m2 = 0.0;
    // The reference computes in float for float tensors; follow its formulas on the float-rounded mean.
    const float meanf = (float)mean;
    const float varN = (float)m2;
    float invstd = 0.f;
    if (varN != 0.f || (float)eps != 0.f) invstd = 1.f / sqrtf((float)(m2 / n) + (float)eps);
    const float unbiased = (float)(m2 / (n - 1.0));
    save_mean[c] = meanf;
    save_std[c] = invstd;
    running_mean[c] = (float)((1.0 - momentum) * (double)running_mean[c] + momentum * (double)meanf);
    running_var[c] = (float)((1.0 - momentum) * (double)running_var[c] + momentum * (double)unbiased);
}

// The CTA that hands in the last partial of a channel finishes the channel: ticket counter per channel, zero
// before the launch and zero again after it.  Returns true in every thread of that CTA.
__device__ __forceinline__ bool last_cta_of_channel(unsigned int *counters, int c, int chunks, int *flag)
{
    if (threadIdx.x == 0) {
        __threadfence();                                  // this CTA's partial is visible before its ticket
        *flag = atomicAdd(counters + c, 1u) == (unsigned int)(chunks - 1);
    }
    __syncthreads();
    const bool last = *flag != 0;
    if (last) __threadfence();                            // the other CTAs' partials are visible after their tickets
    return last;
}

// Chan's merge of two (count, mean, M2) triples; either side may be empty.
__device__ __forceinline__ void chan_merge(double &n, double &mean, double &m2, double nb, double mb, double m2b)
{
    if (nb <= 0.0) return;
    const double nt = n + nb, delta = mb - mean;
    mean += delta * nb / nt;
    m2 += m2b + delta * delta * n * nb / nt;
    n = nt;
}

// The same merge as finish_stats_channel, by one warp: every lane folds its share of the chunks, then the lanes are
// merged pairwise (fp64 divisions are slow; 37 chunks in one thread took 10 us).
__device__ __forceinline__ void finish_stats_channel_warp(const ChunkStat *part, int c, int chunks, float *running_mean,
                                                          float *running_var, float *save_mean, float *save_std,
                                                          double momentum, double eps)
{
    const int lane = threadIdx.x & 31;
    double n = 0.0, mean = 0.0, m2 = 0.0;
    for (int j = lane; j < chunks; j += 32) {
        const float4 raw = __ldcg(reinterpret_cast<const float4 *>(part + c * chunks + j));
        if (raw.w <= 0.f) continue;
        const double nb = raw.w;
        chan_merge(n, mean, m2, nb, (double)raw.x + (double)raw.y / nb, (double)raw.z - (double)raw.y * (double)raw.y / nb);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double nb = __shfl_xor_sync(0xffffffffu, n, o), mb = __shfl_xor_sync(0xffffffffu, mean, o),
                     m2b = __shfl_xor_sync(0xffffffffu, m2, o);
        // both partners must end up with the same triple: merge in a fixed order (lower lane first)
        if (lane & o) {
            double n2 = nb, mean2 = mb, m22 = m2b;
            chan_merge(n2, mean2, m22, n, mean, m2);
            n = n2; mean = mean2; m2 = m22;
        } else {
            chan_merge(n, mean, m2, nb, mb, m2b);
        }
    }
    if (lane != 0) return;
    if (m2 < 0.0) m2 = 0.0;
    const float meanf = (float)mean;
    const float varN = (float)m2;
    float invstd = 0.f;
    if (varN != 0.f || (float)eps != 0.f) invstd = 1.f / sqrtf((float)(m2 / n) + (float)eps);
    const float unbiased = (float)(m2 / (n - 1.0));
    save_mean[c] = meanf;
    save_std[c] = invstd;
    running_mean[c] = (float)((1.0 - momentum) * (double)running_mean[c] + momentum * (double)meanf);
    running_var[c] = (float)((1.0 - momentum) * (double)running_var[c] + momentum * (double)unbiased);
}

// Walks the planes [n0, n1) of channel c as one flat sequence of items of type T (float4 or float), blockDim.x items
// apart per thread, and fetches them U at a time so that every thread keeps U loads in flight.  `mask` has bit u set
// for every slot that was filled; items arrive in walk order, so sums taken slot by slot do not depend on U.
template <typename T, int U>
struct PlaneWalk {
    const float *x;
    int C, S, c, n1, L, qstep, rstep, n, i;
    __device__ __forceinline__ void init(const float *x_, int C_, int S_, int c_, int n0, int n1_)
    {
        x = x_; C = C_; S = S_; c = c_; n1 = n1_;
        L = S / (int)(sizeof(T) / sizeof(float));
        qstep = (int)blockDim.x / L; rstep = (int)blockDim.x % L;
        n = n0 + (int)threadIdx.x / L; i = (int)threadIdx.x % L;
    }
    // the same walk over a second tensor of the same shape
    template <bool TWO>
    __device__ __forceinline__ unsigned load(T (&v)[U], T (&w)[U], const float *y)
    {
        unsigned mask = 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (n < n1) {
                const size_t off = ((size_t)n * C + c) * S;
                v[u] = __ldg(reinterpret_cast<const T *>(x + off) + i);
                if (TWO) w[u] = __ldg(reinterpret_cast<const T *>(y + off) + i);
                mask |= 1u << u;
                n += qstep; i += rstep;
                if (i >= L) { i -= L; ++n; }
            }
        }
        return mask;
    }
};

// Shifted sums of one chunk: s1 = sum (x - k), s2 = sum (x - k)^2.  The shift k is the mean of the chunk's first (up to)
// 32 elements: close to the channel mean, so the sums of (x - k) stay small and keep their fp32 accuracy even when a
// single element is an outlier.  The first batch of loads is issued before the probe for k, so its latency is hidden.
template <typename T, int U>
__device__ __forceinline__ void chunk_sums(const float *x, int C, int S, int c, int n0, int n1, float *k_s, float *s1_out,
                                           float *s2_out, float *k_out)
{
    PlaneWalk<T, U> w;
    w.init(x, C, S, c, n0, n1);
    T a[U], b[U];
    unsigned ma = w.template load<false>(a, a, nullptr), mb = 0;
    if (threadIdx.x < 32) {
        const long long cnt = (long long)(n1 - n0) * S;
        const int m = cnt < 32 ? (int)cnt : 32;
        float v = 0.f;
        if ((int)threadIdx.x < m) {
            const int e = (int)threadIdx.x, pn = n0 + e / S;
            v = __ldg(x + ((size_t)pn * C + c) * S + (e - (e / S) * S));
        }
        v = warp_sum(v);
        if (threadIdx.x == 0) *k_s = v / (float)m;
    }
    __syncthreads();
    const float k = *k_s;
    float s1 = 0.f, s2 = 0.f;
    auto acc1 = [&](float v) { const float t = v - k; s1 += t; s2 = fmaf(t, t, s2); };
    auto acc = [&](const T (&v)[U], unsigned m) {
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (m >> u & 1u) {
                if constexpr (sizeof(T) == 16) {
                    const float4 q = *reinterpret_cast<const float4 *>(&v[u]);
                    const float e = q.x - k, f = q.y - k, g = q.z - k, h = q.w - k;
                    s1 += (e + f) + (g + h);
                    s2 = fmaf(e, e, s2); s2 = fmaf(f, f, s2); s2 = fmaf(g, g, s2); s2 = fmaf(h, h, s2);
                } else {
                    acc1(*reinterpret_cast<const float *>(&v[u]));
                }
            }
    };
    for (;;) {
        if (!ma) break;
        mb = w.template load<false>(b, b, nullptr);
        acc(a, ma);
        if (!mb) break;
        ma = w.template load<false>(a, a, nullptr);
        acc(b, mb);
    }
    *s1_out = s1; *s2_out = s2; *k_out = k;
}

// grid = C * chunks.  One partial statistic per CTA; with `counters` the last CTA of a channel also merges the
// partials (no second launch).
__global__ void __launch_bounds__(256)
stats_kernel(const float *__restrict__ x, ChunkStat *__restrict__ part, int N, int C, int S, int chunks,
             unsigned int *__restrict__ counters, float *__restrict__ running_mean, float *__restrict__ running_var,
             float *__restrict__ save_mean, float *__restrict__ save_std, double momentum, double eps)
{
    __shared__ float sh[8];
    __shared__ int flag;
    const int c = blockIdx.x / chunks, j = blockIdx.x % chunks;
    int n0, n1;
    chunk_range(N, chunks, j, &n0, &n1);
    __shared__ float k_s;
    float k = 0.f, s1 = 0.f, s2 = 0.f;
    if (n0 < n1) {
        const bool vec = (S % 4 == 0) && (((uintptr_t)x & 15) == 0);
        if (vec) chunk_sums<float4, 4>(x, C, S, c, n0, n1, &k_s, &s1, &s2, &k);
        else chunk_sums<float, 8>(x, C, S, c, n0, n1, &k_s, &s1, &s2, &k);
        s1 = block_sum(s1, sh);
        s2 = block_sum(s2, sh);
    }
    if (threadIdx.x == 0) part[blockIdx.x] = ChunkStat{k, s1, s2, n0 < n1 ? (float)((long long)(n1 - n0) * S) : 0.f};
    if (!counters) return;
    if (last_cta_of_channel(counters, c, chunks, &flag)) {
        if (threadIdx.x < 32) finish_stats_channel_warp(part, c, chunks, running_mean, running_var, save_mean, save_std, momentum, eps);
        if (threadIdx.x == 0) counters[c] = 0u;
    }
}

// One thread per channel: the merge as a separate launch (more channels than ticket counters).
__global__ void __launch_bounds__(128)
stats_finish_kernel(const ChunkStat *__restrict__ part, int C, int chunks, float *__restrict__ running_mean,
                    float *__restrict__ running_var, float *__restrict__ save_mean, float *__restrict__ save_std,
                    double momentum, double eps)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) finish_stats_channel(part, c, chunks, running_mean, running_var, save_mean, save_std, momentum, eps);
}

// gamma * (x - mean) * invstd + beta with every rounding pinned (no fused multiply-add), so that the backward
// kernels can recompute the sign of the forward value bit for bit.
__device__ __forceinline__ float bn_value(float v, float mean, float invstd, float g, float b)
{
    return __fadd_rn(__fmul_rn(__fmul_rn(g, __fsub_rn(v, mean)), invstd), b);
}

// y = gamma * (x - mean) * invstd + beta, per plane.  Training reads mean / invstd from save_*, inference
// derives them from the running statistics.
// GROUP threads (a warp for small planes, the whole CTA for large ones) share a plane.
template <bool RELU, int GROUP>
__global__ void __launch_bounds__(256)
apply_kernel(const float *__restrict__ x, float *__restrict__ y, const float *__restrict__ weight,
             const float *__restrict__ bias, const float *__restrict__ mean_v, const float *__restrict__ std_or_var,
             int train, float eps, int C, int S, long long planes)
{
    auto act = [](float v) { return RELU ? (v > 0.f ? v : 0.f) : v; };
    const bool vec = (S % 4 == 0) && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
    constexpr int PER_CTA = 256 / GROUP;
    const int sub = (int)threadIdx.x / GROUP, t = (int)threadIdx.x % GROUP;
    for (long long pl = (long long)blockIdx.x * PER_CTA + sub; pl < planes; pl += (long long)gridDim.x * PER_CTA) {
        const int c = (int)(pl % C);
        const float mean = __ldg(mean_v + c);
        const float invstd = train ? __ldg(std_or_var + c) : 1.f / sqrtf(__ldg(std_or_var + c) + eps);
        const float g = weight ? __ldg(weight + c) : 1.f;
        const float b = bias ? __ldg(bias + c) : 0.f;
        const float *xp = x + pl * S;
        float *yp = y + pl * S;
        if (vec) {
            const float4 *x4 = reinterpret_cast<const float4 *>(xp);
            float4 *y4 = reinterpret_cast<float4 *>(yp);
#pragma unroll 4
            for (int i = t; i < S / 4; i += GROUP) {
                const float4 v = __ldg(x4 + i);
                float4 o;
                o.x = act(bn_value(v.x, mean, invstd, g, b));
                o.y = act(bn_value(v.y, mean, invstd, g, b));
                o.z = act(bn_value(v.z, mean, invstd, g, b));
                o.w = act(bn_value(v.w, mean, invstd, g, b));
                y4[i] = o;
            }
        } else {
            for (int i = t; i < S; i += GROUP) yp[i] = act(bn_value(__ldg(xp + i), mean, invstd, g, b));
        }
    }
}

// Planes whose size is not a multiple of 4 (7x7 = 49 elements): the tensor is walked as one flat array of 16-byte
// items, four per thread and iteration; an item may straddle planes, so the channel is tracked element by element.
template <bool RELU>
__global__ void __launch_bounds__(256)
apply_flat_kernel(const float *__restrict__ x, float *__restrict__ y, const float *__restrict__ weight,
                  const float *__restrict__ bias, const float *__restrict__ mean_v, const float *__restrict__ std_or_var,
                  int train, float eps, unsigned C, unsigned S, unsigned total)
{
    auto act = [](float v) { return RELU ? (v > 0.f ? v : 0.f) : v; };
    float mean = 0.f, invstd = 0.f, g = 1.f, b = 0.f;
    auto fetch = [&](unsigned c) {
        mean = __ldg(mean_v + c);
        invstd = train ? __ldg(std_or_var + c) : 1.f / sqrtf(__ldg(std_or_var + c) + eps);
        g = weight ? __ldg(weight + c) : 1.f;
        b = bias ? __ldg(bias + c) : 0.f;
    };
    auto item = [&](unsigned q, const float4 v) {
        const unsigned e = q * 4u, pl = e / S;
        unsigned r = e - pl * S, c = pl % C;
        fetch(c);
        const float in[4] = {v.x, v.y, v.z, v.w};
        float out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[j] = act(bn_value(in[j], mean, invstd, g, b));
            if (j < 3 && ++r == S) {
                r = 0;
                if (++c == C) c = 0;
                fetch(c);
            }
        }
        reinterpret_cast<float4 *>(y)[q] = make_float4(out[0], out[1], out[2], out[3]);
    };
    const unsigned items = total / 4u, stride = gridDim.x * blockDim.x, tid = blockIdx.x * blockDim.x + threadIdx.x;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    constexpr unsigned U = 4;
    for (unsigned q = tid; q < items; q += U * stride) {
        float4 v[U];
#pragma unroll
        for (unsigned u = 0; u < U; ++u)
            if (q + u * stride < items) v[u] = __ldg(x4 + q + u * stride);
#pragma unroll
        for (unsigned u = 0; u < U; ++u)
            if (q + u * stride < items) item(q + u * stride, v[u]);
    }
    if (tid < total - items * 4u) {
        const unsigned e = items * 4u + tid;
        fetch((e / S) % C);
        y[e] = act(bn_value(__ldg(x + e), mean, invstd, g, b));
    }
}

// Per-channel coefficients of the input gradient:
//   gx = (gy - (x - mean) * proj - gmean) * gscale      (training)
//   gx = gy * gscale                                     (inference)
struct GradCoef {
    float mean, proj, gmean, gscale;
    float invstd, gamma, beta, pad;     // forward coefficients, for the sign of the fused ReLU's input
};

// Backward, pass 2 for channel c: totals the chunk sums in fp64, accumulates gradWeight / gradBias and publishes
// the coefficients of the input gradient.
__device__ __forceinline__ void finish_grad_channel(const float2 *part, int c, int chunks, long long count, const float *weight,
                                                    const float *bias, const float *mean_v, const float *std_or_var,
                                                    int train, double eps, double scale, float *grad_weight,
                                                    float *grad_bias, GradCoef *coef)
{
    double s = 0.0, d = 0.0;
    for (int j = 0; j < chunks; ++j) {
        const float2 p = __ldcg(part + c * chunks + j);   // written by other CTAs
        s += (double)p.x;
        d += (double)p.y;
    }
    const float mean = mean_v[c];
    const float stdv = train ? std_or_var[c] : (float)(1.0 / sqrt((double)std_or_var[c] + eps));
    const float w = weight ? weight[c] : 1.f;
    const double norm = 1.0 / (double)count;
    GradCoef k;
    k.mean = mean;
    k.gmean = (float)(s * norm);
    k.proj = (float)(d * norm * (double)stdv * (double)stdv);
    k.gscale = stdv * w;
    k.invstd = train ? std_or_var[c] : 1.f / sqrtf(std_or_var[c] + (float)eps);   // as the forward kernel computes it
    k.gamma = w;
    k.beta = bias ? bias[c] : 0.f;
    k.pad = 0.f;
    coef[c] = k;
    if (grad_weight) grad_weight[c] = (float)((double)grad_weight[c] + scale * d * (double)stdv);
    if (grad_bias) grad_bias[c] = (float)((double)grad_bias[c] + scale * s);
}

__global__ void __launch_bounds__(128)
grad_finish_kernel(const float2 *__restrict__ part, int C, int chunks, long long count,
                   const float *__restrict__ weight, const float *__restrict__ bias, const float *__restrict__ mean_v,
                   const float *__restrict__ std_or_var, int train, double eps, double scale,
                   float *__restrict__ grad_weight, float *__restrict__ grad_bias, GradCoef *__restrict__ coef)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) finish_grad_channel(part, c, chunks, count, weight, bias, mean_v, std_or_var, train, eps, scale, grad_weight, grad_bias, coef);
}

// Backward, pass 1: per (channel, chunk) sums of gy and gy * (x - mean).
template <bool RELU>
__global__ void __launch_bounds__(256)
grad_stats_kernel(const float *__restrict__ x, const float *__restrict__ gy, float2 *__restrict__ part,
                  const float *__restrict__ mean_v, const float *__restrict__ std_or_var, const float *__restrict__ weight,
                  const float *__restrict__ bias, int train, float eps, int N, int C, int S, int chunks,
                  unsigned int *__restrict__ counters, double eps_d, double scale, float *__restrict__ grad_weight,
                  float *__restrict__ grad_bias, GradCoef *__restrict__ coef)
{
    __shared__ float sh[8];
    __shared__ int flag;
    const int c = blockIdx.x / chunks, j = blockIdx.x % chunks;
    int n0, n1;
    chunk_range(N, chunks, j, &n0, &n1);
    const float mean = __ldg(mean_v + c);
    // fused ReLU: the gradient passes only where the forward value was positive; its sign is recomputed from x
    float invstd = 0.f, gam = 1.f, bet = 0.f;
    if (RELU) {
        invstd = train ? __ldg(std_or_var + c) : 1.f / sqrtf(__ldg(std_or_var + c) + eps);
        gam = weight ? __ldg(weight + c) : 1.f;
        bet = bias ? __ldg(bias + c) : 0.f;
    }
    float s = 0.f, d = 0.f;
    const bool vec = (S % 4 == 0) && ((((uintptr_t)x | (uintptr_t)gy) & 15) == 0);
    auto one = [&](float v, float g) {
        if (RELU) g = bn_value(v, mean, invstd, gam, bet) > 0.f ? g : 0.f;
        return g;
    };
    if (vec) {
        constexpr int U = 2;
        PlaneWalk<float4, U> w;
        w.init(x, C, S, c, n0, n1);
        float4 xa[U], ga[U], xb[U], gb[U];
        auto acc = [&](const float4 (&xv)[U], const float4 (&gv)[U], unsigned m) {
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (m >> u & 1u) {
                    const float4 v = xv[u];
                    float4 g = gv[u];
                    g.x = one(v.x, g.x); g.y = one(v.y, g.y); g.z = one(v.z, g.z); g.w = one(v.w, g.w);
                    s += (g.x + g.y) + (g.z + g.w);
                    d = fmaf(g.x, v.x - mean, d); d = fmaf(g.y, v.y - mean, d);
                    d = fmaf(g.z, v.z - mean, d); d = fmaf(g.w, v.w - mean, d);
                }
        };
        unsigned ma = w.load<true>(xa, ga, gy), mb = 0;
        for (;;) {
            if (!ma) break;
            mb = w.load<true>(xb, gb, gy);
            acc(xa, ga, ma);
            if (!mb) break;
            ma = w.load<true>(xa, ga, gy);
            acc(xb, gb, mb);
        }
    } else {
        constexpr int U = 4;
        PlaneWalk<float, U> w;
        w.init(x, C, S, c, n0, n1);
        float xa[U], ga[U], xb[U], gb[U];
        auto acc = [&](const float (&xv)[U], const float (&gv)[U], unsigned m) {
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (m >> u & 1u) {
                    const float g = one(xv[u], gv[u]);
                    s += g;
                    d = fmaf(g, xv[u] - mean, d);
                }
        };
        unsigned ma = w.load<true>(xa, ga, gy), mb = 0;
        for (;;) {
            if (!ma) break;
            mb = w.load<true>(xb, gb, gy);
            acc(xa, ga, ma);
            if (!mb) break;
            ma = w.load<true>(xa, ga, gy);
            acc(xb, gb, mb);
        }
    }
    s = block_sum(s, sh);
    d = block_sum(d, sh);
    if (threadIdx.x == 0) part[blockIdx.x] = make_float2(s, d);
    if (!counters) return;
    if (last_cta_of_channel(counters, c, chunks, &flag)) {
        if (threadIdx.x == 0) {
            finish_grad_channel(part, c, chunks, (long long)N * S, weight, bias, mean_v, std_or_var, train, eps_d, scale, grad_weight,
                                grad_bias, coef);
            counters[c] = 0u;
        }
    }
}

// Backward, pass 3: the input gradient.
template <bool RELU, int GROUP>
__global__ void __launch_bounds__(256)
grad_apply_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ gx,
                  const GradCoef *__restrict__ coef, int train, int C, int S, long long planes)
{
    const bool vec = (S % 4 == 0) && ((((uintptr_t)x | (uintptr_t)gy | (uintptr_t)gx) & 15) == 0);
    constexpr int PER_CTA = 256 / GROUP;
    const int sub = (int)threadIdx.x / GROUP, t = (int)threadIdx.x % GROUP;
    for (long long pl = (long long)blockIdx.x * PER_CTA + sub; pl < planes; pl += (long long)gridDim.x * PER_CTA) {
        const GradCoef k = coef[pl % C];
        const float *xp = x + pl * S;
        const float *gp = gy + pl * S;
        float *op = gx + pl * S;
        if (vec) {
            const float4 *x4 = reinterpret_cast<const float4 *>(xp);
            const float4 *g4 = reinterpret_cast<const float4 *>(gp);
            float4 *o4 = reinterpret_cast<float4 *>(op);
#pragma unroll 4
            for (int i = t; i < S / 4; i += GROUP) {
                float4 g = __ldg(g4 + i);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (RELU || train) v = __ldg(x4 + i);
                if (RELU) {
                    g.x = bn_value(v.x, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g.x : 0.f;
                    g.y = bn_value(v.y, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g.y : 0.f;
                    g.z = bn_value(v.z, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g.z : 0.f;
                    g.w = bn_value(v.w, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g.w : 0.f;
                }
                float4 o;
                if (train) {
                    o.x = (g.x - (v.x - k.mean) * k.proj - k.gmean) * k.gscale;
                    o.y = (g.y - (v.y - k.mean) * k.proj - k.gmean) * k.gscale;
                    o.z = (g.z - (v.z - k.mean) * k.proj - k.gmean) * k.gscale;
                    o.w = (g.w - (v.w - k.mean) * k.proj - k.gmean) * k.gscale;
                } else {
                    o.x = g.x * k.gscale; o.y = g.y * k.gscale; o.z = g.z * k.gscale; o.w = g.w * k.gscale;
                }
                o4[i] = o;
            }
        } else {
            for (int i = t; i < S; i += GROUP) {
                float g = __ldg(gp + i);
                const float v = (RELU || train) ? __ldg(xp + i) : 0.f;
                if (RELU) g = bn_value(v, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g : 0.f;
                op[i] = train ? (g - (v - k.mean) * k.proj - k.gmean) * k.gscale : g * k.gscale;
            }
        }
    }
}

// The flat walk of apply_flat_kernel for the input gradient.
template <bool RELU>
__global__ void __launch_bounds__(256)
grad_apply_flat_kernel(const float *__restrict__ x, const float *__restrict__ gy, float *__restrict__ gx,
                       const GradCoef *__restrict__ coef, int train, unsigned C, unsigned S, unsigned total)
{
    GradCoef k;
    auto fetch = [&](unsigned c) {
        const float4 *p = reinterpret_cast<const float4 *>(coef + c);
        const float4 a = __ldg(p), b = __ldg(p + 1);
        k.mean = a.x; k.proj = a.y; k.gmean = a.z; k.gscale = a.w;
        k.invstd = b.x; k.gamma = b.y; k.beta = b.z; k.pad = b.w;
    };
    auto one = [&](float v, float g) {
        if (RELU) g = bn_value(v, k.mean, k.invstd, k.gamma, k.beta) > 0.f ? g : 0.f;
        return train ? (g - (v - k.mean) * k.proj - k.gmean) * k.gscale : g * k.gscale;
    };
    auto item = [&](unsigned q, const float4 v, const float4 g) {
        const unsigned e = q * 4u, pl = e / S;
        unsigned r = e - pl * S, c = pl % C;
        fetch(c);
        const float vin[4] = {v.x, v.y, v.z, v.w}, gin[4] = {g.x, g.y, g.z, g.w};
        float out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[j] = one(vin[j], gin[j]);
            if (j < 3 && ++r == S) {
                r = 0;
                if (++c == C) c = 0;
                fetch(c);
            }
        }
        reinterpret_cast<float4 *>(gx)[q] = make_float4(out[0], out[1], out[2], out[3]);
    };
    const unsigned items = total / 4u, stride = gridDim.x * blockDim.x, tid = blockIdx.x * blockDim.x + threadIdx.x;
    const float4 *x4 = reinterpret_cast<const float4 *>(x), *g4 = reinterpret_cast<const float4 *>(gy);
    const bool need_x = RELU || train;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr unsigned U = 4;
    for (unsigned q = tid; q < items; q += U * stride) {
        float4 v[U], g[U];
#pragma unroll
        for (unsigned u = 0; u < U; ++u) {
            v[u] = zero;
            if (q + u * stride < items) {
                g[u] = __ldg(g4 + q + u * stride);
                if (need_x) v[u] = __ldg(x4 + q + u * stride);
            }
        }
#pragma unroll
        for (unsigned u = 0; u < U; ++u)
            if (q + u * stride < items) item(q + u * stride, v[u], g[u]);
    }
    if (tid < total - items * 4u) {
        const unsigned e = items * 4u + tid;
        fetch((e / S) % C);
        gx[e] = one(need_x ? __ldg(x + e) : 0.f, __ldg(gy + e));
    }
}

// Ticket counters at the start of the workspace: one per channel for the forward statistics, one for the gradient
// sums.  Zero when a call is enqueued, zero again when its kernels have run.
constexpr int kMaxCounterChannels = 4096;
constexpr size_t kCounterBytes = (size_t)2 * kMaxCounterChannels * sizeof(unsigned int);

// Chunks per channel so that C * chunks CTAs fill the GPU a few times over, at most one chunk per image.
static int pick_chunks(int N, int C)
{
    const int want = ceil_div(sm_count() * 8, C);
    return std::max(1, std::min(N, want));
}

// Planes of up to 1024 elements are handled by one warp each, larger ones by a whole CTA.
static bool small_planes(int S) { return S <= 1024; }
static int plane_grid(long long planes, int S)
{
    const long long cap = (long long)sm_count() * 16;
    const long long per_cta = small_planes(S) ? 8 : 1;
    return (int)std::max(1LL, std::min((planes + per_cta - 1) / per_cta, cap));
}

// Planes that are not a multiple of 16 bytes take the flat kernels (32-bit element indices, 16-byte aligned tensors).
static bool flat_applies(int S, long long planes, const void *a, const void *b, const void *c)
{
    return S % 4 != 0 && planes * S >= 4 && planes * S < (1LL << 32) && ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0);
}
static int flat_grid(unsigned total)
{
    return (int)std::max(1LL, std::min(ceil_div_ll((long long)(total / 4u), 1024), (long long)sm_count() * 8));
}

template <bool RELU>
static void launch_apply(const float *x, float *y, const float *weight, const float *bias, const float *mean_v,
                         const float *std_or_var, int train, float eps, int C, int S, long long planes, cudaStream_t stream)
{
    if (flat_applies(S, planes, x, y, y)) {
        const unsigned total = (unsigned)(planes * S);
        apply_flat_kernel<RELU><<<flat_grid(total), 256, 0, stream>>>(x, y, weight, bias, mean_v, std_or_var, train, eps, (unsigned)C, (unsigned)S, total);
        return;
    }
    if (small_planes(S)) apply_kernel<RELU, 32><<<plane_grid(planes, S), 256, 0, stream>>>(x, y, weight, bias, mean_v, std_or_var, train, eps, C, S, planes);
    else apply_kernel<RELU, 256><<<plane_grid(planes, S), 256, 0, stream>>>(x, y, weight, bias, mean_v, std_or_var, train, eps, C, S, planes);
}
template <bool RELU>
static void launch_grad_apply(const float *x, const float *gy, float *gx, const GradCoef *coef, int train, int C, int S,
                              long long planes, cudaStream_t stream)
{
    if (flat_applies(S, planes, x, gy, gx)) {
        const unsigned total = (unsigned)(planes * S);
        grad_apply_flat_kernel<RELU><<<flat_grid(total), 256, 0, stream>>>(x, gy, gx, coef, train, (unsigned)C, (unsigned)S, total);
        return;
    }
    if (small_planes(S)) grad_apply_kernel<RELU, 32><<<plane_grid(planes, S), 256, 0, stream>>>(x, gy, gx, coef, train, C, S, planes);
    else grad_apply_kernel<RELU, 256><<<plane_grid(planes, S), 256, 0, stream>>>(x, gy, gx, coef, train, C, S, planes);
}

}  // namespace bn
}  // namespace cunn

using namespace cunn;
using namespace cunn::bn;

// Workspace layout: [ticket counters, kCounterBytes] [chunk partials] [gradient coefficients].
extern "C" CUNN_API size_t cunn_b200_batchnorm_workspace(int N, int C)
{
    if (N <= 0 || C <= 0) return 0;
    const size_t chunks = (size_t)pick_chunks(N, C);
    return kCounterBytes + (((size_t)C * chunks * sizeof(ChunkStat) + 255) & ~(size_t)255) + (size_t)C * sizeof(GradCoef) + 256;
}

static int bn_forward_impl(const float *x, float *y, const float *weight, const float *bias, float *running_mean,
                           float *running_var, float *save_mean, float *save_std, int N, int C, int S, int train,
                           double momentum, double eps, void *workspace, size_t workspace_bytes, cunn_stream_t stream_,
                           bool relu)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    CUNN_CHECK_ARG(N >= 0 && C > 0 && S > 0, "bad batch-norm sizes N=%d C=%d S=%d", N, C, S);
    CUNN_CHECK_ARG((long long)N * C * (long long)S < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && y && running_mean && running_var, "null tensor pointer");
    const long long planes = (long long)N * C;
    if (train) {
        CUNN_CHECK_ARG(save_mean && save_std, "training-mode batch norm needs save_mean and save_std");
        const int chunks = pick_chunks(N, C);
        const size_t need = kCounterBytes + (size_t)C * chunks * sizeof(ChunkStat);
        CUNN_CHECK_ARG(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                       "batch norm needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                       workspace ? workspace_bytes : (size_t)0);
        unsigned int *counters = C <= kMaxCounterChannels ? (unsigned int *)workspace : nullptr;
        ChunkStat *part = (ChunkStat *)((char *)workspace + kCounterBytes);
        stats_kernel<<<C * chunks, 256, 0, stream>>>(x, part, N, C, S, chunks, counters, running_mean, running_var, save_mean,
                                                     save_std, momentum, eps);
        CUNN_LAUNCH_CHECK("batch norm statistics");
        if (!counters) {
            stats_finish_kernel<<<ceil_div(C, 128), 128, 0, stream>>>(part, C, chunks, running_mean, running_var, save_mean,
                                                                     save_std, momentum, eps);
            CUNN_LAUNCH_CHECK("batch norm statistics finish");
        }
        if (relu) launch_apply<true>(x, y, weight, bias, save_mean, save_std, 1, (float)eps, C, S, planes, stream);
        else launch_apply<false>(x, y, weight, bias, save_mean, save_std, 1, (float)eps, C, S, planes, stream);
    } else {
        if (relu) launch_apply<true>(x, y, weight, bias, running_mean, running_var, 0, (float)eps, C, S, planes, stream);
        else launch_apply<false>(x, y, weight, bias, running_mean, running_var, 0, (float)eps, C, S, planes, stream);
    }
    CUNN_LAUNCH_CHECK("batch norm apply");
    return 0;
}

extern "C" CUNN_API int cunn_b200_batchnorm_forward(const float *x, float *y, const float *weight, const float *bias,
                                                    float *running_mean, float *running_var, float *save_mean,
                                                    float *save_std, int N, int C, int S, int train, double momentum,
                                                    double eps, void *workspace, size_t workspace_bytes,
                                                    cunn_stream_t stream)
{
    return bn_forward_impl(x, y, weight, bias, running_mean, running_var, save_mean, save_std, N, C, S, train, momentum, eps,
                           workspace, workspace_bytes, stream, false);
}

extern "C" CUNN_API int cunn_b200_batchnorm_relu_forward(const float *x, float *y, const float *weight, const float *bias,
                                                         float *running_mean, float *running_var, float *save_mean,
                                                         float *save_std, int N, int C, int S, int train, double momentum,
                                                         double eps, void *workspace, size_t workspace_bytes,
                                                         cunn_stream_t stream)
{
    return bn_forward_impl(x, y, weight, bias, running_mean, running_var, save_mean, save_std, N, C, S, train, momentum, eps,
                           workspace, workspace_bytes, stream, true);
}

static int bn_backward_impl(const float *x, const float *gy, bool relu, const float *bias, float *gx, float *grad_weight,
                            float *grad_bias, const float *weight, const float *running_mean, const float *running_var,
                            const float *save_mean, const float *save_std, int N, int C, int S, int train, double scale,
                            double eps, void *workspace, size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    CUNN_CHECK_ARG(N >= 0 && C > 0 && S > 0, "bad batch-norm sizes N=%d C=%d S=%d", N, C, S);
    CUNN_CHECK_ARG((long long)N * C * (long long)S < (1LL << 31), "tensors of 2^31 or more elements are not supported");
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy, "null tensor pointer");
    CUNN_CHECK_ARG(train ? (save_mean && save_std) : (running_mean && running_var),
                   "batch norm backward needs %s", train ? "save_mean and save_std" : "running_mean and running_var");
    const int chunks = pick_chunks(N, C);
    const size_t part_bytes = ((size_t)C * chunks * sizeof(ChunkStat) + 255) & ~(size_t)255;
    const size_t need = kCounterBytes + part_bytes + (size_t)C * sizeof(GradCoef);
    CUNN_CHECK_ARG(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                   "batch norm backward needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                   workspace ? workspace_bytes : (size_t)0);
    unsigned int *counters = C <= kMaxCounterChannels ? (unsigned int *)workspace + kMaxCounterChannels : nullptr;
    float2 *part = (float2 *)((char *)workspace + kCounterBytes);
    GradCoef *coef = (GradCoef *)((char *)workspace + kCounterBytes + part_bytes);
    const float *mean_v = train ? save_mean : running_mean;
    const float *sv = train ? save_std : running_var;
    const long long planes = (long long)N * C;
    // inference-mode input gradient needs no sums; they are still required for gradWeight / gradBias
    const bool need_sums = train || grad_weight || grad_bias;
    if (need_sums) {
        if (relu) grad_stats_kernel<true><<<C * chunks, 256, 0, stream>>>(x, gy, part, mean_v, sv, weight, bias, train, (float)eps, N, C, S, chunks,
                                                                          counters, eps, scale, grad_weight, grad_bias, coef);
        else grad_stats_kernel<false><<<C * chunks, 256, 0, stream>>>(x, gy, part, mean_v, sv, weight, bias, train, (float)eps, N, C, S, chunks,
                                                                       counters, eps, scale, grad_weight, grad_bias, coef);
        CUNN_LAUNCH_CHECK("batch norm gradient sums");
    } else {
        CUNN_CUDA(cudaMemsetAsync(part, 0, (size_t)C * chunks * sizeof(float2), stream));
    }
    if (!need_sums || !counters) {
        grad_finish_kernel<<<ceil_div(C, 128), 128, 0, stream>>>(part, C, chunks, (long long)N * S, weight, bias, mean_v, sv, train,
                                                                eps, scale, grad_weight, grad_bias, coef);
        CUNN_LAUNCH_CHECK("batch norm gradient finish");
    }
    if (gx) {
        if (relu) launch_grad_apply<true>(x, gy, gx, coef, train, C, S, planes, stream);
        else launch_grad_apply<false>(x, gy, gx, coef, train, C, S, planes, stream);
        CUNN_LAUNCH_CHECK("batch norm input gradient");
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_batchnorm_backward(const float *x, const float *gy, float *gx, float *grad_weight,
                                                     float *grad_bias, const float *weight, const float *running_mean,
                                                     const float *running_var, const float *save_mean,
                                                     const float *save_std, int N, int C, int S, int train, double scale,
                                                     double eps, void *workspace, size_t workspace_bytes,
                                                     cunn_stream_t stream)
{
    return bn_backward_impl(x, gy, false, nullptr, gx, grad_weight, grad_bias, weight, running_mean, running_var, save_mean, save_std,
                            N, C, S, train, scale, eps, workspace, workspace_bytes, stream);
}

extern "C" CUNN_API int cunn_b200_batchnorm_relu_backward(const float *x, const float *gy, float *gx, float *grad_weight,
                                                          float *grad_bias, const float *weight, const float *bias,
                                                          const float *running_mean, const float *running_var,
                                                          const float *save_mean, const float *save_std, int N, int C,
                                                          int S, int train, double scale, double eps, void *workspace,
                                                          size_t workspace_bytes, cunn_stream_t stream)
{
    return bn_backward_impl(x, gy, true, bias, gx, grad_weight, grad_bias, weight, running_mean, running_var, save_mean, save_std, N, C,
                            S, train, scale, eps, workspace, workspace_bytes, stream);
}
