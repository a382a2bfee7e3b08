// SpatialConvolutionMM on the 5th-generation tensor cores (tcgen05 / TMEM), fp32 in and out.
//
// The reference unfolds every image into a column buffer and calls SGEMM per image.  Here the three
// passes are implicit GEMMs — no column buffer exists — computed by tcgen05.mma.kind::tf32 with a
// 3xTF32 split: every fp32 operand value v is used as hi (its upper 19 bits) and lo = v - hi, and each
// K step issues lo*hi + hi*lo + hi*hi into fp32 TMEM accumulators.  The dropped lo*lo term and the tf32
// truncation of lo are ~2^-20 relative, i.e. fp32-class accuracy.
//
//   forward      D[pixel, k_out]        = sum_{c,kh,kw}  x(pixel; c,kh,kw)   * W[k_out][c,kh,kw]
//   input grad   D[pixel, c]            = sum_{k,kh,kw}  gy(pixel; k,kh,kw)  * W[k][c][flipped kh,kw]   (stride 1)
//   weight grad  D[k_out, (c,kh,kw)]    = sum_{img,pix}  gy[img][k_out][pix] * x(pix; c,kh,kw)          (split over images)
//
// Three kernel families share these roles:
//   * pw::pw_gemm_kernel<OP, BN, KS> — the persistent, warp-specialised kernel (further down): KS = 1 for 1x1
//     stride-1 convolutions whose operands are plain matrices in memory, KS = 3 / 0 for 3x3 / any kernel of up to
//     32 taps gathered element by element with asynchronous copies;
//   * conv_gemm_kernel<OP, KS, BN> (next) — one CTA per 128 x BN tile for kernels of more than 32 taps: all 256
//     threads gather operand values (two k-blocks in flight in registers), split them and store 16-byte pieces
//     into K-major tiles in the 128-byte swizzle; one thread issues the MMAs of the k-block and commits them to
//     the mbarrier that frees the stage; the epilogue reads the accumulator with tcgen05.ld (lane = tile row)
//     and writes coalesced NCHW rows;
//   * stemconv.cu — fp32-pipe kernels for the 3-channel 3x3 first layer.
// Every wait is bounded.  Input gradients for stride > 1 use a plain gather kernel (no network on the
// benchmarked path needs them: a strided first layer has no input gradient).
#include "common.cuh"
#include "stemconv.h"

#include <algorithm>

namespace cunn {
namespace mm {

enum Op : int { OP_FWD = 0, OP_DGRAD = 1, OP_WGRAD = 2 };

constexpr int BM = 128;       // tile rows (TMEM lanes)
constexpr int BK = 32;        // k-block: 8 chunks of 4 values (16 bytes)
constexpr int THREADS = 256;
constexpr int SBO = 1024;     // bytes between 8-row groups of a K-major tile (rows of 128 bytes = one k-block)

struct GemmParams {
    const float *a_src;   // FWD: x; DGRAD: gy; WGRAD: gy
    const float *b_src;   // FWD: W; DGRAD: W; WGRAD: x
    const float *bias;    // FWD only, may be null
    float *out;           // FWD: y; DGRAD: gx; WGRAD: partial sums [splits][M_total][N_total]
    int *status;
    // geometry of the gathered image operand (FWD: x; DGRAD: gy; WGRAD: x)
    int g_C, g_H, g_W;            // channels, rows, cols of that tensor
    int g_padH, g_padW, g_dH, g_dW;
    int kH, kW;
    int pix_W, pix_HW;            // row length and plane size of the pixel grid the gather is driven by
    // convolution sizes
    int C, K;                     // input / output channels
    int n_img;
    // GEMM sizes
    int M_total, N_total, Kd;
    int kblocks;                  // k-blocks per CTA
    int out_HW;                   // FWD / DGRAD: pixels per image of the output tensor
    // WGRAD
    int imgs_per_split, pix_blocks;  // images per split, k-blocks per image
};

// ---- tcgen05 wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with accumulation always on: no predicate to set up.
__device__ __forceinline__ void umma_tf32_acc(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc)
{
    asm volatile("tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, 1;" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has finished reading shared memory
// and writing TMEM.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major tile in the 128-byte swizzle (row r holds its eight 16-byte chunks
// at positions chunk ^ (r & 7); groups of 8 rows are 1024 bytes apart).  The tensor core reads this form without
// bank conflicts; the unswizzled 8 x 16-byte core-matrix form measured about 20 % slower.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(SBO >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::tf32: fp32 accumulator, tf32 A and B, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t instr_desc(int n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// hi = v rounded to tf32 (low 13 mantissa bits zero), lo = v - hi (exact in fp32).
__device__ __forceinline__ void split_tf32(float v, float &hi, float &lo)
{
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    hi = __uint_as_float(h);
    lo = v - hi;
}

// Byte offset of the 16-byte piece (row, chunk) inside an operand tile.
__device__ __forceinline__ uint32_t piece_offset(int row, int kc) { return (uint32_t)(row * 128 + ((kc ^ (row & 7)) << 4)); }

__device__ __forceinline__ void store_split(unsigned char *hi_tile, unsigned char *lo_tile, int row, int kc, const float4 &v)
{
    float4 h, l;
    split_tf32(v.x, h.x, l.x);
    split_tf32(v.y, h.y, l.y);
    split_tf32(v.z, h.z, l.z);
    split_tf32(v.w, h.w, l.w);
    const uint32_t off = piece_offset(row, kc);
    *reinterpret_cast<float4 *>(hi_tile + off) = h;
    *reinterpret_cast<float4 *>(lo_tile + off) = l;
}

// k index -> (channel, kh, kw).  KS = 1 or 3 makes the divisions compile-time; KS = 0 is generic.
template <int KS>
__device__ __forceinline__ void split_k(const GemmParams &p, int k, int &c, int &kh, int &kw)
{
    if (KS == 1) { c = k; kh = 0; kw = 0; }
    else if (KS == 3) { c = k / 9; const int r = k - c * 9; kh = r / 3; kw = r - kh * 3; }
    else { const int kk = p.kH * p.kW; c = k / kk; const int r = k - c * kk; kh = r / p.kW; kw = r - kh * p.kW; }
}

// Row of the gathered image operand: which image, and the top-left corner of its window.
struct PixRow {
    const float *img;   // channel 0 of this pixel's image in the gathered tensor (null: row outside the problem)
    int ih0, iw0;
};

// Four consecutive k values of the gathered operand for one pixel row (zero outside the image / problem).
template <int KS>
__device__ __forceinline__ float4 gather_pix_chunk(const GemmParams &p, const PixRow &r, int k0)
{
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int k = k0 + j;
        float x = 0.f;
        if (r.img && k < p.Kd) {
            int c, kh, kw;
            split_k<KS>(p, k, c, kh, kw);
            const int ih = r.ih0 + kh, iw = r.iw0 + kw;
            if ((unsigned)ih < (unsigned)p.g_H && (unsigned)iw < (unsigned)p.g_W)
                x = __ldg(r.img + ((size_t)c * p.g_H + ih) * p.g_W + iw);
        }
        v[j] = x;
    }
    return make_float4(v[0], v[1], v[2], v[3]);
}

// Four consecutive values of a row-major [rows][len] matrix row (zero past the end).
__device__ __forceinline__ float4 rowmajor_chunk(const float *row, int k0, int len, bool vec_ok)
{
    if (!row || k0 >= len) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec_ok && k0 + 3 < len) return __ldg(reinterpret_cast<const float4 *>(row + k0));
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (k0 + j < len) ? __ldg(row + k0 + j) : 0.f;
    return make_float4(v[0], v[1], v[2], v[3]);
}

template <int OP, int KS, int BN>
__global__ void __launch_bounds__(THREADS, 1)
conv_gemm_kernel(const GemmParams p)
{
    constexpr int A_TILE = BM * BK * 4;             // bytes of one hi (or lo) A tile
    constexpr int B_TILE = BN * BK * 4;
    constexpr int STAGE = 2 * (A_TILE + B_TILE);
    constexpr int STAGES = (STAGE * 4 <= 200 * 1024) ? 4 : (STAGE * 3 <= 200 * 1024 ? 3 : 2);
    constexpr int A_PER = BM * 8 / THREADS;         // 16-byte pieces per thread per k-block
    constexpr int B_PER = (BN * 8 + THREADS - 1) / THREADS;
    // The tensor core adds each MMA result into its fp32 accumulator with truncation, so a long chain of
    // accumulations drifts (error grows with the number of steps).  K-blocks are therefore dealt
    // round-robin to NACC independent TMEM accumulators, which the epilogue adds up in fp32: chains are
    // NACC times shorter and their partial sums smaller.
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    constexpr int NACC = (512 / ACC_COLS) > 8 ? 8 : (512 / ACC_COLS);
    constexpr uint32_t TMEM_COLS = ACC_COLS * NACC;

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[STAGES + 1];           // stage-free barriers + accumulator-ready barrier
    __shared__ uint32_t tmem_base_s;
    __shared__ int pixtab[2][BK][2];                // WGRAD: (ih0, iw0) of the 32 pixels of a k-block, double buffered

    const int tid = threadIdx.x, warp = tid >> 5;
    const int m0 = blockIdx.x * BM;                 // first tile row
    const int n0 = blockIdx.y * BN;                 // first tile column
    const int split = blockIdx.z;                   // WGRAD: image range

    if (tid == 0) {
        for (int s = 0; s <= STAGES; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // ---- per-thread operand rows ------------------------------------------------------------------
    // A pieces: row = tid % 128, chunks kc = tid / 128 + 2 i.  B pieces: piece q = i * 256 + tid -> row q % BN, chunk q / BN.
    const int a_row = tid & (BM - 1);
    const int a_kc0 = tid >> 7;
    PixRow a_pix{nullptr, 0, 0};
    const float *a_rowptr = nullptr;                // WGRAD: gy row of this k_out (per image offset added later)
    if (OP != OP_WGRAD) {
        const int m = m0 + a_row;
        if (m < p.M_total) {
            const int img = m / p.pix_HW, pix = m - img * p.pix_HW;
            const int ph = pix / p.pix_W, pw = pix - ph * p.pix_W;
            a_pix.img = p.a_src + (size_t)img * p.g_C * p.g_H * p.g_W;
            a_pix.ih0 = ph * p.g_dH - p.g_padH;
            a_pix.iw0 = pw * p.g_dW - p.g_padW;
        }
    } else {
        const int m = m0 + a_row;
        if (m < p.M_total) a_rowptr = p.a_src + (size_t)m * p.pix_HW;   // + img * K * oHW
    }
    const bool b_vec = (OP == OP_FWD) ? ((p.Kd & 3) == 0 && ((uintptr_t)p.b_src & 15) == 0)
                                      : (OP == OP_WGRAD && KS == 1 && (p.pix_HW & 3) == 0 && ((uintptr_t)p.b_src & 15) == 0 &&
                                         p.g_dH == 1 && p.g_dW == 1 && p.g_padH == 0 && p.g_padW == 0);
    const bool a_vec = OP == OP_WGRAD && (p.pix_HW & 3) == 0 && ((uintptr_t)p.a_src & 15) == 0;

    // Loads the pieces of k-block `kb` (CTA-local index) into registers.
    auto load_block = [&](int kb, float4 (&ra)[A_PER], float4 (&rb)[B_PER]) {
        if (OP != OP_WGRAD) {
            const int kbase = kb * BK;
#pragma unroll
            for (int i = 0; i < A_PER; ++i) ra[i] = gather_pix_chunk<KS>(p, a_pix, kbase + (a_kc0 + 2 * i) * 4);
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const int q = i * THREADS + tid;
                const int row = q % BN, kc = q / BN;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (kc < 8 && n0 + row < p.N_total) {
                    const int k0 = kbase + kc * 4;
                    if (OP == OP_FWD) {
                        v = rowmajor_chunk(p.b_src + (size_t)(n0 + row) * p.Kd, k0, p.Kd, b_vec);
                    } else {
                        // DGRAD: B[c][(ko,kh,kw)] = W[ko][c][kH-1-kh][kW-1-kw]
                        float t[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int k = k0 + j;
                            float x = 0.f;
                            if (k < p.Kd) {
                                int ko, kh, kw;
                                split_k<KS>(p, k, ko, kh, kw);
                                x = __ldg(p.b_src + (((size_t)ko * p.C + (n0 + row)) * p.kH + (p.kH - 1 - kh)) * p.kW + (p.kW - 1 - kw));
                            }
                            t[j] = x;
                        }
                        v = make_float4(t[0], t[1], t[2], t[3]);
                    }
                }
                rb[i] = v;
            }
        } else {
            // k runs over (image, pixel); a k-block never straddles images
            const int img = split * p.imgs_per_split + kb / p.pix_blocks;
            const int pb = kb - (kb / p.pix_blocks) * p.pix_blocks;
            const bool img_ok = img < p.n_img && kb / p.pix_blocks < p.imgs_per_split;
#pragma unroll
            for (int i = 0; i < A_PER; ++i) {
                const int k0 = pb * BK + (a_kc0 + 2 * i) * 4;
                ra[i] = rowmajor_chunk((img_ok && a_rowptr) ? a_rowptr + (size_t)img * p.K * p.pix_HW : nullptr, k0, p.pix_HW, a_vec);
            }
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const int q = i * THREADS + tid;
                const int row = q % BN, kc = q / BN;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int n = n0 + row;
                if (kc < 8 && n < p.N_total && img_ok) {
                    int c, kh, kw;
                    split_k<KS>(p, n, c, kh, kw);
                    const float *plane = p.b_src + ((size_t)img * p.C + c) * p.g_H * p.g_W;
                    const int k0 = pb * BK + kc * 4;
                    if (b_vec) {
                        v = rowmajor_chunk(plane, k0, p.pix_HW, true);
                    } else {
                        float t[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int pix = k0 + j;
                            float x = 0.f;
                            if (pix < p.pix_HW) {
                                const int ih = pixtab[kb & 1][kc * 4 + j][0] + kh, iw = pixtab[kb & 1][kc * 4 + j][1] + kw;
                                if ((unsigned)ih < (unsigned)p.g_H && (unsigned)iw < (unsigned)p.g_W) x = __ldg(plane + (size_t)ih * p.g_W + iw);
                            }
                            t[j] = x;
                        }
                        v = make_float4(t[0], t[1], t[2], t[3]);
                    }
                }
                rb[i] = v;
            }
        }
    };
    // WGRAD: window corners of the 32 pixels of k-block kb (same for every image)
    auto fill_pixtab = [&](int kb) {
        if (OP == OP_WGRAD && tid < BK) {
            const int pb = kb % p.pix_blocks;
            const int pix = pb * BK + tid;
            const int oh = pix / p.pix_W, ow = pix - oh * p.pix_W;
            pixtab[kb & 1][tid][0] = oh * p.g_dH - p.g_padH;
            pixtab[kb & 1][tid][1] = ow * p.g_dW - p.g_padW;
        }
    };
    auto store_block = [&](int stage, const float4 (&ra)[A_PER], const float4 (&rb)[B_PER]) {
        unsigned char *sa_hi = smem + (size_t)stage * STAGE;
        unsigned char *sa_lo = sa_hi + A_TILE;
        unsigned char *sb_hi = sa_lo + A_TILE;
        unsigned char *sb_lo = sb_hi + B_TILE;
#pragma unroll
        for (int i = 0; i < A_PER; ++i) store_split(sa_hi, sa_lo, a_row, a_kc0 + 2 * i, ra[i]);
#pragma unroll
        for (int i = 0; i < B_PER; ++i) {
            const int q = i * THREADS + tid;
            const int row = q % BN, kc = q / BN;
            if (kc < 8) store_split(sb_hi, sb_lo, row, kc, rb[i]);
        }
    };
    auto issue_mmas = [&](int stage, int kb) {
        const uint32_t d_tmem = tmem_base + (uint32_t)((kb % NACC) * ACC_COLS);
        const bool first = kb < NACC;   // first k-block of this accumulator overwrites it
        const uint32_t sa_hi = smem_u32(smem + (size_t)stage * STAGE);
        const uint32_t sa_lo = sa_hi + A_TILE, sb_hi = sa_lo + A_TILE, sb_lo = sb_hi + B_TILE;
        constexpr uint32_t idesc = instr_desc(BN < 16 ? 16 : BN);
#pragma unroll
        for (int j = 0; j < BK / 8; ++j) {
            const uint32_t koff = (uint32_t)j * 32;           // two 16-byte chunks per MMA; the swizzle is applied to the address
            const uint64_t ah = smem_desc(sa_hi + koff), al = smem_desc(sa_lo + koff);
            const uint64_t bh = smem_desc(sb_hi + koff), bl = smem_desc(sb_lo + koff);
            umma_tf32(d_tmem, al, bh, idesc, (first && j == 0) ? 0u : 1u);
            umma_tf32(d_tmem, ah, bl, idesc, 1u);
            umma_tf32(d_tmem, ah, bh, idesc, 1u);
        }
    };

    // ---- main loop: two k-blocks in flight in registers, STAGES in shared memory -------------------
    const int KB = p.kblocks;
    float4 ra0[A_PER], rb0[B_PER], ra1[A_PER], rb1[B_PER];
    bool ok = true;
    fill_pixtab(0);
    if (OP == OP_WGRAD) __syncthreads();
    if (KB > 0) load_block(0, ra0, rb0);
    fill_pixtab(1);
    if (OP == OP_WGRAD) __syncthreads();
    if (KB > 1) load_block(1, ra1, rb1);
    for (int kb = 0; kb < KB && ok; kb += 2) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int k = kb + half;
            if (k >= KB) break;
            const int stage = k % STAGES;
            if (k >= STAGES) {
                // the MMAs that read this stage (k-block k - STAGES) must have finished
                if (!mbar_wait(smem_u32(bars + stage), (uint32_t)(((k / STAGES) - 1) & 1), p.status)) { ok = false; break; }
            }
            if (half == 0) store_block(stage, ra0, rb0);
            else store_block(stage, ra1, rb1);
            fence_async_smem();          // generic-proxy stores -> visible to the tensor core's async proxy
            fill_pixtab(k + 2);          // (k + 2) & 1 == k & 1: this block's table is no longer needed after the sync below
            __syncthreads();
            if (tid == 0) {
                tc_fence_after();
                issue_mmas(stage, k);
                umma_commit(smem_u32(bars + stage));
            }
            if (k + 2 < KB) {
                if (half == 0) load_block(k + 2, ra0, rb0);
                else load_block(k + 2, ra1, rb1);
            }
        }
    }
    // ---- epilogue ----------------------------------------------------------------------------------
    if (tid == 0) umma_commit(smem_u32(bars + STAGES));      // arrives when every MMA above has completed
    if (ok && KB > 0) ok = mbar_wait(smem_u32(bars + STAGES), 0u, p.status);
    tc_fence_after();
    if (ok) {
        const int quarter = warp & 3;                // TMEM lanes this warp may read
        const int row = quarter * 32 + (tid & 31);   // tile row == TMEM lane
        const int m = m0 + row;
        constexpr int HALF = (BN >= 64) ? BN / 2 : BN;
        const int col_begin = (BN >= 64) ? (warp >> 2) * HALF : 0;
        const bool do_cols = (BN >= 64) || (warp < 4);
        size_t out_base = 0;
        if (OP != OP_WGRAD && m < p.M_total) {
            const int img = m / p.out_HW, pix = m - img * p.out_HW;
            out_base = (size_t)img * p.N_total * p.out_HW + pix;
        }
        if (do_cols) {
            for (int cc = col_begin; cc < col_begin + HALF; cc += 32) {
                float acc[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = 0.f;
                const int nacc = KB < NACC ? KB : NACC;   // accumulators that received at least one k-block
                for (int a = 0; a < nacc; ++a) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * ACC_COLS + cc), r);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(r[j]);
                }
                if (m < p.M_total) {
                    if (OP != OP_WGRAD) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int n = n0 + cc + j;
                            if (cc + j < BN && n < p.N_total) {
                                float v = acc[j];
                                if (OP == OP_FWD && p.bias) v += __ldg(p.bias + n);
                                p.out[out_base + (size_t)n * p.out_HW] = v;
                            }
                        }
                    } else {
                        float *dst = p.out + ((size_t)split * p.M_total + m) * p.N_total + n0 + cc;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (cc + j < BN && n0 + cc + j < p.N_total) dst[j] = acc[j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// gW[i] += scale * sum_s partial[s][i], in split order.
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float *__restrict__ partial, float *__restrict__ gw, long long n, int splits, float scale)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += __ldg(partial + (size_t)k * n + i);
        gw[i] += scale * s;
    }
}

// Bias gradient: gb[k] += scale * sum over images and pixels of gy[img][k][pix].  One CTA per (k, chunk).
__global__ void __launch_bounds__(256)
bias_partial_kernel(const float *__restrict__ gy, float *__restrict__ part, int n_img, int K, int HW, int chunks)
{
    __shared__ float sh[8];
    const int k = blockIdx.x / chunks, j = blockIdx.x % chunks;
    const int per = n_img / chunks, extra = n_img % chunks;
    const int i0 = j * per + min(j, extra), i1 = i0 + per + (j < extra ? 1 : 0);
    float s = 0.f;
    for (int img = i0; img < i1; ++img) {
        const float *g = gy + ((size_t)img * K + k) * HW;
        for (int i = threadIdx.x; i < HW; i += blockDim.x) s += __ldg(g + i);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[w];
        part[blockIdx.x] = t;
    }
}
__global__ void __launch_bounds__(128)
bias_finish_kernel(const float *__restrict__ part, float *__restrict__ gb, int K, int chunks, float scale)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= K) return;
    double s = 0.0;
    for (int j = 0; j < chunks; ++j) s += (double)part[k * chunks + j];
    gb[k] = (float)((double)gb[k] + (double)scale * s);
}

// Both reductions of a weight-gradient pass in one launch: gW[i] += scale * sum_s partial[s][i] for i < n, and
// gb[k] += scale * sum_j bias_part[k][j] for the K threads after them (bias_part may be null).
__global__ void __launch_bounds__(256)
wgrad_bias_reduce_kernel(const float *__restrict__ partial, float *__restrict__ gw, long long n, int splits, float scale,
                         const float *__restrict__ bias_part, float *__restrict__ gb, int K)
{
    const long long total = n + (bias_part ? K : 0);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        if (i < n) {
            float s = 0.f;
            for (int k = 0; k < splits; ++k) s += __ldg(partial + (size_t)k * n + i);
            gw[i] += scale * s;
        } else {
            const int k = (int)(i - n);
            double s = 0.0;
            for (int j = 0; j < splits; ++j) s += (double)bias_part[(size_t)k * splits + j];
            gb[k] = (float)((double)gb[k] + (double)scale * s);
        }
    }
}

// y[img][q][pix] += bias[q]: the bias of a transposed convolution, whose product comes out of the input-gradient kernels.
__global__ void __launch_bounds__(256)
add_plane_bias_kernel(float *__restrict__ y, const float *__restrict__ bias, int Q, int HW, long long total)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        y[i] += __ldg(bias + (int)((i / HW) % Q));
}

// Input gradient for any stride: gather form, one thread per input pixel (correctness path).
__global__ void __launch_bounds__(256)
dgrad_gather_kernel(const float *__restrict__ gy, const float *__restrict__ w, float *__restrict__ gx, int C, int H, int W,
                    int K, int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int oH, int oW, long long total)
{
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int wi = (int)(idx % W);
        long long t = idx / W;
        const int h = (int)(t % H);
        t /= H;
        const int c = (int)(t % C);
        const long long n = t / C;
        float s = 0.f;
        for (int kh = 0; kh < kH; ++kh) {
            const int a = h + padH - kh * dilH;
            if (a < 0 || a % dH) continue;
            const int oh = a / dH;
            if (oh >= oH) continue;
            for (int kw = 0; kw < kW; ++kw) {
                const int b = wi + padW - kw * dilW;
                if (b < 0 || b % dW) continue;
                const int ow = b / dW;
                if (ow >= oW) continue;
                for (int k = 0; k < K; ++k)
                    s = fmaf(__ldg(w + (((size_t)k * C + c) * kH + kh) * kW + kw), __ldg(gy + ((n * K + k) * oH + oh) * (size_t)oW + ow), s);
            }
        }
        gx[idx] = s;
    }
}

// ---------------------------------------------------------------------------
// Pointwise convolutions (1x1, stride 1, no padding): persistent kernel
// ---------------------------------------------------------------------------
//
// A 1x1 convolution is a plain matrix product per image and every operand is already laid out the way the
// tensor core can take it, so nothing is gathered element by element:
//
//   forward      D[pixel, ko] = sum_c  x[img][c][pix]   * W[ko][c]      A: 4 pixels of one channel = 16 contiguous bytes (M-major)
//                                                                        B: 4 channels of one filter = 16 contiguous bytes (K-major)
//   input grad   D[pixel, c]  = sum_ko gy[img][ko][pix] * W[ko][c]      A: M-major as above;  B: 4 channels c of one ko (N-major)
//   weight grad  D[ko, c]     = sum_{img,pix} gy[img][ko][pix] * x[img][c][pix]      A, B: 4 pixels of one row (K-major);
//                                                                        k runs over (image, pixel) of this tile's image range
//
// tcgen05.mma takes M/N-major operands through the major bits of the instruction descriptor, so a 16-byte
// asynchronous copy lands an operand piece in shared memory in its final place, no transposition.  One CTA per SM
// walks a strided list of tiles; operand copies run three k-blocks ahead of the MMAs ACROSS tile boundaries, and
// four epilogue warps drain finished accumulators to global memory while the next tile is being produced (when the
// accumulators fit twice in TMEM the MMAs of the next tile run under it as well).
namespace pw {

constexpr int PRODUCERS = 512;           // threads that copy, split and run the epilogue (16 warps)
constexpr int EPILOGUE_WARPS = 4;         // warps that only drain accumulators: TMEM -> registers -> global memory
constexpr int THREADS = PRODUCERS + 32 + 32 * EPILOGUE_WARPS;   // + one warp that only issues the MMAs
constexpr int TILE = 128 * 128;          // 128 rows x 32 k values (16 KiB) in either layout
constexpr int MN_ATOM = 512;             // M/N-major tile: bytes of one swizzle atom (32 rows x 4 k values)
constexpr int MN_KATOM = 4 * MN_ATOM;    // ... bytes from one group of 4 k values to the next (4 atoms cover 128 rows)
constexpr int RAW_STAGES = 4;            // raw fp32 tiles (A, B) filled by asynchronous copies; split in place they become the hi tiles
constexpr int LO_BUFS = 2;               // lo tiles (A, B) of the k-blocks whose MMAs are in flight
constexpr int PREFETCH = 3;              // k-blocks the copies run ahead of the MMAs
constexpr int STAGE_COLS = 64;           // output columns staged at a time for the bulk-store epilogue (x 128 rows x 4 bytes)
constexpr size_t OUT_STAGE = (size_t)STAGE_COLS * BM * 4;
constexpr size_t SMEM = (size_t)(RAW_STAGES + LO_BUFS) * 2 * TILE + OUT_STAGE + 1024;
static_assert(8 * MN_KATOM == TILE, "both layouts fill the tile");

struct Params {
    const float *a, *b, *bias;
    float *out;        // FWD: y; DGRAD: gx; WGRAD: partial sums [splits][M_total][N_total]
    float *bias_part;  // WGRAD: [M_total][splits] row sums of gy, or null
    int *status;
    int HW;            // pixels per image plane
    int M_total, N_total, Kd;
    int n_tiles, tiles_per_split, total_tiles;   // tile = (split * m_tiles + m_tile) * n_tiles + n_tile
    int kblocks;       // k-blocks per tile
    int n_img, imgs_per_split, splits;
    int vec_a, vec_b;  // 16-byte global loads allowed for A / B
    // kernels larger than 1x1 (KS != 1): the unfolded operand is gathered from a [g_C, g_H, g_W] image tensor, the
    // pixel grid that drives the gather is pix_W wide (HW = its size)
    int g_C, g_H, g_W, kH, kW, dH, dW, padH, padW, pix_W;
    int dilH, dilW;    // distance between kernel taps (SpatialDilatedConvolution; 1 for SpatialConvolutionMM)
    int nacc, sets;    // accumulators per tile (nacc - 1 for the hi*hi products, k-blocks round-robin, + 1 for the cross terms), accumulator sets in TMEM (1 or 2)
    int bulk_out;      // FWD/DGRAD: planes of >= 1024 pixels (a multiple of 4), 16-byte aligned output: the columns of a tile leave as bulk stores
    int gpi;           // tensor-map kernels: groups of 32 pixels per image, ceil(HW / 32)
};

// 3xTF32 split of a raw fp32 tile in place.  The tensor core reads only the upper 19 bits of a tf32 operand,
// so the raw value itself serves as hi = v with the low 13 mantissa bits dropped; lo = v - hi is exact in fp32
// and is the only tile that has to be written.
__device__ __forceinline__ float lo_part(float v) { return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u); }
__device__ __forceinline__ void store_lo_at(unsigned char *lo_tile, uint32_t off, const float4 &v)
{
    *reinterpret_cast<float4 *>(lo_tile + off) = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
}
__device__ __forceinline__ uint64_t desc_of(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// M/N-major operand in the 128B-base-32B swizzle: leading offset = atom to atom along M/N, stride offset = along K.
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr)
{
    return desc_of(addr, MN_ATOM, MN_KATOM) | (1ull << 61);
}
__host__ __device__ constexpr uint32_t idesc_of(int n, bool a_mn, bool b_mn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ float4 ldg4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// Asynchronous 16- and 4-byte copies global -> shared; `on` false writes zeros without reading `src`.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool on)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(on ? 16u : 0u) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, bool on)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(on ? 4u : 0u) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 1-D bulk copy shared -> global through the TMA unit (16-byte aligned addresses, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_s2g_nocommit(void *dst, uint32_t src_smem, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Barrier among the producer warps only (hardware barrier 2).
__device__ __forceinline__ void producers_sync() { asm volatile("bar.sync 2, %0;" ::"n"(PRODUCERS) : "memory"); }
// Barrier among the epilogue warps only (hardware barrier 1; barrier 0 is __syncthreads).
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * EPILOGUE_WARPS) : "memory"); }

// Where the operand loads of one thread stand: tile, k-block and the thread's element offsets inside that tile.
// M/N-major pieces: lane = group of 4 rows, k = warp + 16 i.  K-major pieces: chunk kc = tid & 7, rows (tid >> 3) + 64 i.
// KS = 1: pointwise.  KS = 3 / 0: 3x3 / any kernel of up to 32 taps, any stride and padding: the same tiles, but
// the unfolded operand is gathered with 4-byte copies (zero-filled outside the image).
template <int OP, int BN, int KS>
struct Loader {
    int tile, kb;
    int a_off[4];       // FWD/DGRAD: element offsets of the thread's 4 pixels (channel 0); WGRAD: [0..1] row offsets
    int b_off[2];       // FWD: offsets of the thread's two filter rows (+ chunk); DGRAD: [0] first column; WGRAD: row offsets
    unsigned a_mask, b_mask;
    int img, pix, img_end;   // WGRAD: image and pixel of the thread's chunk in the current k-block
    unsigned tapmask[4];     // KS != 1, FWD/DGRAD: bit t set when tap t of pixel j lies inside the image
    int img2, pix2;          // KS != 1, WGRAD: image and pixel of this lane's column (k = lane) of the unfolded operand

    __device__ __forceinline__ int taps(const Params &p) const { return KS == 3 ? 9 : p.kH * p.kW; }
    __device__ __forceinline__ int kcols(const Params &p) const { return KS == 3 ? 3 : p.kW; }

    // rowtab (KS != 1, WGRAD): shared table of the tile's 128 unfolded rows: x = offset of the row's tap inside an image
    // (-1: row outside the problem), y = tap row offset | tap column offset << 16 (dilation applied)
    __device__ __forceinline__ void setup(const Params &p, int t, int2 *rowtab)
    {
        const int tid = threadIdx.x, lane = tid & 31;
        tile = t;
        kb = 0;
        a_mask = b_mask = 0;
        if (OP != OP_WGRAD) {
            const int m_tile = t / p.n_tiles, n_tile = t - m_tile * p.n_tiles;
            const int m = m_tile * BM + lane * 4, n0 = n_tile * BN;
            if (KS != 1) {
                // gathered operand: this lane's four rows are lane, lane + 32, lane + 64, lane + 96, so that one copy
                // instruction of the warp covers 32 consecutive pixels (and 128 consecutive bytes of shared memory)
                const int kk = taps(p), kw_n = kcols(p);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    a_off[j] = 0;
                    tapmask[j] = 0;
                    const int mj = m_tile * BM + lane + 32 * j;
                    if (mj < p.M_total) {
                        const int im = mj / p.HW, r = mj - im * p.HW;
                        const int ph = r / p.pix_W, pw_ = r - ph * p.pix_W;
                        const int ih0 = ph * p.dH - p.padH, iw0 = pw_ * p.dW - p.padW;
                        a_off[j] = im * p.g_C * p.g_H * p.g_W + ih0 * p.g_W + iw0;
                        a_mask |= 1u << j;
                        for (int t2 = 0; t2 < kk; ++t2) {
                            const int kh = t2 / kw_n, kw = t2 - kh * kw_n;
                            if ((unsigned)(ih0 + kh * p.dilH) < (unsigned)p.g_H && (unsigned)(iw0 + kw * p.dilW) < (unsigned)p.g_W) tapmask[j] |= 1u << t2;
                        }
                    }
                }
            } else if (p.vec_a) {
                if (m < p.M_total) {
                    const int im = m / p.HW;
                    a_off[0] = im * p.Kd * p.HW + (m - im * p.HW);
                    a_mask = 15u;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    a_off[j] = 0;
                    if (m + j < p.M_total) {
                        const int im = (m + j) / p.HW;
                        a_off[j] = im * p.Kd * p.HW + (m + j - im * p.HW);
                        a_mask |= 1u << j;
                    }
                }
            }
            if (OP == OP_FWD) {
                const int kc = tid & 7;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int row = (tid >> 3) + 64 * i, n = n0 + row;
                    b_off[i] = n * p.Kd + kc * 4;
                    if (row < BN && n < p.N_total) b_mask |= 1u << i;
                }
            } else {
                if (KS != 1) {
                    b_off[0] = n0 + lane;                  // gathered: columns lane + 32 j
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (lane + 32 * j < BN && n0 + lane + 32 * j < p.N_total) b_mask |= 1u << j;
                } else {
                    const int col = n0 + lane * 4;
                    b_off[0] = col;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (lane * 4 < BN && col + j < p.N_total) b_mask |= 1u << j;
                }
            }
        } else {
            const int split = t / p.tiles_per_split, r = t - split * p.tiles_per_split;
            const int m_tile = r / p.n_tiles, n_tile = r - m_tile * p.n_tiles;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = (tid >> 3) + 64 * i;
                const int m = m_tile * BM + row, n = n_tile * BN + row;
                a_off[i] = m * p.HW;
                b_off[i] = n * p.HW;
                if (m < p.M_total) a_mask |= 1u << i;
                if (row < BN && n < p.N_total) b_mask |= 1u << i;
            }
            img = split * p.imgs_per_split;
            img_end = min(p.n_img, img + p.imgs_per_split);
            if (KS != 1) {
                // every producer has issued the copies of the previous tile before the table changes
                producers_sync();
                if (tid < BM) {
                    const int n = n_tile * BN + tid;
                    int2 e = make_int2(-1, 0);
                    if (tid < BN && n < p.N_total) {
                        // unfolded row n = (channel, kh, kw)
                        const int kk = taps(p), kw_n = kcols(p);
                        const int c = n / kk, t2 = n - c * kk, kh = t2 / kw_n, kw = t2 - kh * kw_n;
                        e.x = (c * p.g_H + kh * p.dilH) * p.g_W + kw * p.dilW;
                        e.y = (kh * p.dilH) | ((kw * p.dilW) << 16);
                    }
                    rowtab[tid] = e;
                }
                producers_sync();
                img2 = img;
                pix2 = lane;
                while (pix2 >= p.HW) { pix2 -= p.HW; ++img2; }
            }
            pix = (tid & 7) * 4;
            while (pix >= p.HW) { pix -= p.HW; ++img; }
        }
    }

    // Moves to the next k-block of this CTA's tile list.
    __device__ __forceinline__ void advance(const Params &p, int2 *rowtab)
    {
        if (++kb == p.kblocks) {
            const int t = tile + (int)gridDim.x;
            if (t < p.total_tiles) setup(p, t, rowtab);
            else tile = t;
        } else if (OP == OP_WGRAD) {
            pix += BK;
            while (pix >= p.HW) { pix -= p.HW; ++img; }
            if (KS != 1) {
                pix2 += BK;
                while (pix2 >= p.HW) { pix2 -= p.HW; ++img2; }
            }
        }
    }

    // Copies four consecutive pixels of one row, starting at this thread's (image, pixel), to shared memory.
    __device__ __forceinline__ void row_chunk(const Params &p, uint32_t dst, const float *base, int stride, bool vec, bool on) const
    {
        if (vec) {
            const bool ok = on && img < img_end;
            cp_async16(dst, ok ? base + (size_t)img * stride + pix : base, ok);
            return;
        }
        int ij = img, pj = pix;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            while (pj >= p.HW) { pj -= p.HW; ++ij; }
            const bool ok = on && ij < img_end;
            cp_async4(dst + 4 * j, ok ? base + (size_t)ij * stride + pj : base, ok);
            ++pj;
        }
    }

    // Issues the asynchronous copies of this thread's pieces of the current k-block into the raw tiles at
    // shared-memory addresses sa / sb (+ the piece offsets); masked pieces are zero-filled.
    __device__ __forceinline__ void issue(const Params &p, uint32_t sa, uint32_t sb, const uint32_t (&a_so)[2],
                                          const uint32_t (&b_so)[2], const bool (&b_store)[2], const uint32_t (&g_so)[2],
                                          const int2 *rowtab) const
    {
        const int tid = threadIdx.x, warp = tid >> 5;
        if (tile >= p.total_tiles) return;
        if (OP != OP_WGRAD) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int k = kb * BK + warp + 16 * i;
                const bool kok = k < p.Kd;
                if (KS != 1) {
                    const int kk = taps(p), kw_n = kcols(p);
                    const int c = k / kk, t2 = k - c * kk, kh = t2 / kw_n, kw = t2 - kh * kw_n;
                    const int koff = (c * p.g_H + kh * p.dilH) * p.g_W + kw * p.dilW;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool ok = kok && (tapmask[j] >> t2 & 1u);
                        cp_async4(sa + g_so[i] + MN_ATOM * j, ok ? p.a + (a_off[j] + koff) : p.a, ok);
                    }
                } else if (p.vec_a) {
                    const bool ok = kok && a_mask;
                    cp_async16(sa + a_so[i], ok ? p.a + a_off[0] + k * p.HW : p.a, ok);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool ok = kok && (a_mask >> j & 1u);
                        cp_async4(sa + a_so[i] + 4 * j, ok ? p.a + a_off[j] + k * p.HW : p.a, ok);
                    }
                }
            }
            if (OP == OP_FWD) {
                const int k0 = kb * BK + (tid & 7) * 4;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (!b_store[i]) continue;
                    const float *src = p.b + b_off[i] + kb * BK;
                    const bool rok = (b_mask >> i & 1u) != 0;
                    if (p.vec_b) {
                        const bool ok = rok && k0 < p.Kd;
                        cp_async16(sb + b_so[i], ok ? src : p.b, ok);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = rok && k0 + j < p.Kd;
                            cp_async4(sb + b_so[i] + 4 * j, ok ? src + j : p.b, ok);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int k = kb * BK + warp + 16 * i;
                    const bool kok = k < p.Kd;
                    if (KS != 1) {
                        // B[c][(ko, kh, kw)] = W[ko][c][kH-1-kh][kW-1-kw]: the tap index runs backwards
                        const int kk = taps(p);
                        const int ko = k / kk, t2 = k - ko * kk;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = kok && (b_mask >> j & 1u);
                            cp_async4(sb + g_so[i] + MN_ATOM * j, ok ? p.b + ((size_t)(ko * p.N_total + b_off[0] + 32 * j) * kk + (kk - 1 - t2)) : p.b, ok);
                        }
                        continue;
                    }
                    if (!b_store[i]) continue;
                    const float *src = p.b + (size_t)(kok ? k : 0) * p.N_total + b_off[0];
                    if (p.vec_b) {
                        const bool ok = kok && b_mask;
                        cp_async16(sb + b_so[i], ok ? src : p.b, ok);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = kok && (b_mask >> j & 1u);
                            cp_async4(sb + b_so[i] + 4 * j, ok ? src + j : p.b, ok);
                        }
                    }
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                row_chunk(p, sa + a_so[i], p.a + a_off[i], p.M_total * p.HW, p.vec_a != 0, (a_mask >> i & 1u) != 0);
                if (KS == 1 && b_store[i]) row_chunk(p, sb + b_so[i], p.b + b_off[i], p.N_total * p.HW, p.vec_b != 0, (b_mask >> i & 1u) != 0);
            }
            if (KS != 1) {
                // unfolded operand: this lane owns column k = lane (one output pixel) of rows warp, warp + 16, ...:
                // x[img][c][oh * dH - padH + kh * dilH][ow * dW - padW + kw * dilW]; one copy instruction of the warp
                // fills the 128 bytes of one tile row
                const int lane = tid & 31;
                const int oh = pix2 / p.pix_W, ow = pix2 - oh * p.pix_W;
                const int ih = oh * p.dH - p.padH, iw = ow * p.dW - p.padW;
                const bool pix_ok = img2 < img_end;
                const float *img_base = p.b + (size_t)(pix_ok ? img2 : 0) * p.g_C * p.g_H * p.g_W + (ih * p.g_W + iw);
                const uint32_t dst0 = sb + (uint32_t)(warp * 128 + (((lane >> 2) ^ (warp & 7)) << 4) + (lane & 3) * 4);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int row = warp + 16 * q;
                    if (row >= BN) break;
                    const int2 e = rowtab[row];
                    const bool ok = pix_ok && e.x >= 0 && (unsigned)(ih + (e.y & 0xffff)) < (unsigned)p.g_H &&
                                    (unsigned)(iw + (e.y >> 16)) < (unsigned)p.g_W;
                    cp_async4(dst0 + (uint32_t)q * 2048u, ok ? img_base + e.x : p.b, ok);
                }
            }
        }
    }
};

template <int OP, int BN, int KS>
__global__ void __launch_bounds__(THREADS, 1)
pw_gemm_kernel(const Params p)
{
    constexpr bool A_MN = OP != OP_WGRAD;     // A is M-major (forward, input gradient)
    constexpr bool B_MN = OP == OP_DGRAD;     // B is N-major (input gradient)
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t idesc = idesc_of(BN, A_MN, B_MN);

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[RAW_STAGES + 2]; // MMAs-of-this-stage-done barriers, then one accumulators-ready barrier per set
    __shared__ uint64_t full[RAW_STAGES];     // stage split and visible to the tensor core: one arrival per producer warp
    __shared__ uint64_t accfree[2];           // accumulator set drained: one arrival per epilogue warp
    __shared__ uint32_t tmem_base_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < RAW_STAGES + 2; ++s) mbar_init(smem_u32(bars + s), 1);
        for (int s = 0; s < RAW_STAGES; ++s) mbar_init(smem_u32(full + s), PRODUCERS / 32);
        for (int s = 0; s < 2; ++s) mbar_init(smem_u32(accfree + s), EPILOGUE_WARPS);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    const int KB = p.kblocks;
    const int my_tiles = ((int)blockIdx.x < p.total_tiles) ? (p.total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total_it = my_tiles * KB;
    const int nhi_used = KB < p.nacc - 1 ? KB : p.nacc - 1;   // hi accumulators that received a k-block; the lo one always did
    const uint32_t set_cols = (uint32_t)(p.nacc * ACC_COLS);

    // shared-memory offsets of this thread's pieces (same for every stage)
    uint32_t a_so[2], b_so[2], g_so[2];
    bool b_store[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int k = warp + 16 * i;                    // M/N-major: k inside the block
        const int row = (tid >> 3) + 64 * i;            // K-major: tile row
        // 128-byte rows of 32 consecutive M/N values, four k rows per 512-byte atom, the 32-byte chunk index
        // XORed with the row index (the tensor core's 128B-base-32B swizzle, the only M/N-major form for tf32)
        const uint32_t mn = (uint32_t)((lane >> 3) * MN_ATOM + (k >> 2) * MN_KATOM + (k & 3) * 128 +
                                       ((((lane & 7) >> 1) ^ (k & 3)) << 5) + ((lane & 1) << 4));
        const uint32_t km = piece_offset(row, tid & 7);   // K-major: 128-byte swizzle
        a_so[i] = A_MN ? mn : km;
        b_so[i] = B_MN ? mn : km;
        b_store[i] = B_MN ? (lane * 4 < BN) : (row < BN);
        if (OP == OP_WGRAD && KS != 1) {
            // gathered K-major operand: warp w copies rows w, w + 16, ... element by element, so it also splits them:
            // this lane takes chunks (lane & 3) * 2 + i of row w + 16 * (lane >> 2)
            const int grow = warp + 16 * (lane >> 2);
            b_so[i] = piece_offset(grow, (lane & 3) * 2 + i);
            b_store[i] = grow < BN;
        }
        // gathered M/N-major operand (KS != 1): this lane copies element (row = lane + 32 j, k), 4 bytes each; j adds
        // one 512-byte atom.  The 32 lanes of one copy instruction fill one 128-byte row of an atom.
        g_so[i] = (uint32_t)((k >> 2) * MN_KATOM + (k & 3) * 128 + (((lane >> 3) ^ (k & 3)) << 5) + (((lane >> 2) & 1) << 4) + (lane & 3) * 4);
    }

    float bsum[2] = {0.f, 0.f};                         // WGRAD: running row sums of gy (bias gradient)
    unsigned char *const lo_base = smem + (size_t)RAW_STAGES * 2 * TILE;
    // Splits this thread's own pieces of raw stage `rs` (its copies have landed): the raw tile is the hi tile,
    // lo goes to the same offset of lo buffer `lb`.
    auto split_block = [&](int rs, int lb) {
        unsigned char *a_hi = smem + (size_t)rs * 2 * TILE, *b_hi = a_hi + TILE;
        unsigned char *a_lo = lo_base + (size_t)lb * 2 * TILE, *b_lo = a_lo + TILE;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 va = *reinterpret_cast<const float4 *>(a_hi + a_so[i]);
            store_lo_at(a_lo, a_so[i], va);
            if (OP == OP_WGRAD) bsum[i] += (va.x + va.y) + (va.z + va.w);
            if (b_store[i]) {
                const float4 vb = *reinterpret_cast<const float4 *>(b_hi + b_so[i]);
                store_lo_at(b_lo, b_so[i], vb);
            }
        }
    };
    // hi*hi products go to accumulator d_hi, the two small cross terms to d_lo: the tensor core truncates when it
    // accumulates, and the error of a chain scales with the magnitude it carries, so the large terms get the short
    // chains (k-blocks round-robin over nacc - 1 accumulators) and all cross terms share one.
    // Epilogue warps: reads the accumulators of tile `t` (the `count`-th tile of this CTA), writes the warp's 32
    // rows of the output and hands the accumulator set back to the MMA warp.
    auto epilogue = [&](int t, int count) -> bool {
        const int set = (p.sets == 2) ? (count & 1) : 0;
        const uint32_t parity = (uint32_t)(((p.sets == 2) ? (count >> 1) : count) & 1);
        if (!mbar_wait(smem_u32(bars + RAW_STAGES + set), parity, p.status)) return false;
        tc_fence_after();
        const int quarter = warp & 3;                            // the TMEM lanes this warp may read
        const int row = quarter * 32 + lane;
        int m, n_tile0;
        size_t dst_off = 0;
        if (OP != OP_WGRAD) {
            const int m_tile = t / p.n_tiles, n_tile = t - m_tile * p.n_tiles;
            m = m_tile * BM + row;
            n_tile0 = n_tile * BN;
            if (m < p.M_total) {
                const int im = m / p.HW;
                dst_off = (size_t)im * p.N_total * p.HW + (m - im * p.HW) + (size_t)n_tile0 * p.HW;
            }
        } else {
            const int split = t / p.tiles_per_split, r2 = t - split * p.tiles_per_split;
            const int m_tile = r2 / p.n_tiles, n_tile = r2 - m_tile * p.n_tiles;
            m = m_tile * BM + row;
            n_tile0 = n_tile * BN;
            dst_off = ((size_t)split * p.M_total + m) * p.N_total + n_tile0;
        }
        if (OP != OP_WGRAD) {
            // Whole tile inside the problem and planes long enough: stage 64 columns x 128 pixels in shared memory
            // ([column][pixel], so a column is 512 contiguous bytes of one output plane) and let the TMA unit write
            // each column as one bulk store (two when the tile crosses into the next image).
            const int m_tile0 = (t / p.n_tiles) * BM;
            if (p.bulk_out && m_tile0 + BM <= p.M_total) {
                float *stage = reinterpret_cast<float *>(smem + (size_t)(RAW_STAGES + LO_BUFS) * 2 * TILE);
                const int e = tid - (PRODUCERS + 32);            // 0 .. 127
                const int im0 = m_tile0 / p.HW, pix0 = m_tile0 - im0 * p.HW;
                const int len0 = min(BM, p.HW - pix0);
#pragma unroll 1
                for (int cbase = 0; cbase < BN; cbase += STAGE_COLS) {
                    bulk_wait_read_all();                        // this thread's earlier bulk stores have left the buffer
                    epilogue_sync();
#pragma unroll 1
                    for (int c0 = cbase; c0 < cbase + STAGE_COLS && c0 < BN; c0 += 16) {
                        float acc[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
                        for (int a2 = 0; a2 <= nhi_used; ++a2) {
                            const int a = a2 < nhi_used ? a2 : p.nacc - 1;
                            uint32_t r[16];
                            tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)set * set_cols + (uint32_t)(a * ACC_COLS + c0), r);
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r[j]);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) stage[(c0 - cbase + j) * BM + row] = acc[j];
                    }
                    fence_async_smem();                          // staged values -> visible to the bulk copy engine
                    epilogue_sync();
                    const int col = cbase + e, n = n_tile0 + col;
                    if (e < STAGE_COLS && col < BN && n < p.N_total) {
                        const uint32_t src = smem_u32(stage + e * BM);
                        float *dst = p.out + ((size_t)im0 * p.N_total + n) * p.HW + pix0;
                        bulk_s2g_nocommit(dst, src, (uint32_t)len0 * 4u);
                        if (len0 < BM) bulk_s2g_nocommit(p.out + ((size_t)(im0 + 1) * p.N_total + n) * p.HW, src + (uint32_t)len0 * 4u, (uint32_t)(BM - len0) * 4u);
                        bulk_commit();
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(accfree + set));
                return true;
            }
        }
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {                    // 16 columns at a time keeps the register count down
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)                         // the bias loads are in flight while TMEM is read
                acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
            for (int a2 = 0; a2 <= nhi_used; ++a2) {
                const int a = a2 < nhi_used ? a2 : p.nacc - 1;
                uint32_t r[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)set * set_cols + (uint32_t)(a * ACC_COLS + c0), r);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r[j]);
            }
            if (m < p.M_total) {
                const int n0 = n_tile0 + c0;
                if (OP != OP_WGRAD) {
                    float *dst = p.out + dst_off + (size_t)c0 * p.HW;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (n0 + j < p.N_total) dst[(size_t)j * p.HW] = acc[j];
                    }
                } else {
                    float *dst = p.out + dst_off + c0;
                    if ((p.N_total & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            if (n0 + j < p.N_total) *reinterpret_cast<float4 *>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + j < p.N_total) dst[j] = acc[j];
                    }
                }
            }
        }
        tc_fence_before();                                       // the TMEM reads above are ordered before the arrival
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(accfree + set));
        return true;
    };

    bool ok = true;
    if (warp == PRODUCERS / 32) {
        // ---- MMA warp: waits for a split stage, issues its twelve MMAs, commits them to the stage's barrier.  The tensor
        // pipe takes one of these MMAs every 64 clocks only if the issuing thread keeps up: every instruction between two
        // tcgen05.mma of this one thread is time the pipe idles.  So one lane runs the whole loop, descriptors are a
        // constant upper word + a lower word that advances by additions, ring positions and barrier parities are carried
        // incrementally, and the steady state uses the form without a predicate. ----
        if (lane == 0) {
            constexpr uint32_t A_LOW = A_MN ? ((uint32_t)(MN_ATOM >> 4) << 16) : (1u << 16);
            constexpr uint32_t B_LOW = B_MN ? ((uint32_t)(MN_ATOM >> 4) << 16) : (1u << 16);
            constexpr uint32_t A_HIGH = (A_MN ? (uint32_t)(MN_KATOM >> 4) : (uint32_t)(SBO >> 4)) | (1u << 14) | ((A_MN ? 1u : 2u) << 29);
            constexpr uint32_t B_HIGH = (B_MN ? (uint32_t)(MN_KATOM >> 4) : (uint32_t)(SBO >> 4)) | (1u << 14) | ((B_MN ? 1u : 2u) << 29);
            constexpr uint32_t A_STEP = A_MN ? (uint32_t)(2 * MN_KATOM >> 4) : 2u;     // 8 k values further, in 16-byte units
            constexpr uint32_t B_STEP = B_MN ? (uint32_t)(2 * MN_KATOM >> 4) : 2u;
            constexpr uint32_t STAGE_STEP = (uint32_t)(2 * TILE >> 4);
            const uint32_t raw0 = (smem_u32(smem) >> 4) & 0x3fffu, lo0 = (smem_u32(lo_base) >> 4) & 0x3fffu;
            auto desc = [](uint32_t low, uint32_t high) { return ((uint64_t)high << 32) | low; };
            const int nhi = p.nacc - 1;
            int rs = 0, lb = 0, kb = 0, set = 0, hi_slot = 0;
            uint32_t full_parity = 0, free_parity = 0;             // accfree is first awaited on the second use of a set (its phase 0)
            bool first_round = true;
            uint32_t acc0 = tmem_base;
            for (int i = 0; i < total_it; ++i) {
                if (!mbar_wait(smem_u32(full + rs), full_parity, p.status)) break;
                if (kb == 0 && !first_round) {
                    // the epilogue warps must have drained the tile that used this accumulator set before
                    if (!mbar_wait(smem_u32(accfree + set), free_parity, p.status)) break;
                }
                tc_fence_after();
                const uint32_t d_hi = acc0 + (uint32_t)(hi_slot * ACC_COLS), d_lo = acc0 + (uint32_t)(nhi * ACC_COLS);
                const uint32_t ah = (raw0 + (uint32_t)rs * STAGE_STEP) | A_LOW, bh = (raw0 + (uint32_t)rs * STAGE_STEP + (uint32_t)(TILE >> 4)) | B_LOW;
                const uint32_t al = (lo0 + (uint32_t)lb * STAGE_STEP) | A_LOW, bl = (lo0 + (uint32_t)lb * STAGE_STEP + (uint32_t)(TILE >> 4)) | B_LOW;
                if (kb < nhi || kb == 0) {
                    // first k-blocks of a tile: the first MMA into an accumulator overwrites it
                    const uint32_t keep_lo = kb == 0 ? 0u : 1u, keep_hi = kb < nhi ? 0u : 1u;
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        umma_tf32(d_lo, desc(al + j * A_STEP, A_HIGH), desc(bh + j * B_STEP, B_HIGH), idesc, j == 0 ? keep_lo : 1u);
                        umma_tf32(d_lo, desc(ah + j * A_STEP, A_HIGH), desc(bl + j * B_STEP, B_HIGH), idesc, 1u);
                        umma_tf32(d_hi, desc(ah + j * A_STEP, A_HIGH), desc(bh + j * B_STEP, B_HIGH), idesc, j == 0 ? keep_hi : 1u);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        umma_tf32_acc(d_lo, desc(al + j * A_STEP, A_HIGH), desc(bh + j * B_STEP, B_HIGH), idesc);
                        umma_tf32_acc(d_lo, desc(ah + j * A_STEP, A_HIGH), desc(bl + j * B_STEP, B_HIGH), idesc);
                        umma_tf32_acc(d_hi, desc(ah + j * A_STEP, A_HIGH), desc(bh + j * B_STEP, B_HIGH), idesc);
                    }
                }
                umma_commit(smem_u32(bars + rs));
                if (++rs == RAW_STAGES) { rs = 0; full_parity ^= 1u; }
                if (++lb == LO_BUFS) lb = 0;
                if (++hi_slot == nhi) hi_slot = 0;
                if (++kb == KB) {
                    umma_commit(smem_u32(bars + RAW_STAGES + set));
                    kb = 0;
                    hi_slot = 0;
                    acc0 += set_cols;
                    if (++set == p.sets) { set = 0; acc0 = tmem_base; if (!first_round) free_parity ^= 1u; first_round = false; }
                }
            }
        }
    } else if (warp > PRODUCERS / 32) {
        // ---- epilogue warps: one pass over this CTA's tiles ----
        for (int count = 0; count < my_tiles; ++count) {
            if (!epilogue((int)blockIdx.x + count * (int)gridDim.x, count)) { ok = false; break; }
        }
        bulk_wait_read_all();                                    // shared memory must outlive the last bulk stores' reads
    } else {
        Loader<OP, BN, KS> L;
        L.tile = (int)blockIdx.x;
        L.kb = 0;
        int2 *rowtab = reinterpret_cast<int2 *>(smem + (size_t)(RAW_STAGES + LO_BUFS) * 2 * TILE);   // in the output staging area, which the weight gradient does not use
        if (my_tiles > 0) L.setup(p, L.tile, rowtab);
        const uint32_t smem_a0 = smem_u32(smem);
        // copies of the first PREFETCH k-blocks; one commit group per k-block, empty ones included, so that
        // "all but the newest PREFETCH - 1 groups" always means "k-block i has landed"
    #pragma unroll
        for (int i = 0; i < PREFETCH; ++i) {
            if (i < total_it) {
                L.issue(p, smem_a0 + (uint32_t)(i * 2 * TILE), smem_a0 + (uint32_t)(i * 2 * TILE + TILE), a_so, b_so, b_store, g_so, rowtab);
                L.advance(p, rowtab);
            }
            cp_async_commit();
        }

        int c_tile = (int)blockIdx.x, c_kb = 0;                // tile and k-block of the block being split
        for (int i = 0; i < total_it; ++i) {
            const int rs = i % RAW_STAGES, lb = i % LO_BUFS;
            cp_async_wait<PREFETCH - 1>();                     // this thread's pieces of k-block i are in shared memory
            if (i >= LO_BUFS) {
                // the MMAs of k-block i - 2 read this lo buffer
                const int j = i - LO_BUFS;
                if (!mbar_wait(smem_u32(bars + j % RAW_STAGES), (uint32_t)((j / RAW_STAGES) & 1), p.status)) { ok = false; break; }
            }
            if (KS != 1) __syncwarp();                         // gathered pieces were filled by several lanes of this warp
            split_block(rs, lb);
            fence_async_smem();                                // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(full + rs));
            // refill the raw stage that k-block i - 1 used with k-block i + PREFETCH, once its MMAs have read it
            if (i + PREFETCH < total_it) {
                if (i >= 1) {
                    const int j = i - 1;
                    if (!mbar_wait(smem_u32(bars + j % RAW_STAGES), (uint32_t)((j / RAW_STAGES) & 1), p.status)) { ok = false; break; }
                }
                const int ns = (i + PREFETCH) % RAW_STAGES;
                L.issue(p, smem_a0 + (uint32_t)(ns * 2 * TILE), smem_a0 + (uint32_t)(ns * 2 * TILE + TILE), a_so, b_so, b_store, g_so, rowtab);
                L.advance(p, rowtab);
            }
            cp_async_commit();
            if (c_kb == KB - 1) {
                if (OP == OP_WGRAD) {
                    // bias gradient: the eight chunk lanes of a row hold its partial sums
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        float sum = bsum[r];
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                        const int split = c_tile / p.tiles_per_split, r2 = c_tile - split * p.tiles_per_split;
                        const int m_tile = r2 / p.n_tiles, n_tile = r2 - m_tile * p.n_tiles;
                        const int m = m_tile * BM + (tid >> 3) + 64 * r;
                        if (p.bias_part && n_tile == 0 && (tid & 7) == 0 && m < p.M_total) p.bias_part[(size_t)m * p.splits + split] = sum;
                        bsum[r] = 0.f;
                    }
                }
                c_kb = 0;
                c_tile += (int)gridDim.x;
            } else {
                ++c_kb;
            }
        }
        cp_async_wait<0>();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace pw

#include "pw_tma.cuh"

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

typedef void (*GemmKernel)(const GemmParams);

template <int OP, int KS>
static GemmKernel pick_bn(int bn)
{
    switch (bn) {
        case 32: return conv_gemm_kernel<OP, KS, 32>;
        case 64: return conv_gemm_kernel<OP, KS, 64>;
        case 128: return conv_gemm_kernel<OP, KS, 128>;
        default: return conv_gemm_kernel<OP, KS, 256>;
    }
}
template <int OP>
static GemmKernel pick_kernel(int ks, int bn)
{
    if (ks == 1) return pick_bn<OP, 1>(bn);
    if (ks == 3) return pick_bn<OP, 3>(bn);
    return pick_bn<OP, 0>(bn);
}

static size_t smem_bytes(int bn)
{
    const size_t stage = 2 * ((size_t)BM * BK * 4 + (size_t)bn * BK * 4);
    const int stages = (stage * 4 <= 200 * 1024) ? 4 : (stage * 3 <= 200 * 1024 ? 3 : 2);
    return stage * stages + 1024;   // + alignment slack
}

static int pick_bn_for(int n_total)
{
    if (n_total <= 32) return 32;
    if (n_total <= 64) return 64;
    if (n_total <= 128 || n_total % 256 != 0) return 128;
    return 128;
}

static int launch(GemmKernel kern, const GemmParams &p, dim3 grid, int bn, cudaStream_t stream)
{
    const size_t smem = smem_bytes(bn);
    CUNN_CUDA(cudaFuncSetAttribute((const void *)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    void *args[] = {(void *)&p};
    CUNN_CUDA(cudaLaunchKernel((const void *)kern, grid, dim3(THREADS), args, smem, stream));
    return 0;
}

static int check(int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, int *oH, int *oW,
                 int dilH = 1, int dilW = 1)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(dilW > 0 && dilH > 0, "dilation should be greater than zero, but got dilationH: %d, dilationW: %d", dilH, dilW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && K > 0 && H > 0 && W > 0 && padH >= 0 && padW >= 0, "bad convolution sizes");
    const int spanH = dilH * (kH - 1) + 1, spanW = dilW * (kW - 1) + 1;   // extent of the dilated kernel
    CUNN_CHECK_ARG(spanH < (1 << 15) && spanW < (1 << 15), "dilated kernel extent too large");
    *oH = (H + 2 * padH - spanH) / dH + 1;
    *oW = (W + 2 * padW - spanW) / dW + 1;
    CUNN_CHECK_ARG(H + 2 * padH >= spanH && W + 2 * padW >= spanW && *oH >= 1 && *oW >= 1,
                   "Given input size: (%d x %d x %d). Calculated output size: (%d x %d x %d). Output size is too small", C, H,
                   W, K, *oH, *oW);
    CUNN_CHECK_ARG((long long)N * C * (long long)H * W < (1LL << 31) && (long long)N * K * (long long)(*oH) * (*oW) < (1LL << 31) &&
                       (long long)C * kH * kW < (1 << 24),
                   "tensors of 2^31 or more elements are not supported");
    return 0;
}

static int ks_of(int kH, int kW) { return (kH == 1 && kW == 1) ? 1 : (kH == 3 && kW == 3) ? 3 : 0; }

static void wgrad_plan(int N, int C, int K, int kk, int oHW, int *bn, int *splits, int *imgs_per_split, int *pix_blocks)
{
    *bn = pick_bn_for(C * kk);
    const int tiles = ceil_div(K, BM) * ceil_div(C * kk, *bn);
    int s = std::max(1, std::min(N, (2 * sm_count()) / std::max(1, tiles)));
    *imgs_per_split = ceil_div(N, s);
    *splits = ceil_div(N, *imgs_per_split);
    *pix_blocks = ceil_div(oHW, BK);
}


// ---- pointwise path ----------------------------------------------------------------------------------
static bool pw_applies(int kH, int kW, int dH, int dW, int padH, int padW)
{
    return kH == 1 && kW == 1 && dH == 1 && dW == 1 && padH == 0 && padW == 0;
}
static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

typedef void (*PwKernel)(const pw::Params);
template <int OP, int KS>
static PwKernel pw_pick_bn(int bn)
{
    switch (bn) {
        case 32: return pw::pw_gemm_kernel<OP, 32, KS>;
        case 64: return pw::pw_gemm_kernel<OP, 64, KS>;
        default: return pw::pw_gemm_kernel<OP, 128, KS>;
    }
}
template <int OP>
static PwKernel pw_pick(int bn, int ks = 1)
{
    if (ks == 1) return pw_pick_bn<OP, 1>(bn);
    if (ks == 3) return pw_pick_bn<OP, 3>(bn);
    return pw_pick_bn<OP, 0>(bn);
}
// Kernels of up to 32 taps run on the same persistent kernel with a gathering loader.
static bool gather_applies(int kH, int kW) { return kH * kW <= 32; }
// loader variant of the gathering path: 3x3 has its own instantiation, everything else (a strided or padded 1x1
// included) the one with run-time kernel sizes
static int gather_ks(int kH, int kW) { return (kH == 3 && kW == 3) ? 3 : 0; }
static void set_geometry(pw::Params &q, int gC, int gH, int gW, int kH, int kW, int dH, int dW, int padH, int padW, int pixW,
                         int dilH, int dilW)
{
    q.g_C = gC; q.g_H = gH; q.g_W = gW; q.kH = kH; q.kW = kW; q.dH = dH; q.dW = dW; q.padH = padH; q.padW = padW; q.pix_W = pixW;
    q.dilH = dilH; q.dilW = dilW;
}
static int pw_bn_for(int n_total) { return n_total <= 32 ? 32 : (n_total <= 64 ? 64 : 128); }

// Accumulators per tile and accumulator sets: the hi*hi products of the k-blocks are dealt round-robin to `nacc - 1`
// accumulators to keep the tensor core's truncating accumulation chains short, the cross terms share the last one; two sets (epilogue overlapped with the next tile) when
// they fit in the 512 TMEM columns.
static void pw_accumulators(int bn, int kblocks, int *nacc, int *sets, bool wgrad = false)
{
    if (bn == 128 && wgrad) {
        // sums over pixels of random-sign products cancel: the weight gradient is the pass most sensitive to the
        // accumulation chains, and its long k loops make the epilogue a small share anyway
        if (kblocks <= 8) { *nacc = 2; *sets = 2; }
        else { *nacc = 4; *sets = 1; }
    } else if (bn == 128) {
        // two sets let the MMAs of the next tile run while the epilogue warps drain this one; beyond 16 k-blocks the
        // chains (12 MMAs per k-block and accumulator) get long enough to need four accumulators for the 1e-4 bar
        if (kblocks <= 16) { *nacc = 2; *sets = 2; }
        else { *nacc = 4; *sets = 1; }
    } else if (bn == 64) {
        if (kblocks <= 48) { *nacc = 4; *sets = 2; }
        else { *nacc = 8; *sets = 1; }
    } else {
        *nacc = 8; *sets = 2;
    }
}

static int pw_launch(PwKernel kern, pw::Params &p, cudaStream_t stream)
{
    const int grid = std::min(p.total_tiles, sm_count());
    CUNN_CUDA(cudaFuncSetAttribute((const void *)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pw::SMEM));
    void *args[] = {(void *)&p};
    CUNN_CUDA(cudaLaunchKernel((const void *)kern, dim3(grid), dim3(pw::THREADS), args, pw::SMEM, stream));
    return 0;
}

// ---- tensor-map kernels (pw_tma.cuh) -----------------------------------------------------------------------------
static int g_use_tma = 1;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// The driver's encoder, looked up through the runtime so that the library does not link libcuda.
static EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return (EncodeTiledFn)ptr;
    }();
    return fn;
}
// fp32 tensor [d2][d1][d0] (d0 contiguous; d2 = 0: two dimensions), boxes of box0 x box1 (x 1), zero fill outside.
static int make_map(CUtensorMap *m, const float *base, long long d0, long long d1, long long d2, int box0, int box1, CUtensorMapSwizzle swz)
{
    const cuuint32_t rank = d2 ? 3 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)(d2 ? d2 : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)d0 * 4, (cuuint64_t)d0 * (cuuint64_t)d1 * 4};
    cuuint32_t box[3] = {(cuuint32_t)box0, (cuuint32_t)box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}
static bool tma_applies(const void *a, const void *b, const void *c, int HW, int C)
{
    return g_use_tma && HW % 4 == 0 && C % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(c) && encode_tiled() != nullptr;
}
// Accumulator plan of the tensor-map kernels: tiles of one or two k-blocks put all products into one accumulator and
// use up to four accumulator sets, so that the MMA warp runs several tiles ahead of the epilogue warps; longer tiles
// follow pw_accumulators.
static void tma_accumulators(int bn, int kblocks, int *nacc, int *sets, bool wgrad = false)
{
    const int cols = std::max(bn, 32);
    if (kblocks <= 2) {
        *nacc = 1;
        *sets = std::min((int)pwt::MAX_SETS, 512 / cols);
        return;
    }
    pw_accumulators(bn, kblocks, nacc, sets, wgrad);
}
typedef void (*PwTmaKernel)(const pw::Params, const CUtensorMap, const CUtensorMap, const CUtensorMap);
// 4 splitter + 8 epilogue warps for every tile length: measured against 8 + 4 and 16 + 4 on tiles of 8, 16 and 32 k-blocks,
// 4 + 8 was never slower (16 + 4 runs at 80 registers and was 4-14 % slower).
template <int OP>
static PwTmaKernel pw_tma_pick(int bn)
{
    switch (bn) {
        case 32: return pwt::pw_tma_kernel<OP, 32, 4, 8, 4, 2>;
        case 64: return pwt::pw_tma_kernel<OP, 64, 4, 8, 4, 2>;
        default: return pwt::pw_tma_kernel<OP, 128, 4, 8, 4, 2>;
    }
}
// `mo` is the map of the output tensor for the bulk-store epilogue (forward / input gradient); kernels that do not use
// it get a copy of `ma`.
static int pw_tma_launch(PwTmaKernel kern, pw::Params &p, CUtensorMap &ma, CUtensorMap &mb, CUtensorMap &mo, cudaStream_t stream)
{
    const int grid = std::min(p.total_tiles, sm_count());
    const size_t smem_bytes = pw::SMEM;
    const int threads = pwt::tma_threads(4, 8);          // every configuration has 14 warps
    CUNN_CUDA(cudaFuncSetAttribute((const void *)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    void *args[] = {(void *)&p, (void *)&ma, (void *)&mb, (void *)&mo};
    CUNN_CUDA(cudaLaunchKernel((const void *)kern, dim3(grid), dim3(threads), args, smem_bytes, stream));
    return 0;
}

// Splits of the image range for the weight gradient on the persistent kernel: every tile takes `imgs_per_split`
// images.  Candidates are scored by (waves of the persistent grid) x (images per tile) — the time of the slowest
// CTA — and tiles longer than ~128 k-blocks are avoided when a shorter choice exists (accumulation chains).
static void pw_wgrad_plan(int N, int C, int K, int HW, int *bn, int *splits, int *imgs_per_split)
{
    *bn = pw_bn_for(C);
    const long long tiles_mn = (long long)ceil_div(K, BM) * ceil_div(C, *bn);
    const int grid = sm_count();
    const long long kb_per_img = ceil_div_ll(HW, BK);
    int best_ips = 1;
    double best = -1.0;
    for (int ips = 1; ips <= N; ++ips) {
        const long long tiles = tiles_mn * ceil_div(N, ips);
        const long long waves = ceil_div_ll(tiles, grid);
        // in k-blocks: the tile's own loop + about six more for its prologue, its 64 KB of partial sums and their
        // share of the final reduction
        double cost = (double)waves * ((double)ips * kb_per_img + 6.0);
        if (ips > 1 && (long long)ips * kb_per_img > 128) cost *= 1.0 + 0.25 * (double)((long long)ips * kb_per_img - 128) / 128.0;
        if (best < 0.0 || cost < best * 0.999) { best = cost; best_ips = ips; }
    }
    *imgs_per_split = best_ips;
    *splits = ceil_div(N, best_ips);
}

}  // namespace mm
}  // namespace cunn

using namespace cunn;
using namespace cunn::mm;

static int conv_forward(const float *x, const float *weight, const float *bias, float *y, int N, int C, int H, int W, int K,
                        int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW, dilH, dilW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    const bool dilated = dilH != 1 || dilW != 1;
    CUNN_CHECK_ARG(!dilated || gather_applies(kH, kW), "dilated kernels of more than 32 taps are not supported");
    if (!dilated && stem::applies(C, K, kH, kW)) return stem::forward(x, weight, bias, y, N, H, W, oH, oW, dH, dW, padH, padW, stream);
    if (pw_applies(kH, kW, dH, dW, padH, padW)) {
        pw::Params q{};
        q.a = x; q.b = weight; q.bias = bias; q.out = y; q.status = device_status_ptr();
        q.HW = H * W; q.M_total = N * H * W; q.N_total = K; q.Kd = C; q.kblocks = ceil_div(C, BK);
        const int bn = pw_bn_for(K);
        q.n_tiles = ceil_div(K, bn); q.tiles_per_split = 0; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
        q.n_img = N; q.imgs_per_split = N; q.splits = 1;
        if (tma_applies(x, weight, y, q.HW, C)) {
            alignas(64) CUtensorMap ma, mb, mo;
            q.gpi = ceil_div(q.HW, 32); q.M_total = N * q.gpi * 32; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
            q.bulk_out = (q.HW % 32 == 0) && q.HW >= 8 * BM;
            tma_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
            if (make_map(&ma, x, q.HW, C, N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return 1;
            if (make_map(&mb, weight, C, K, 0, 32, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return 1;
            if (q.bulk_out) { if (make_map(&mo, y, q.HW, K, N, BM, pwt::HALF_STAGE_COLS, CU_TENSOR_MAP_SWIZZLE_NONE)) return 1; }
            else mo = ma;
            return pw_tma_launch(pw_tma_pick<OP_FWD>(bn), q, ma, mb, mo, stream);
        }
        q.vec_a = (q.HW % 4 == 0) && aligned16(x); q.vec_b = (C % 4 == 0) && aligned16(weight);
        q.bulk_out = (q.HW % 4 == 0) && q.HW >= 8 * BM && aligned16(y);
        pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
        return pw_launch(pw_pick<OP_FWD>(bn), q, stream);
    }
    if (gather_applies(kH, kW)) {
        pw::Params q{};
        q.a = x; q.b = weight; q.bias = bias; q.out = y; q.status = device_status_ptr();
        q.HW = oH * oW; q.M_total = N * oH * oW; q.N_total = K; q.Kd = C * kH * kW; q.kblocks = ceil_div(q.Kd, BK);
        set_geometry(q, C, H, W, kH, kW, dH, dW, padH, padW, oW, dilH, dilW);
        const int bn = pw_bn_for(K);
        q.n_tiles = ceil_div(K, bn); q.tiles_per_split = 0; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
        q.n_img = N; q.imgs_per_split = N; q.splits = 1;
        q.vec_a = 0; q.vec_b = (q.Kd % 4 == 0) && aligned16(weight);
        q.bulk_out = (q.HW % 4 == 0) && q.HW >= 8 * BM && aligned16(y);
        pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
        return pw_launch(pw_pick<OP_FWD>(bn, gather_ks(kH, kW)), q, stream);
    }
    GemmParams p{};
    p.a_src = x; p.b_src = weight; p.bias = bias; p.out = y; p.status = device_status_ptr();
    p.g_C = C; p.g_H = H; p.g_W = W; p.g_padH = padH; p.g_padW = padW; p.g_dH = dH; p.g_dW = dW; p.kH = kH; p.kW = kW;
    p.pix_W = oW; p.pix_HW = oH * oW; p.C = C; p.K = K; p.n_img = N;
    p.M_total = N * oH * oW; p.N_total = K; p.Kd = C * kH * kW; p.kblocks = ceil_div(p.Kd, BK); p.out_HW = oH * oW;
    const int bn = pick_bn_for(K);
    dim3 grid(ceil_div(p.M_total, BM), ceil_div(K, bn), 1);
    return launch(pick_kernel<OP_FWD>(ks_of(kH, kW), bn), p, grid, bn, stream);
}

static int conv_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H, int W, int K, int kH, int kW,
                           int dH, int dW, int padH, int padW, int dilH, int dilW, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW, dilH, dilW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    const bool dilated = dilH != 1 || dilW != 1;
    CUNN_CHECK_ARG(!dilated || gather_applies(kH, kW), "dilated kernels of more than 32 taps are not supported");
    if (pw_applies(kH, kW, dH, dW, padH, padW)) {
        pw::Params q{};
        q.a = gy; q.b = weight; q.bias = nullptr; q.out = gx; q.status = device_status_ptr();
        q.HW = H * W; q.M_total = N * H * W; q.N_total = C; q.Kd = K; q.kblocks = ceil_div(K, BK);
        const int bn = pw_bn_for(C);
        q.n_tiles = ceil_div(C, bn); q.tiles_per_split = 0; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
        q.n_img = N; q.imgs_per_split = N; q.splits = 1;
        if (tma_applies(gy, weight, gx, q.HW, C)) {
            alignas(64) CUtensorMap ma, mb, mo;
            q.gpi = ceil_div(q.HW, 32); q.M_total = N * q.gpi * 32; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
            q.bulk_out = (q.HW % 32 == 0) && q.HW >= 8 * BM;
            tma_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
            if (make_map(&ma, gy, q.HW, K, N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return 1;
            if (make_map(&mb, weight, C, K, 0, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return 1;
            if (q.bulk_out) { if (make_map(&mo, gx, q.HW, C, N, BM, pwt::HALF_STAGE_COLS, CU_TENSOR_MAP_SWIZZLE_NONE)) return 1; }
            else mo = ma;
            return pw_tma_launch(pw_tma_pick<OP_DGRAD>(bn), q, ma, mb, mo, stream);
        }
        q.vec_a = (q.HW % 4 == 0) && aligned16(gy); q.vec_b = (C % 4 == 0) && aligned16(weight);
        q.bulk_out = (q.HW % 4 == 0) && q.HW >= 8 * BM && aligned16(gx);
        pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
        return pw_launch(pw_pick<OP_DGRAD>(bn), q, stream);
    }
    if (dH == 1 && dW == 1 && padH <= dilH * (kH - 1) && padW <= dilW * (kW - 1) && (!dilated || gather_applies(kH, kW))) {
        // stride 1: a convolution of gy with the kernel rotated by 180 degrees and padding dil (k - 1) - pad
        if (gather_applies(kH, kW)) {
            pw::Params q{};
            q.a = gy; q.b = weight; q.bias = nullptr; q.out = gx; q.status = device_status_ptr();
            q.HW = H * W; q.M_total = N * H * W; q.N_total = C; q.Kd = K * kH * kW; q.kblocks = ceil_div(q.Kd, BK);
            set_geometry(q, K, oH, oW, kH, kW, 1, 1, dilH * (kH - 1) - padH, dilW * (kW - 1) - padW, W, dilH, dilW);
            const int bn = pw_bn_for(C);
            q.n_tiles = ceil_div(C, bn); q.tiles_per_split = 0; q.total_tiles = ceil_div(q.M_total, BM) * q.n_tiles;
            q.n_img = N; q.imgs_per_split = N; q.splits = 1;
            q.vec_a = 0; q.vec_b = 0;
            q.bulk_out = (q.HW % 4 == 0) && q.HW >= 8 * BM && aligned16(gx);
            pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets);
            return pw_launch(pw_pick<OP_DGRAD>(bn, gather_ks(kH, kW)), q, stream);
        }
        GemmParams p{};
        p.a_src = gy; p.b_src = weight; p.bias = nullptr; p.out = gx; p.status = device_status_ptr();
        p.g_C = K; p.g_H = oH; p.g_W = oW; p.g_padH = kH - 1 - padH; p.g_padW = kW - 1 - padW; p.g_dH = 1; p.g_dW = 1;
        p.kH = kH; p.kW = kW; p.pix_W = W; p.pix_HW = H * W; p.C = C; p.K = K; p.n_img = N;
        p.M_total = N * H * W; p.N_total = C; p.Kd = K * kH * kW; p.kblocks = ceil_div(p.Kd, BK); p.out_HW = H * W;
        const int bn = pick_bn_for(C);
        dim3 grid(ceil_div(p.M_total, BM), ceil_div(C, bn), 1);
        return launch(pick_kernel<OP_DGRAD>(ks_of(kH, kW), bn), p, grid, bn, stream);
    }
    const long long total = (long long)N * C * H * W;
    const int blocks = (int)std::max(1LL, std::min(ceil_div_ll(total, 256), (long long)sm_count() * 16));
    dgrad_gather_kernel<<<blocks, 256, 0, stream>>>(gy, weight, gx, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW, oH, oW, total);
    CUNN_LAUNCH_CHECK("convmm grad input (gather)");
    return 0;
}

static size_t conv_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                      int dilH, int dilW)
{
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW, dilH, dilW) || N == 0) return 0;
    const bool dilated = dilH != 1 || dilW != 1;
    if (!dilated && stem::applies(C, K, kH, kW)) return stem::wgrad_workspace_bytes();
    int bn, splits, ips, pb;
    if (pw_applies(kH, kW, dH, dW, padH, padW)) {
        pw_wgrad_plan(N, C, K, H * W, &bn, &splits, &ips);
        return (size_t)splits * K * C * sizeof(float) + (size_t)K * splits * sizeof(float) + 256;
    }
    if (gather_applies(kH, kW)) {
        pw_wgrad_plan(N, C * kH * kW, K, oH * oW, &bn, &splits, &ips);
        return (size_t)splits * K * C * kH * kW * sizeof(float) + (size_t)K * splits * sizeof(float) + 256;
    }
    wgrad_plan(N, C, K, kH * kW, oH * oW, &bn, &splits, &ips, &pb);
    const int chunks = std::max(1, std::min(N, ceil_div(sm_count() * 4, K)));
    return (size_t)splits * K * C * kH * kW * sizeof(float) + (size_t)K * chunks * sizeof(float) + 256;
}

static int conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias, int N, int C, int H, int W, int K,
                         int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, float scale, void *workspace,
                         size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW, dilH, dilW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    const bool dilated = dilH != 1 || dilW != 1;
    CUNN_CHECK_ARG(!dilated || gather_applies(kH, kW), "dilated kernels of more than 32 taps are not supported");
    const size_t need = conv_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW);
    CUNN_CHECK_ARG(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                   "convmm acc_grad needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                   workspace ? workspace_bytes : (size_t)0);
    int bn, splits, ips, pb;
    const int kk = kH * kW;
    if (!dilated && stem::applies(C, K, kH, kW)) {
        const int ctas = stem::wgrad_ctas();
        const long long n = (long long)K * C * kk;
        float *partial = (float *)workspace, *bias_part = partial + (size_t)ctas * n;
        if (stem::weight_grad_partials(x, gy, partial, grad_bias ? bias_part : nullptr, N, H, W, oH, oW, dH, dW, padH, padW, stream)) return 1;
        const int rblocks = (int)std::max(1LL, std::min(ceil_div_ll(n + K, 256), (long long)sm_count() * 8));
        wgrad_bias_reduce_kernel<<<rblocks, 256, 0, stream>>>(partial, grad_weight, n, ctas, scale, grad_bias ? bias_part : nullptr, grad_bias, K);
        CUNN_LAUNCH_CHECK("convmm acc grad reduce");
        return 0;
    }
    if (pw_applies(kH, kW, dH, dW, padH, padW)) {
        pw_wgrad_plan(N, C, K, H * W, &bn, &splits, &ips);
        const long long n = (long long)K * C;
        pw::Params q{};
        q.a = gy; q.b = x; q.bias = nullptr; q.out = (float *)workspace; q.status = device_status_ptr();
        q.bias_part = grad_bias ? (float *)workspace + (size_t)splits * n : nullptr;
        q.HW = H * W; q.M_total = K; q.N_total = C; q.Kd = 0;
        q.kblocks = (int)ceil_div_ll((long long)ips * q.HW, BK);
        q.n_tiles = ceil_div(C, bn); q.tiles_per_split = ceil_div(K, BM) * q.n_tiles; q.total_tiles = q.tiles_per_split * splits;
        q.n_img = N; q.imgs_per_split = ips; q.splits = splits;
        q.vec_a = (q.HW % 4 == 0) && aligned16(gy); q.vec_b = (q.HW % 4 == 0) && aligned16(x);
        if (tma_applies(gy, x, workspace, q.HW, 4)) {
            alignas(64) CUtensorMap ma, mb;
            q.gpi = ceil_div(q.HW, 32); q.kblocks = ips * q.gpi;
            tma_accumulators(bn, q.kblocks, &q.nacc, &q.sets, true);
            if (make_map(&ma, gy, q.HW, K, N, 32, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return 1;
            if (make_map(&mb, x, q.HW, C, N, 32, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return 1;
            if (pw_tma_launch(pw_tma_pick<OP_WGRAD>(bn), q, ma, mb, ma, stream)) return 1;
        } else {
        pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets, true);
        if (pw_launch(pw_pick<OP_WGRAD>(bn), q, stream)) return 1;
        }
        const int rblocks = (int)std::max(1LL, std::min(ceil_div_ll(n + K, 256), (long long)sm_count() * 8));
        wgrad_bias_reduce_kernel<<<rblocks, 256, 0, stream>>>((const float *)workspace, grad_weight, n, splits, scale, q.bias_part, grad_bias, K);
        CUNN_LAUNCH_CHECK("convmm acc grad reduce");
        return 0;
    }
    if (gather_applies(kH, kW)) {
        const int oHW = oH * oW;
        pw_wgrad_plan(N, C * kk, K, oHW, &bn, &splits, &ips);
        const long long n = (long long)K * C * kk;
        pw::Params q{};
        q.a = gy; q.b = x; q.bias = nullptr; q.out = (float *)workspace; q.status = device_status_ptr();
        q.bias_part = grad_bias ? (float *)workspace + (size_t)splits * n : nullptr;
        q.HW = oHW; q.M_total = K; q.N_total = C * kk; q.Kd = 0;
        q.kblocks = (int)ceil_div_ll((long long)ips * oHW, BK);
        set_geometry(q, C, H, W, kH, kW, dH, dW, padH, padW, oW, dilH, dilW);
        q.n_tiles = ceil_div(C * kk, bn); q.tiles_per_split = ceil_div(K, BM) * q.n_tiles; q.total_tiles = q.tiles_per_split * splits;
        q.n_img = N; q.imgs_per_split = ips; q.splits = splits;
        q.vec_a = (oHW % 4 == 0) && aligned16(gy); q.vec_b = 0;
        pw_accumulators(bn, q.kblocks, &q.nacc, &q.sets, true);
        if (pw_launch(pw_pick<OP_WGRAD>(bn, gather_ks(kH, kW)), q, stream)) return 1;
        const int rblocks = (int)std::max(1LL, std::min(ceil_div_ll(n + K, 256), (long long)sm_count() * 8));
        wgrad_bias_reduce_kernel<<<rblocks, 256, 0, stream>>>((const float *)workspace, grad_weight, n, splits, scale, q.bias_part, grad_bias, K);
        CUNN_LAUNCH_CHECK("convmm acc grad reduce");
        return 0;
    }
    wgrad_plan(N, C, K, kk, oH * oW, &bn, &splits, &ips, &pb);
    GemmParams p{};
    p.a_src = gy; p.b_src = x; p.bias = nullptr; p.out = (float *)workspace; p.status = device_status_ptr();
    p.g_C = C; p.g_H = H; p.g_W = W; p.g_padH = padH; p.g_padW = padW; p.g_dH = dH; p.g_dW = dW; p.kH = kH; p.kW = kW;
    p.pix_W = oW; p.pix_HW = oH * oW; p.C = C; p.K = K; p.n_img = N;
    p.M_total = K; p.N_total = C * kk; p.Kd = 0; p.kblocks = ips * pb; p.out_HW = 0;
    p.imgs_per_split = ips; p.pix_blocks = pb;
    dim3 grid(ceil_div(K, BM), ceil_div(C * kk, bn), splits);
    if (launch(pick_kernel<OP_WGRAD>(ks_of(kH, kW), bn), p, grid, bn, stream)) return 1;
    const long long n = (long long)K * C * kk;
    const int rblocks = (int)std::max(1LL, std::min(ceil_div_ll(n, 256), (long long)sm_count() * 8));
    wgrad_reduce_kernel<<<rblocks, 256, 0, stream>>>((const float *)workspace, grad_weight, n, splits, scale);
    CUNN_LAUNCH_CHECK("convmm acc grad reduce");
    if (grad_bias) {
        const int chunks = std::max(1, std::min(N, ceil_div(sm_count() * 4, K)));
        float *part = (float *)workspace + (size_t)splits * n;
        bias_partial_kernel<<<K * chunks, 256, 0, stream>>>(gy, part, N, K, oH * oW, chunks);
        CUNN_LAUNCH_CHECK("convmm bias gradient");
        bias_finish_kernel<<<ceil_div(K, 128), 128, 0, stream>>>(part, grad_bias, K, chunks, scale);
        CUNN_LAUNCH_CHECK("convmm bias gradient finish");
    }
    return 0;
}

extern "C" CUNN_API void cunn_b200_convmm_set_tma(int on) { cunn::mm::g_use_tma = on ? 1 : 0; }
extern "C" CUNN_API int cunn_b200_convmm_get_tma(void) { return cunn::mm::g_use_tma; }

extern "C" CUNN_API int cunn_b200_convmm_forward(const float *x, const float *weight, const float *bias, float *y, int N,
                                                 int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH,
                                                 int padW, cunn_stream_t stream)
{
    return conv_forward(x, weight, bias, y, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, stream);
}

extern "C" CUNN_API int cunn_b200_convmm_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H,
                                                    int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                                    cunn_stream_t stream)
{
    return conv_grad_input(gy, weight, gx, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, stream);
}

extern "C" CUNN_API size_t cunn_b200_convmm_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW, int dH,
                                                               int dW, int padH, int padW)
{
    return conv_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1);
}

extern "C" CUNN_API int cunn_b200_convmm_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                                  int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                                  int padH, int padW, float scale, void *workspace, size_t workspace_bytes,
                                                  cunn_stream_t stream)
{
    return conv_acc_grad(x, gy, grad_weight, grad_bias, N, C, H, W, K, kH, kW, dH, dW, padH, padW, 1, 1, scale, workspace,
                         workspace_bytes, stream);
}

extern "C" CUNN_API int cunn_b200_dilated_conv_forward(const float *x, const float *weight, const float *bias, float *y, int N,
                                                       int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH,
                                                       int padW, int dilH, int dilW, cunn_stream_t stream)
{
    return conv_forward(x, weight, bias, y, N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW, stream);
}

extern "C" CUNN_API int cunn_b200_dilated_conv_grad_input(const float *gy, const float *weight, float *gx, int N, int C,
                                                          int H, int W, int K, int kH, int kW, int dH, int dW, int padH,
                                                          int padW, int dilH, int dilW, cunn_stream_t stream)
{
    return conv_grad_input(gy, weight, gx, N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW, stream);
}

extern "C" CUNN_API size_t cunn_b200_dilated_conv_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW,
                                                                     int dH, int dW, int padH, int padW, int dilH, int dilW)
{
    return conv_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW);
}

extern "C" CUNN_API int cunn_b200_dilated_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                                        int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                                        int padH, int padW, int dilH, int dilW, float scale, void *workspace,
                                                        size_t workspace_bytes, cunn_stream_t stream)
{
    return conv_acc_grad(x, gy, grad_weight, grad_bias, N, C, H, W, K, kH, kW, dH, dW, padH, padW, dilH, dilW, scale, workspace,
                         workspace_bytes, stream);
}

// ---------------------------------------------------------------------------
// SpatialFullDilatedConvolution (transposed convolution): x [N,P,H,W], weight [P,Q,kH,kW], y [N,Q,OH,OW].
// It is the adjoint of the convolution that maps [N,Q,OH,OW] to [N,P,H,W] with the same weight array read as
// [K = P][C = Q][kH][kW], so its forward is that convolution's input gradient (plus bias), its input gradient is that
// convolution's forward, and its weight gradient is that convolution's weight gradient with the roles of the
// activations and the output gradient exchanged.
// ---------------------------------------------------------------------------

static int full_check(int N, int P, int H, int W, int Q, int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW,
                      int adjH, int adjW, int *OH, int *OW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(dilW > 0 && dilH > 0, "dilation should be greater than zero, but got dilationH: %d, dilationW: %d", dilH, dilW);
    CUNN_CHECK_ARG(adjH >= 0 && adjW >= 0 && (adjW < dW || adjW < dilW) && (adjH < dH || adjH < dilH),
                   "output padding must be smaller than either stride or dilation, but got adjH: %d adjW: %d dH: %d dW: %d "
                   "dilationH: %d dilationW: %d", adjH, adjW, dH, dW, dilH, dilW);
    CUNN_CHECK_ARG(adjH < dH && adjW < dW, "output padding of at least the stride is not supported (adjH: %d adjW: %d dH: %d dW: %d)",
                   adjH, adjW, dH, dW);
    CUNN_CHECK_ARG(N >= 0 && P > 0 && Q > 0 && H > 0 && W > 0 && padH >= 0 && padW >= 0, "bad convolution sizes");
    const long long oh = (long long)(H - 1) * dH - 2 * padH + (dilH * (kH - 1) + 1) + adjH;
    const long long ow = (long long)(W - 1) * dW - 2 * padW + (dilW * (kW - 1) + 1) + adjW;
    CUNN_CHECK_ARG(oh >= 1 && ow >= 1 && oh < (1 << 24) && ow < (1 << 24),
                   "Given input size: (%d x %d x %d). Calculated output size: (%d x %lld x %lld). Output size is too small", P, H, W,
                   Q, oh, ow);
    *OH = (int)oh; *OW = (int)ow;
    return 0;
}

static int bias_chunks(int N, int Q) { return std::max(1, std::min(N, ceil_div(sm_count() * 4, Q))); }

extern "C" CUNN_API int cunn_b200_full_conv_forward(const float *x, const float *weight, const float *bias, float *y, int N,
                                                    int P, int H, int W, int Q, int kH, int kW, int dH, int dW, int padH,
                                                    int padW, int dilH, int dilW, int adjH, int adjW, cunn_stream_t stream_)
{
    clear_error();
    int OH, OW;
    if (full_check(N, P, H, W, Q, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW, &OH, &OW)) return 1;
    if (conv_grad_input(x, weight, y, N, Q, OH, OW, P, kH, kW, dH, dW, padH, padW, dilH, dilW, stream_)) return 1;
    if (bias && N > 0) {
        const long long total = (long long)N * Q * OH * OW;
        const int blocks = (int)std::max(1LL, std::min(ceil_div_ll(total, 256), (long long)sm_count() * 16));
        add_plane_bias_kernel<<<blocks, 256, 0, (cudaStream_t)stream_>>>(y, bias, Q, OH * OW, total);
        CUNN_LAUNCH_CHECK("full convolution bias");
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_full_conv_grad_input(const float *gy, const float *weight, float *gx, int N, int P, int H,
                                                       int W, int Q, int kH, int kW, int dH, int dW, int padH, int padW,
                                                       int dilH, int dilW, int adjH, int adjW, cunn_stream_t stream_)
{
    clear_error();
    int OH, OW;
    if (full_check(N, P, H, W, Q, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW, &OH, &OW)) return 1;
    return conv_forward(gy, weight, nullptr, gx, N, Q, OH, OW, P, kH, kW, dH, dW, padH, padW, dilH, dilW, stream_);
}

static size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

extern "C" CUNN_API size_t cunn_b200_full_conv_acc_grad_workspace(int N, int P, int H, int W, int Q, int kH, int kW, int dH,
                                                                  int dW, int padH, int padW, int dilH, int dilW, int adjH,
                                                                  int adjW)
{
    int OH, OW;
    if (full_check(N, P, H, W, Q, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW, &OH, &OW) || N == 0) return 0;
    return round256(conv_acc_grad_workspace(N, Q, OH, OW, P, kH, kW, dH, dW, padH, padW, dilH, dilW)) +
           (size_t)Q * bias_chunks(N, Q) * sizeof(float) + 256;
}

extern "C" CUNN_API int cunn_b200_full_conv_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                                     int N, int P, int H, int W, int Q, int kH, int kW, int dH, int dW,
                                                     int padH, int padW, int dilH, int dilW, int adjH, int adjW, float scale,
                                                     void *workspace, size_t workspace_bytes, cunn_stream_t stream_)
{
    clear_error();
    int OH, OW;
    if (full_check(N, P, H, W, Q, kH, kW, dH, dW, padH, padW, dilH, dilW, adjH, adjW, &OH, &OW)) return 1;
    if (N == 0) return 0;
    const size_t conv_ws = round256(conv_acc_grad_workspace(N, Q, OH, OW, P, kH, kW, dH, dW, padH, padW, dilH, dilW));
    const int chunks = bias_chunks(N, Q);
    const size_t need = conv_ws + (size_t)Q * chunks * sizeof(float) + 256;
    CUNN_CHECK_ARG(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                   "full convolution acc_grad needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                   workspace ? workspace_bytes : (size_t)0);
    // the adjoint convolution's "input" is gy and its "output gradient" is x
    if (conv_acc_grad(gy, x, grad_weight, nullptr, N, Q, OH, OW, P, kH, kW, dH, dW, padH, padW, dilH, dilW, scale, workspace,
                      conv_ws, stream_))
        return 1;
    if (grad_bias) {
        cudaStream_t stream = (cudaStream_t)stream_;
        float *part = (float *)((char *)workspace + conv_ws);
        bias_partial_kernel<<<Q * chunks, 256, 0, stream>>>(gy, part, N, Q, OH * OW, chunks);
        CUNN_LAUNCH_CHECK("full convolution bias gradient");
        bias_finish_kernel<<<ceil_div(Q, 128), 128, 0, stream>>>(part, grad_bias, Q, chunks, scale);
        CUNN_LAUNCH_CHECK("full convolution bias gradient finish");
    }
    return 0;
}
