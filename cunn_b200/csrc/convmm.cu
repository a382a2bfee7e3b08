// SpatialConvolutionMM on the 5th-generation tensor cores (tcgen05 / TMEM), fp32 in and out.
//
// The reference unfolds every image into a column buffer and calls SGEMM per image.  Here the three
// passes are implicit GEMMs — no column buffer exists — computed by tcgen05.mma.kind::tf32 with a
// 3xTF32 split: every fp32 operand value v is written to shared memory twice, as hi = tf32(v) and
// lo = v - hi, and each K step issues hi*hi + hi*lo + lo*hi into one fp32 TMEM accumulator.  The
// dropped lo*lo term and the tf32 rounding of lo are ~2^-21 relative, i.e. fp32-class accuracy.
//
//   forward      D[pixel, k_out]        = sum_{c,kh,kw}  x(pixel; c,kh,kw)   * W[k_out][c,kh,kw]
//   input grad   D[pixel, c]            = sum_{k,kh,kw}  gy(pixel; k,kh,kw)  * W[k][c][flipped kh,kw]   (stride 1)
//   weight grad  D[k_out, (c,kh,kw)]    = sum_{img,pix}  gy[img][k_out][pix] * x(pix; c,kh,kw)          (split over images)
//
// One CTA computes a 128 x BN tile of D.  All 256 threads gather operand values from global memory
// (coalesced along pixels, two k-blocks in flight in registers), split them and store 16-byte pieces
// into K-major, non-swizzled core-matrix layout (8 rows x 16 bytes); one thread then issues the MMAs of
// the k-block and commits them to the mbarrier that frees the stage.  The epilogue reads the
// accumulator with tcgen05.ld (lane = tile row) and writes coalesced NCHW rows.  Every wait is bounded.
//
// Input gradients for stride > 1 use a plain gather kernel (no network on the benchmarked path needs
// them: a strided first layer has no input gradient).
#include "common.cuh"

#include <algorithm>

namespace cunn {
namespace mm {

enum Op : int { OP_FWD = 0, OP_DGRAD = 1, OP_WGRAD = 2 };

constexpr int BM = 128;       // tile rows (TMEM lanes)
constexpr int BK = 32;        // k-block: 8 chunks of 4 values (16 bytes)
constexpr int THREADS = 256;
constexpr int LBO = 128;      // bytes between the two 16-byte K chunks of an MMA (adjacent core matrices)
constexpr int SBO = 1024;     // bytes between 8-row groups: 8 chunks x 128 bytes

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

// Shared-memory matrix descriptor: K-major, no swizzle, core matrices of 8 rows x 16 bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)(LBO >> 4) << 16) | ((uint64_t)(SBO >> 4) << 32) | (1ull << 46);
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
__device__ __forceinline__ uint32_t piece_offset(int row, int kc) { return (uint32_t)((row >> 3) * SBO + kc * LBO + (row & 7) * 16); }

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
            const uint32_t koff = (uint32_t)j * 2 * LBO;      // two 16-byte chunks per MMA
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

// Input gradient for any stride: gather form, one thread per input pixel (correctness path).
__global__ void __launch_bounds__(256)
dgrad_gather_kernel(const float *__restrict__ gy, const float *__restrict__ w, float *__restrict__ gx, int C, int H, int W,
                    int K, int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW, long long total)
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
            const int a = h + padH - kh;
            if (a < 0 || a % dH) continue;
            const int oh = a / dH;
            if (oh >= oH) continue;
            for (int kw = 0; kw < kW; ++kw) {
                const int b = wi + padW - kw;
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

static int check(int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH, int padW, int *oH, int *oW)
{
    CUNN_CHECK_ARG(kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    CUNN_CHECK_ARG(dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    CUNN_CHECK_ARG(N >= 0 && C > 0 && K > 0 && H > 0 && W > 0 && padH >= 0 && padW >= 0, "bad convolution sizes");
    *oH = (H + 2 * padH - kH) / dH + 1;
    *oW = (W + 2 * padW - kW) / dW + 1;
    CUNN_CHECK_ARG(H + 2 * padH >= kH && W + 2 * padW >= kW && *oH >= 1 && *oW >= 1,
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

}  // namespace mm
}  // namespace cunn

using namespace cunn;
using namespace cunn::mm;

extern "C" CUNN_API int cunn_b200_convmm_forward(const float *x, const float *weight, const float *bias, float *y, int N,
                                                 int C, int H, int W, int K, int kH, int kW, int dH, int dW, int padH,
                                                 int padW, cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && weight && y, "null tensor pointer");
    GemmParams p{};
    p.a_src = x; p.b_src = weight; p.bias = bias; p.out = y; p.status = device_status_ptr();
    p.g_C = C; p.g_H = H; p.g_W = W; p.g_padH = padH; p.g_padW = padW; p.g_dH = dH; p.g_dW = dW; p.kH = kH; p.kW = kW;
    p.pix_W = oW; p.pix_HW = oH * oW; p.C = C; p.K = K; p.n_img = N;
    p.M_total = N * oH * oW; p.N_total = K; p.Kd = C * kH * kW; p.kblocks = ceil_div(p.Kd, BK); p.out_HW = oH * oW;
    const int bn = pick_bn_for(K);
    dim3 grid(ceil_div(p.M_total, BM), ceil_div(K, bn), 1);
    return launch(pick_kernel<OP_FWD>(ks_of(kH, kW), bn), p, grid, bn, stream);
}

extern "C" CUNN_API int cunn_b200_convmm_grad_input(const float *gy, const float *weight, float *gx, int N, int C, int H,
                                                    int W, int K, int kH, int kW, int dH, int dW, int padH, int padW,
                                                    cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(gy && weight && gx, "null tensor pointer");
    if (dH == 1 && dW == 1 && padH <= kH - 1 && padW <= kW - 1) {
        // stride 1: a convolution of gy with the kernel rotated by 180 degrees and padding k - 1 - pad
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
    dgrad_gather_kernel<<<blocks, 256, 0, stream>>>(gy, weight, gx, C, H, W, K, kH, kW, dH, dW, padH, padW, oH, oW, total);
    CUNN_LAUNCH_CHECK("convmm grad input (gather)");
    return 0;
}

extern "C" CUNN_API size_t cunn_b200_convmm_acc_grad_workspace(int N, int C, int H, int W, int K, int kH, int kW, int dH,
                                                               int dW, int padH, int padW)
{
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW) || N == 0) return 0;
    int bn, splits, ips, pb;
    wgrad_plan(N, C, K, kH * kW, oH * oW, &bn, &splits, &ips, &pb);
    const int chunks = std::max(1, std::min(N, ceil_div(sm_count() * 4, K)));
    return (size_t)splits * K * C * kH * kW * sizeof(float) + (size_t)K * chunks * sizeof(float) + 256;
}

extern "C" CUNN_API int cunn_b200_convmm_acc_grad(const float *x, const float *gy, float *grad_weight, float *grad_bias,
                                                  int N, int C, int H, int W, int K, int kH, int kW, int dH, int dW,
                                                  int padH, int padW, float scale, void *workspace, size_t workspace_bytes,
                                                  cunn_stream_t stream_)
{
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    int oH, oW;
    if (check(N, C, H, W, K, kH, kW, dH, dW, padH, padW, &oH, &oW)) return 1;
    if (N == 0) return 0;
    CUNN_CHECK_ARG(x && gy && grad_weight, "null tensor pointer");
    const size_t need = cunn_b200_convmm_acc_grad_workspace(N, C, H, W, K, kH, kW, dH, dW, padH, padW);
    CUNN_CHECK_ARG(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                   "convmm acc_grad needs %zu bytes of 16-byte aligned workspace, got %zu", need,
                   workspace ? workspace_bytes : (size_t)0);
    int bn, splits, ips, pb;
    const int kk = kH * kW;
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
