// Pointwise (1x1, stride 1, no padding) convolution GEMMs whose operand tiles are fetched by the TMA unit.
//
// Same roles, tiles and 3xTF32 scheme as pw::pw_gemm_kernel (convmm.cu); what differs is how the raw fp32 tiles reach
// shared memory and how the warps are divided.  There 16 producer warps issue element copies; here ONE thread issues
// tensor-map copies (cp.async.bulk.tensor, one destination CTA each) that land the tiles directly in the layouts the tensor core
// reads, 4 or 8 warps derive the lo tiles (an element-wise map over the 16 KB tile: lo = v - tf32(v)), one warp issues the
// MMAs and 8 or 4 warps drain accumulators, up to four accumulator sets ahead for tiles of one or two k-blocks.
//
//   K-major operand (weights of the forward pass; both operands of the weight gradient, whose reduction runs over
//   pixels): one box of 32 k values x rows, 128-byte rows, hardware 128-byte swizzle = piece_offset().
//   M/N-major operand (activations of forward / input gradient: pixels contiguous; weights of the input gradient: input
//   channels contiguous): the tile is cut into groups of 32 consecutive M/N positions; a group is one box of
//   32 positions x 32 k values = 32 rows of 128 bytes in the 128B-base-32B swizzle, 4 KB; the matrix descriptor steps
//   512 bytes per 4 k values inside a group and 4096 bytes from group to group.
//
// A group of pixels never crosses an image: an image of HW pixels is ceil(HW / 32) groups, the last one padded by the
// TMA unit's zero fill, and GEMM row m means (group m / 32, pixel m % 32 of it).  For HW a multiple of 32 this is the flat
// pixel index.  The weight gradient's k-blocks are (image, group) pairs likewise; zero-filled pixels add nothing.
//
// Requirements (checked by the host, which otherwise keeps the element-copy kernel): HW a multiple of 4 and all three
// tensors 16-byte aligned (tensor-map strides are multiples of 16 bytes), input channels a multiple of 4 for the
// weight matrix's row stride.
#pragma once

#include <cuda.h>

namespace pwt {

using namespace pw;

// Warps: [0, SW) splitters, [SW, SW + EW) epilogue, then one warp that issues the MMAs and one whose lane 0 issues the
// copies.  The library runs SW = 4, EW = 8 (two epilogue warps per TMEM lane quarter, each half of the columns; 448 threads,
// up to 128 registers each): tiles of few k-blocks spend their time in the epilogue, and on long tiles it measured equal
// to 8 + 4 and 4-14 % faster than 16 + 4 (704 threads, 80 registers).
__host__ __device__ constexpr int tma_threads(int sw, int ew) { return (sw + ew + 2) * 32; }
constexpr int MAX_STAGES = 5;                                    // barriers are laid out for up to five raw stages
constexpr int MAX_SETS = 4;                                      // accumulator sets in TMEM the MMA warp may run ahead by
constexpr int HALF_STAGE_COLS = 32;                              // bulk-store epilogue: columns one half of the warps stages at a time
constexpr int GROUP_BYTES = 32 * 128;                            // one M/N-major group: 32 positions x 32 k values
constexpr int MN_KSTEP = 512;                                    // M/N-major: bytes from 4 k values to the next 4 inside a group
static_assert(2 * HALF_STAGE_COLS * BM * 4 == (int)OUT_STAGE, "the two halves share the output staging area");

__device__ __forceinline__ uint64_t desc_mn_grouped(uint32_t addr) { return desc_of(addr, GROUP_BYTES, MN_KSTEP) | (1ull << 61); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// Tensor-map store shared -> global of one box (dense rows in shared memory); joins the thread's bulk group.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"((uint64_t)map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
// Barrier among the four epilogue warps of one column half (hardware barriers 1 and 2).
__device__ __forceinline__ void half_sync(int half)
{
    if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Sum over the tile's accumulators of 16 columns starting at TMEM address `t0` (+ a * acc_cols), on top of `acc`.
// PAIRS: accumulators are read two at a time, so that two loads are in flight per wait (16 more registers).
template <bool PAIRS>
__device__ __forceinline__ void gather_acc16(float (&acc)[16], uint32_t t0, int nhi_used, int nacc, int acc_cols)
{
    const int n = nhi_used + 1;                                   // the hi accumulators that were used, then the lo one
    for (int a2 = 0; a2 < n; a2 += PAIRS ? 2 : 1) {
        const int a = a2 < nhi_used ? a2 : nacc - 1;
        uint32_t r0[16], r1[16];
        tmem_ld16_issue(t0 + (uint32_t)(a * acc_cols), r0);
        const bool two = PAIRS && a2 + 1 < n;
        if (two) {
            const int b = a2 + 1 < nhi_used ? a2 + 1 : nacc - 1;
            tmem_ld16_issue(t0 + (uint32_t)(b * acc_cols), r1);
        }
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r0[j]);
        if (two) {
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r1[j]);
        }
    }
}

// Epilogue of one tile for one epilogue warp: sums the tile's accumulators (TMEM address `tset`: first column of the
// accumulator set), adds the bias and writes the warp's 32 rows (TMEM lane quarter `quarter`) x its half of the columns.
// `el` is the thread's index inside its half (0 .. 127), `stage_base` the 32 KB output staging area in shared memory.
template <int OP, int BN, int HALVES>
__device__ __forceinline__ void drain_tile(const Params &p, const CUtensorMap &map_out, float *stage_base, uint32_t tset, int t, int nhi_used,
                                           int quarter, int half, int lane, int el)
{
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    constexpr int HALF_COLS = BN / HALVES;
    const int row = quarter * 32 + lane;
    const int col_lo = half * HALF_COLS, col_hi = col_lo + HALF_COLS;
    const uint32_t tsrc = tset + ((uint32_t)(quarter * 32) << 16);
    int n_tile0;
    size_t dst_off = 0;
    bool row_ok, done = false;
    if (OP != OP_WGRAD) {
        const int m_tile = t / p.n_tiles, n_tile = t - m_tile * p.n_tiles;
        n_tile0 = n_tile * BN;
        const int g = m_tile * 4 + quarter, im = g / p.gpi, pix = (g - im * p.gpi) * 32 + lane;
        row_ok = im < p.n_img && pix < p.HW;
        dst_off = ((size_t)im * p.N_total + n_tile0) * p.HW + pix;
        if (p.bulk_out && (m_tile + 1) * BM <= p.n_img * p.HW) {
            // planes of a multiple of 32 (and >= 1024) pixels: rows are flat pixel indices; each half stages 32 columns x
            // 128 pixels at a time and the TMA unit writes every column's 512-byte run (two runs across an image boundary)
            float *stage = stage_base + half * HALF_STAGE_COLS * BM;
            const int m_tile0 = m_tile * BM;
            const int im0 = m_tile0 / p.HW, pix0 = m_tile0 - im0 * p.HW;
            const int len0 = min(BM, p.HW - pix0);
#pragma unroll 1
            for (int cbase = col_lo; cbase < col_hi; cbase += HALF_STAGE_COLS) {
                bulk_wait_read_all();                        // this thread's earlier bulk stores have left the buffer
                half_sync(half);
#pragma unroll 1
                for (int c0 = cbase; c0 < cbase + HALF_STAGE_COLS && c0 < col_hi; c0 += 16) {
                    float acc[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
                    gather_acc16<HALVES == 2>(acc, tsrc + (uint32_t)c0, nhi_used, p.nacc, ACC_COLS);
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[(c0 - cbase + j) * BM + row] = acc[j];
                }
                fence_async_smem();
                half_sync(half);
                if (len0 == BM && HALF_COLS >= HALF_STAGE_COLS) {
                    // the tile lies inside one image: one tensor-map store writes the 128 pixels x 32 columns staged
                    // by this half (columns past the last output channel are clipped by the map's bounds)
                    if (el == 0) {
                        tma_store_3d(&map_out, smem_u32(stage), pix0, n_tile0 + cbase, im0);
                        bulk_commit();
                    }
                    continue;
                }
                const int col = cbase + el, n = n_tile0 + col;
                if (el < HALF_STAGE_COLS && col < col_hi && n < p.N_total) {
                    const uint32_t src = smem_u32(stage + el * BM);
                    float *dst = p.out + ((size_t)im0 * p.N_total + n) * p.HW + pix0;
                    bulk_s2g_nocommit(dst, src, (uint32_t)len0 * 4u);
                    if (len0 < BM) bulk_s2g_nocommit(p.out + ((size_t)(im0 + 1) * p.N_total + n) * p.HW, src + (uint32_t)len0 * 4u, (uint32_t)(BM - len0) * 4u);
                    bulk_commit();
                }
            }
            done = true;
        }
    } else {
        const int split = t / p.tiles_per_split, r2 = t - split * p.tiles_per_split;
        const int m_tile = r2 / p.n_tiles, n_tile = r2 - m_tile * p.n_tiles;
        const int m = m_tile * BM + row;
        n_tile0 = n_tile * BN;
        row_ok = m < p.M_total;
        dst_off = ((size_t)split * p.M_total + m) * p.N_total + n_tile0;
    }
    if (!done) {
#pragma unroll 1
        for (int c0 = col_lo; c0 < col_hi; c0 += 16) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
                acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
            gather_acc16<HALVES == 2>(acc, tsrc + (uint32_t)c0, nhi_used, p.nacc, ACC_COLS);
            if (row_ok) {
                const int n0 = n_tile0 + c0;
                if (OP != OP_WGRAD) {
                    float *dst = p.out + dst_off + (size_t)c0 * p.HW;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (n0 + j < p.N_total) dst[(size_t)j * p.HW] = acc[j];
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
    }
}

template <int OP, int BN, int SW, int EW, int NS, int NL>
__global__ void __launch_bounds__(tma_threads(SW, EW), 1)
pw_tma_kernel(const Params p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const __grid_constant__ CUtensorMap map_out)
{
    constexpr bool A_MN = OP != OP_WGRAD;
    constexpr bool B_MN = OP == OP_DGRAD;
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t idesc = idesc_of(BN, A_MN, B_MN);
    constexpr uint32_t A_BYTES = TILE;                           // 128 rows (or 4 groups) x 32 k values
    constexpr uint32_t B_BYTES = (uint32_t)BN * 128u;
    constexpr int MMA_WARP = SW + EW, TMA_WARP = MMA_WARP + 1;
    constexpr int SPLITTERS = SW * 32;
    constexpr int SPLIT_PIECES = TILE / 16 / SPLITTERS;          // 16-byte pieces of a tile per splitter thread
    static_assert(SW % 4 == 0 && (EW == 4 || EW == 8) && (SPLIT_PIECES % 4 == 0 || SPLIT_PIECES == 2), "warp roles");

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t mmadone[MAX_STAGES];    // the MMAs that read this raw stage (and the lo buffer of the same k-block) have finished
    __shared__ uint64_t accready[MAX_SETS];     // all MMAs of a tile have finished: its accumulator set can be read
    __shared__ uint64_t accfree[MAX_SETS];      // accumulator set drained: one arrival per epilogue warp
    __shared__ uint64_t rawfull[MAX_STAGES];    // the stage's raw tiles have landed (transaction bytes)
    __shared__ uint64_t full[MAX_STAGES];       // lo tiles written and visible to the tensor core: one arrival per splitter warp
    __shared__ uint32_t tmem_base_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(smem_u32(mmadone + s), 1);
            mbar_init(smem_u32(rawfull + s), 1);
            mbar_init(smem_u32(full + s), SW);
        }
        for (int s = 0; s < MAX_SETS; ++s) { mbar_init(smem_u32(accready + s), 1); mbar_init(smem_u32(accfree + s), EW); }
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    const int KB = p.kblocks;
    // NS raw stages and NL lo buffers of 32 KB (the library runs 4 + 2, which leaves room for the 32 KB output staging area;
    // 4 + 3 and 5 + 2 without the staging area measured within 3 % of it)
    static_assert(NS >= NL && NS <= MAX_STAGES && (size_t)(NS + NL) * 2 * TILE + 1024 <= SMEM, "one completion barrier per raw stage also guards the lo buffers");
    const int my_tiles = ((int)blockIdx.x < p.total_tiles) ? (p.total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total_it = my_tiles * KB;
    // nacc == 1: all three products of every k-block go to one accumulator (tiles of one or two k-blocks, whose chains are
    // short anyway); otherwise the hi*hi products are dealt round-robin to nacc - 1 accumulators and the cross terms share the last
    const int nhi = p.nacc - 1;
    const int nhi_used = KB < nhi ? KB : nhi;
    const uint32_t set_cols = (uint32_t)(p.nacc * ACC_COLS);
    unsigned char *const lo_base = smem + (size_t)NS * 2 * TILE;
    bool ok = true;

    if (warp == TMA_WARP) {
        // ---- copy issue: k-block i goes to raw stage i % NS as soon as the MMAs that read it last are done ----
        if (lane == 0) {
            int t = (int)blockIdx.x, kb = 0;
            for (int i = 0; i < total_it; ++i) {
                const int rs = i % NS;
                if (i >= NS && !mbar_wait(smem_u32(mmadone + rs), (uint32_t)((i / NS - 1) & 1), p.status)) break;
                const uint32_t bar = smem_u32(rawfull + rs);
                const uint32_t sa = smem_u32(smem + (size_t)rs * 2 * TILE), sb = sa + TILE;
                mbar_arrive_expect_tx(bar, A_BYTES + B_BYTES);
                if (OP != OP_WGRAD) {
                    const int m_tile = t / p.n_tiles, n_tile = t - m_tile * p.n_tiles;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int g = m_tile * 4 + j, im = g / p.gpi, p0 = (g - im * p.gpi) * 32;
                        tma_load_3d(sa + (uint32_t)(j * GROUP_BYTES), &map_a, p0, kb * BK, im, bar);     // image >= n_img: zero fill
                    }
                    if (OP == OP_FWD) {
                        tma_load_2d(sb, &map_b, kb * BK, n_tile * BN, bar);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 32; ++j) tma_load_2d(sb + (uint32_t)(j * GROUP_BYTES), &map_b, n_tile * BN + 32 * j, kb * BK, bar);
                    }
                } else {
                    const int split = t / p.tiles_per_split, r = t - split * p.tiles_per_split;
                    const int m_tile = r / p.n_tiles, n_tile = r - m_tile * p.n_tiles;
                    const int im = split * p.imgs_per_split + kb / p.gpi, p0 = (kb % p.gpi) * 32;
                    tma_load_3d(sa, &map_a, p0, m_tile * BM, im, bar);
                    tma_load_3d(sb, &map_b, p0, n_tile * BN, im, bar);
                }
                if (++kb == KB) { kb = 0; t += (int)gridDim.x; }
            }
        }
    } else if (warp == MMA_WARP) {
        // ---- MMA issue.  The tensor pipe takes a 128 x 128 x 8 tf32 MMA every 64 clocks only if the issuing thread keeps up:
        // every instruction between two tcgen05.mma of this single thread is time the pipe idles (measured: 64 clocks per MMA
        // from a bare loop, 102-130 with descriptors rebuilt and counters divided per MMA; running the loop on all 32 lanes with
        // only the instruction predicated was slower).  So: one lane runs the whole loop,
        // descriptors are a constant upper word + a lower word that advances by additions, ring positions and barrier
        // parities are carried incrementally, and the accumulate flags of the steady state are constants. ----
        if (lane == 0) {
            // lower descriptor word = (address >> 4) | 1 << 16 (K-major: leading offset 16 bytes) or | GROUP_BYTES >> 4 << 16
            constexpr uint32_t A_LOW = A_MN ? ((uint32_t)(GROUP_BYTES >> 4) << 16) : (1u << 16);
            constexpr uint32_t B_LOW = B_MN ? ((uint32_t)(GROUP_BYTES >> 4) << 16) : (1u << 16);
            // upper word: stride offset, descriptor version 1, swizzle (128B-base-32B = 1, 128B = 2)
            constexpr uint32_t A_HIGH = (A_MN ? (uint32_t)(MN_KSTEP >> 4) : (uint32_t)(SBO >> 4)) | (1u << 14) | ((A_MN ? 1u : 2u) << 29);
            constexpr uint32_t B_HIGH = (B_MN ? (uint32_t)(MN_KSTEP >> 4) : (uint32_t)(SBO >> 4)) | (1u << 14) | ((B_MN ? 1u : 2u) << 29);
            constexpr uint32_t A_STEP = A_MN ? (uint32_t)(2 * MN_KSTEP >> 4) : 2u;     // 8 k values further, in 16-byte units
            constexpr uint32_t B_STEP = B_MN ? (uint32_t)(2 * MN_KSTEP >> 4) : 2u;
            constexpr uint32_t STAGE_STEP = (uint32_t)(2 * TILE >> 4);
            const uint32_t raw0 = (smem_u32(smem) >> 4) & 0x3fffu, lo0 = (smem_u32(lo_base) >> 4) & 0x3fffu;
            auto desc = [](uint32_t low, uint32_t high) { return ((uint64_t)high << 32) | low; };
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
                if (kb == 0 || (nhi && kb < nhi)) {
                    // first k-block(s) of a tile: the first MMA into an accumulator overwrites it
                    const uint32_t keep_lo = kb == 0 ? 0u : 1u, keep_hi = (nhi && kb < nhi) ? 0u : 1u;
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
                umma_commit(smem_u32(mmadone + rs));
                if (++rs == NS) { rs = 0; full_parity ^= 1u; }
                if (++lb == NL) lb = 0;
                if (nhi && ++hi_slot == nhi) hi_slot = 0;
                if (++kb == KB) {
                    umma_commit(smem_u32(accready + set));
                    kb = 0;
                    hi_slot = 0;
                    acc0 += set_cols;
                    if (++set == p.sets) { set = 0; acc0 = tmem_base; if (!first_round) free_parity ^= 1u; first_round = false; }
                }
            }
        }
    } else if (warp >= SW && warp < MMA_WARP) {
        // ---- epilogue warps: TMEM -> registers -> global memory, one pass over this CTA's tiles.  Warp e reads the TMEM
        // lanes of quarter e % 4 (the hardware's rule) and the columns of half e / 4. ----
        const int e = warp - SW, quarter = e & 3, half = e >> 2;
        for (int count = 0; count < my_tiles; ++count) {
            const int t = (int)blockIdx.x + count * (int)gridDim.x;
            const int set = count % p.sets;
            if (!mbar_wait(smem_u32(accready + set), (uint32_t)((count / p.sets) & 1), p.status)) { ok = false; break; }
            tc_fence_after();
            drain_tile<OP, BN, EW / 4>(p, map_out, reinterpret_cast<float *>(smem + (size_t)(NS + NL) * 2 * TILE), tmem_base + (uint32_t)set * set_cols, t,
                               nhi_used, quarter, half, lane, tid - (SW + 4 * half) * 32);
            tc_fence_before();                                       // the TMEM reads above are ordered before the arrival
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(accfree + set));
        }
        bulk_wait_read_all();                                        // shared memory must outlive the last bulk stores' reads
    } else if (warp < SW) {
        // ---- splitter warps: lo = v - tf32(v), element-wise over the raw tiles; thread t owns the 16-byte pieces at byte
        // offsets 16 t + SPLITTERS * 16 h of both tiles, i.e. row t / 8 + SPLITTERS / 8 * h of a K-major tile ----
        constexpr uint32_t PSTEP = SPLITTERS * 16;
        float bsum[SPLIT_PIECES];                                    // WGRAD: running row sums of gy (bias gradient)
#pragma unroll
        for (int h = 0; h < SPLIT_PIECES; ++h) bsum[h] = 0.f;
        int c_tile = (int)blockIdx.x, c_kb = 0;
        for (int i = 0; i < total_it; ++i) {
            const int rs = i % NS, lb = i % NL;
            if (!mbar_wait(smem_u32(rawfull + rs), (uint32_t)((i / NS) & 1), p.status)) { ok = false; break; }
            if (i >= NL) {
                // the MMAs of k-block i - NL read this lo buffer.  One commit per k-block serves both rings: the barrier of
                // raw stage (i - NL) % NS cannot advance a second time before this wait, because the next k-block that uses
                // that stage is i - NL + NS >= i, whose MMAs need this very split (NS >= NL)
                const int j = i - NL;
                if (!mbar_wait(smem_u32(mmadone + j % NS), (uint32_t)((j / NS) & 1), p.status)) { ok = false; break; }
            }
            const unsigned char *a_hi = smem + (size_t)rs * 2 * TILE, *b_hi = a_hi + TILE;
            unsigned char *a_lo = lo_base + (size_t)lb * 2 * TILE, *b_lo = a_lo + TILE;
            constexpr int PG = SPLIT_PIECES < 4 ? SPLIT_PIECES : 4;      // pieces loaded before their lo values are stored
#pragma unroll
            for (int h0 = 0; h0 < SPLIT_PIECES; h0 += PG) {
                float4 va[PG], vb[PG];
#pragma unroll
                for (int h = 0; h < PG; ++h) {
                    const uint32_t off = (uint32_t)tid * 16u + (uint32_t)(h0 + h) * PSTEP;
                    va[h] = *reinterpret_cast<const float4 *>(a_hi + off);
                    if (off < B_BYTES) vb[h] = *reinterpret_cast<const float4 *>(b_hi + off);
                }
#pragma unroll
                for (int h = 0; h < PG; ++h) {
                    const uint32_t off = (uint32_t)tid * 16u + (uint32_t)(h0 + h) * PSTEP;
                    store_lo_at(a_lo, off, va[h]);
                    if (OP == OP_WGRAD) bsum[h0 + h] += (va[h].x + va[h].y) + (va[h].z + va[h].w);
                    if (off < B_BYTES) store_lo_at(b_lo, off, vb[h]);
                }
            }
            fence_async_smem();                                      // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(full + rs));
            if (c_kb == KB - 1) {
                if (OP == OP_WGRAD) {
                    // bias gradient: the eight lanes that share a row hold its partial sums
#pragma unroll
                    for (int r = 0; r < SPLIT_PIECES; ++r) {
                        float sum = bsum[r];
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                        const int split = c_tile / p.tiles_per_split, r2 = c_tile - split * p.tiles_per_split;
                        const int m_tile = r2 / p.n_tiles, n_tile = r2 - m_tile * p.n_tiles;
                        const int m = m_tile * BM + (tid >> 3) + (SPLITTERS / 8) * r;
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
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace pwt
