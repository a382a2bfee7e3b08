// Pointwise (1x1, stride 1, no padding) convolution GEMMs whose operand tiles are fetched by the TMA unit.
//
// Same roles, tiles, 3xTF32 scheme, accumulator plan and epilogue as pw::pw_gemm_kernel (convmm.cu); what differs is
// how the raw fp32 tiles reach shared memory.  There 16 producer warps issue element copies; here ONE thread issues
// tensor-map copies (cp.async.bulk.tensor, no multicast) that land the tiles directly in the layouts the tensor core
// reads, and the 16 warps only derive the lo tiles (an element-wise map over the 16 KB tile: lo = v - tf32(v)).
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

constexpr int SPLITTERS = 512;                                   // threads that derive the lo tiles (16 warps)
constexpr int MMA_WARP = SPLITTERS / 32;                         // one warp that only issues MMAs
constexpr int EPI_WARP0 = MMA_WARP + 1;                          // four epilogue warps
constexpr int TMA_WARP = EPI_WARP0 + EPILOGUE_WARPS;             // one warp whose lane 0 issues the tensor-map copies
constexpr int TTHREADS = (TMA_WARP + 1) * 32;                    // 704
constexpr int GROUP_BYTES = 32 * 128;                            // one M/N-major group: 32 positions x 32 k values
constexpr int MN_KSTEP = 512;                                    // M/N-major: bytes from 4 k values to the next 4 inside a group

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
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * EPILOGUE_WARPS) : "memory"); }

template <int OP, int BN>
__global__ void __launch_bounds__(TTHREADS, 1)
pw_tma_kernel(const Params p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b)
{
    constexpr bool A_MN = OP != OP_WGRAD;
    constexpr bool B_MN = OP == OP_DGRAD;
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t idesc = idesc_of(BN, A_MN, B_MN);
    constexpr uint32_t A_BYTES = TILE;                           // 128 rows (or 4 groups) x 32 k values
    constexpr uint32_t B_BYTES = (uint32_t)BN * 128u;

    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[RAW_STAGES + 2];   // MMAs of this stage done; then accumulators of set 0 / 1 ready
    __shared__ uint64_t rawfull[RAW_STAGES];    // the stage's raw tiles have landed (transaction bytes)
    __shared__ uint64_t full[RAW_STAGES];       // lo tiles written and visible to the tensor core: one arrival per splitter warp
    __shared__ uint64_t accfree[2];
    __shared__ uint32_t tmem_base_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < RAW_STAGES + 2; ++s) mbar_init(smem_u32(bars + s), 1);
        for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(smem_u32(rawfull + s), 1); mbar_init(smem_u32(full + s), SPLITTERS / 32); }
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
    const int nhi_used = KB < p.nacc - 1 ? KB : p.nacc - 1;
    const uint32_t set_cols = (uint32_t)(p.nacc * ACC_COLS);
    unsigned char *const lo_base = smem + (size_t)RAW_STAGES * 2 * TILE;
    bool ok = true;

    if (warp == TMA_WARP) {
        // ---- copy issue: k-block i goes to raw stage i % RAW_STAGES as soon as the MMAs that read it last are done ----
        if (lane == 0) {
            int t = (int)blockIdx.x, kb = 0;
            for (int i = 0; i < total_it; ++i) {
                const int rs = i % RAW_STAGES;
                if (i >= RAW_STAGES && !mbar_wait(smem_u32(bars + rs), (uint32_t)((i / RAW_STAGES - 1) & 1), p.status)) break;
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
        int kb = 0, count = 0;
        for (int i = 0; i < total_it; ++i) {
            const int rs = i % RAW_STAGES, lb = i % LO_BUFS;
            if (!mbar_wait(smem_u32(full + rs), (uint32_t)((i / RAW_STAGES) & 1), p.status)) { ok = false; break; }
            if (kb == 0 && count >= p.sets) {
                const int set = (p.sets == 2) ? (count & 1) : 0;
                const int use = (p.sets == 2) ? (count >> 1) : count;
                if (!mbar_wait(smem_u32(accfree + set), (uint32_t)((use - 1) & 1), p.status)) { ok = false; break; }
            }
            if (lane == 0) {
                tc_fence_after();
                const int set = (p.sets == 2) ? (count & 1) : 0;
                const uint32_t acc0 = tmem_base + (uint32_t)set * set_cols;
                const int nhi = p.nacc - 1;
                const uint32_t d_hi = acc0 + (uint32_t)((kb % nhi) * ACC_COLS), d_lo = acc0 + (uint32_t)(nhi * ACC_COLS);
                const bool first_hi = kb < nhi, first_lo = kb == 0;
                const uint32_t sa_hi = smem_u32(smem + (size_t)rs * 2 * TILE), sb_hi = sa_hi + TILE;
                const uint32_t sa_lo = smem_u32(lo_base + (size_t)lb * 2 * TILE), sb_lo = sa_lo + TILE;
#pragma unroll
                for (int j = 0; j < BK / 8; ++j) {
                    const uint32_t ao = A_MN ? (uint32_t)(j * 2 * MN_KSTEP) : (uint32_t)(j * 32);
                    const uint32_t bo = B_MN ? (uint32_t)(j * 2 * MN_KSTEP) : (uint32_t)(j * 32);
                    const uint64_t ah = A_MN ? desc_mn_grouped(sa_hi + ao) : smem_desc(sa_hi + ao);
                    const uint64_t al = A_MN ? desc_mn_grouped(sa_lo + ao) : smem_desc(sa_lo + ao);
                    const uint64_t bh = B_MN ? desc_mn_grouped(sb_hi + bo) : smem_desc(sb_hi + bo);
                    const uint64_t bl = B_MN ? desc_mn_grouped(sb_lo + bo) : smem_desc(sb_lo + bo);
                    umma_tf32(d_lo, al, bh, idesc, (first_lo && j == 0) ? 0u : 1u);
                    umma_tf32(d_lo, ah, bl, idesc, 1u);
                    umma_tf32(d_hi, ah, bh, idesc, (first_hi && j == 0) ? 0u : 1u);
                }
                umma_commit(smem_u32(bars + rs));
                if (kb == KB - 1) umma_commit(smem_u32(bars + RAW_STAGES + set));
            }
            __syncwarp();
            if (++kb == KB) { kb = 0; ++count; }
        }
    } else if (warp >= EPI_WARP0) {
        // ---- epilogue warps: TMEM -> registers -> global memory, one pass over this CTA's tiles ----
        const int quarter = warp & 3;                                 // the TMEM lanes this warp may read
        const int row = quarter * 32 + lane;
        for (int count = 0; count < my_tiles && ok; ++count) {
            const int t = (int)blockIdx.x + count * (int)gridDim.x;
            const int set = (p.sets == 2) ? (count & 1) : 0;
            const uint32_t parity = (uint32_t)(((p.sets == 2) ? (count >> 1) : count) & 1);
            if (!mbar_wait(smem_u32(bars + RAW_STAGES + set), parity, p.status)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)set * set_cols;
            int n_tile0;
            size_t dst_off = 0;
            bool row_ok;
            if (OP != OP_WGRAD) {
                const int m_tile = t / p.n_tiles, n_tile = t - m_tile * p.n_tiles;
                n_tile0 = n_tile * BN;
                const int g = m_tile * 4 + quarter, im = g / p.gpi, pix = (g - im * p.gpi) * 32 + lane;
                row_ok = im < p.n_img && pix < p.HW;
                dst_off = ((size_t)im * p.N_total + n_tile0) * p.HW + pix;
                if (p.bulk_out && (m_tile + 1) * BM <= p.n_img * p.HW) {
                    // planes of a multiple of 32 (and >= 1024) pixels: rows are flat pixel indices; stage 64 columns x 128
                    // pixels and let the TMA unit write each column's 512-byte run (two runs across an image boundary)
                    float *stage = reinterpret_cast<float *>(smem + (size_t)(RAW_STAGES + LO_BUFS) * 2 * TILE);
                    const int e = tid - EPI_WARP0 * 32;              // 0 .. 127
                    const int m_tile0 = m_tile * BM;
                    const int im0 = m_tile0 / p.HW, pix0 = m_tile0 - im0 * p.HW;
                    const int len0 = min(BM, p.HW - pix0);
#pragma unroll 1
                    for (int cbase = 0; cbase < BN; cbase += STAGE_COLS) {
                        bulk_wait_read_all();
                        epi_sync();
#pragma unroll 1
                        for (int c0 = cbase; c0 < cbase + STAGE_COLS && c0 < BN; c0 += 16) {
                            float acc[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
                            for (int a2 = 0; a2 <= nhi_used; ++a2) {
                                const int a = a2 < nhi_used ? a2 : p.nacc - 1;
                                uint32_t r[16];
                                tmem_ld16(tsrc + (uint32_t)(a * ACC_COLS + c0), r);
#pragma unroll
                                for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r[j]);
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) stage[(c0 - cbase + j) * BM + row] = acc[j];
                        }
                        fence_async_smem();
                        epi_sync();
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
                    continue;
                }
            } else {
                const int split = t / p.tiles_per_split, r2 = t - split * p.tiles_per_split;
                const int m_tile = r2 / p.n_tiles, n_tile = r2 - m_tile * p.n_tiles;
                const int m = m_tile * BM + row;
                n_tile0 = n_tile * BN;
                row_ok = m < p.M_total;
                dst_off = ((size_t)split * p.M_total + m) * p.N_total + n_tile0;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float acc[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    acc[j] = (OP == OP_FWD && p.bias && n_tile0 + c0 + j < p.N_total) ? __ldg(p.bias + n_tile0 + c0 + j) : 0.f;
                for (int a2 = 0; a2 <= nhi_used; ++a2) {
                    const int a = a2 < nhi_used ? a2 : p.nacc - 1;
                    uint32_t r[16];
                    tmem_ld16(tsrc + (uint32_t)(a * ACC_COLS + c0), r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(r[j]);
                }
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(accfree + set));
        }
        bulk_wait_read_all();
    } else {
        // ---- splitter warps: lo = v - tf32(v), element-wise over the raw tiles; thread t owns the 16-byte pieces at
        // byte offsets 16 t and 16 t + 8192 of both tiles (row t / 8 + 64 i of a K-major tile) ----
        float bsum[2] = {0.f, 0.f};                                  // WGRAD: running row sums of gy (bias gradient)
        int c_tile = (int)blockIdx.x, c_kb = 0;
        for (int i = 0; i < total_it; ++i) {
            const int rs = i % RAW_STAGES, lb = i % LO_BUFS;
            if (!mbar_wait(smem_u32(rawfull + rs), (uint32_t)((i / RAW_STAGES) & 1), p.status)) { ok = false; break; }
            if (i >= LO_BUFS) {
                const int j = i - LO_BUFS;                           // the MMAs of k-block i - 2 read this lo buffer
                if (!mbar_wait(smem_u32(bars + j % RAW_STAGES), (uint32_t)((j / RAW_STAGES) & 1), p.status)) { ok = false; break; }
            }
            const unsigned char *a_hi = smem + (size_t)rs * 2 * TILE, *b_hi = a_hi + TILE;
            unsigned char *a_lo = lo_base + (size_t)lb * 2 * TILE, *b_lo = a_lo + TILE;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t off = (uint32_t)(tid * 16 + h * 8192);
                const float4 va = *reinterpret_cast<const float4 *>(a_hi + off);
                store_lo_at(a_lo, off, va);
                if (OP == OP_WGRAD) bsum[h] += (va.x + va.y) + (va.z + va.w);
                if (off < B_BYTES) {
                    const float4 vb = *reinterpret_cast<const float4 *>(b_hi + off);
                    store_lo_at(b_lo, off, vb);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(full + rs));
            if (c_kb == KB - 1) {
                if (OP == OP_WGRAD) {
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
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace pwt
