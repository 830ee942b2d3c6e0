// CTA-pair kernel with 256 x 256 outputs per CTA, for large problems.
//
// A pair of CTAs (one 2-CTA cluster) computes a 512 x 256 tile: each CTA owns 256 rows of A and
// the whole of its tensor memory, two 128 x 256 FP32 accumulators, one per 128-row part of its
// slab, fed by two UMMA groups per k-block that share the pair's 256 columns of B (each CTA
// stages 128 of them). Per k-block a CTA reads 384 rows of operands from L2 for 256 x 256
// outputs, where the 128 x 256 arrangement of hgemm_tcgen05_kernel<256, 6, 2> reads 256 rows for
// half as many outputs: 0.75 of the L2-to-SM bytes per output, and a wave of tiles that is
// closer to square, so fewer DRAM bytes per wave as well. On a power-capped part the bytes
// moved decide the clock the tensor cores get.
//
// The price is that nothing is left of tensor memory for a second set of accumulators: the MMA
// issuer waits for the epilogue to drain a tile before it starts the next (the producer keeps
// loading ahead meanwhile). Eight epilogue warps, one per (lane quarter, accumulator), keep that
// drain short. Shared memory: 4 stages of 48 KB and one 4 KB staging buffer per epilogue warp.
//
// GROUP = 4 runs two such pairs side by side on a 512 x 512 tile. When the hardware put the four
// CTAs into one cluster, each CTA fetches only half of its A slab and delivers it to the CTA at
// the same position of the other pair as well (MulticastLoad, supplied by the translation unit
// that instantiates this; none is needed for GROUP = 2): 256 rows from L2 per k-block, half the
// bytes per output of the 128 x 256 arrangement.
//
// Operand layouts, swizzle, barriers, bounded waits and the error word are those of
// hgemm_tcgen05_kernel (gemm_kernel.cuh).
#pragma once

#include "gemm_kernel.cuh"

namespace b200 {

constexpr int kBigStages = 4;
constexpr int kBigThreads = 320;  // producer, MMA issuer, eight epilogue warps
constexpr uint32_t kBigABytes = 256 * kBK * 2;
constexpr uint32_t kBigBBytes = 128 * kBK * 2;
constexpr uint32_t kBigStageBytes = kBigABytes + kBigBBytes;
constexpr uint32_t kBigStagingBytes = 8u * 4096u;
constexpr uint32_t kBigTmemCols = 512;
constexpr uint32_t kBigSmemBytes = 1024 + kBigStages * kBigStageBytes + kBigStagingBytes + 256;
static_assert(kBigSmemBytes <= 232448, "over the 227 KB a CTA can have");

// The barrier of the pair's leader CTA (the even rank of the pair), as seen from either CTA of the pair.
__device__ __forceinline__ uint32_t pair_leader_bar(uint32_t local_bar, uint32_t cluster_rank) {
    return map_to_cta(local_bar, cluster_rank & ~1u);
}

// Stands in for MulticastLoad where no group of four exists.
struct NoMulticastLoad {
    static __device__ __forceinline__ void load(uint32_t, const CUtensorMap *, int32_t, int32_t, uint32_t, uint16_t) {}
};

// EPI: apply GemmParams' alpha / beta / bias to each 16-column chunk as it leaves tensor memory and pack C as
// FP16 or BF16 (GemmParams::c_type).
template <int GROUP, class MulticastLoad, bool EPI = false>
__device__ __forceinline__ void hgemm_big_body(const GemmParams &p) {
    static_assert(GROUP == 2 || GROUP == 4, "a work group is one CTA pair or two");
    constexpr int STAGES = kBigStages;
    constexpr uint32_t BN = 256;              // columns per pair
    constexpr uint32_t kTileN = GROUP * 128u;  // columns per work group

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw_addr);
    const uint32_t staging = base + STAGES * kBigStageBytes;
    uint8_t *staging_ptr = base_ptr + STAGES * kBigStageBytes;
    const uint32_t bars = staging + kBigStagingBytes;
    uint8_t *bars_ptr = staging_ptr + kBigStagingBytes;
    const uint32_t full_bar = bars;
    const uint32_t empty_bar = bars + 8u * STAGES;
    const uint32_t tfull_bar = bars + 16u * STAGES;
    const uint32_t tempty_bar = tfull_bar + 8u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_ptr + 16u * STAGES + 16u);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_cta_rank();
    // all four CTAs of a group of four share one cluster (else: clusters of two, no multicast)
    const bool quad = GROUP == 4 && cluster_num_ctas() == 4u;
    const uint32_t pair = GROUP == 4 ? (blockIdx.x >> 1) & 1u : 0u;  // which 256-column part of the group's tile
    const uint32_t half = blockIdx.x & 1u;         // which 256 rows of the super-tile's 512
    const uint32_t worker = blockIdx.x / GROUP;
    const uint32_t workers = gridDim.x / GROUP;
    const uint32_t k_blocks = p.k_blocks;
    const uint32_t my_tiles = worker < p.tiles ? (p.tiles - worker + workers - 1) / workers : 0u;

    if (warp == 0) {
        if (lane < static_cast<uint32_t>(STAGES)) {
            mbar_init(full_bar + 8u * lane, 1);
            mbar_init(empty_bar + 8u * lane, quad ? 2 : 1);
        } else if (lane == static_cast<uint32_t>(STAGES)) {
            mbar_init(tfull_bar, 1);
            mbar_init(tempty_bar, 16);  // eight epilogue warps of each CTA of the pair
        } else if (lane == static_cast<uint32_t>(STAGES) + 1u) {
            *abort_flag = 0;
        }
        fence_mbar_init();
        __syncwarp();
    }
    if (warp == 2 && lane == 0) {
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_b);
        tma_prefetch_desc(&p.tm_c);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t *>(tmem_slot)), kBigTmemCols);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint16_t a_mask = static_cast<uint16_t>((1u << rank) | (1u << (rank ^ 2u)));  // cluster of four only
            pdl_wait_prior_grids();
            for (uint32_t ti = 0; ok && ti < my_tiles; ++ti) {
                const TileCoord tc = tile_coord(worker + ti * workers, p.m_blocks, p.n_blocks, p.group_m);
                const int32_t row_a0 = static_cast<int32_t>(tc.m_blk * 512u + half * 256u);
                const int32_t row_b = static_cast<int32_t>(tc.n_blk * kTileN + pair * BN + half * 128u);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar + 8u * stage, phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = base + stage * kBigStageBytes;
                    const uint32_t sb = sa + kBigABytes;
                    const int32_t kx = static_cast<int32_t>(kb * kBK);
                    if (half == 0) mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * kBigStageBytes);
                    const uint32_t leader = pair_leader_bar(full_bar + 8u * stage, rank);
                    if (quad) {
                        // rows [pair * 128, +128) of the slab, for this CTA and its twin in the other pair
                        MulticastLoad::load(sa + pair * (kBigABytes / 2), &p.tm_a, kx, row_a0 + static_cast<int32_t>(pair * 128u), leader,
                                            a_mask);
                    } else {
                        tma_load_2d_pair(sa, &p.tm_a, kx, row_a0, leader);
                        tma_load_2d_pair(sa + kBigABytes / 2, &p.tm_a, kx, row_a0 + 128, leader);
                    }
                    tma_load_2d_pair(sb, &p.tm_b, kx, row_b, leader);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (pair leaders)
        if (lane == 0 && half == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(256, BN);
            const uint16_t pair_mask = static_cast<uint16_t>(quad ? (0x3u << (2u * pair)) : 0x3u);
            const uint16_t all_mask = static_cast<uint16_t>(quad ? 0xFu : 0x3u);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t ti = 0; ok && ti < my_tiles; ++ti) {
                // both accumulators are in use until the epilogue warps of both CTAs have read them out
                if (!mbar_wait(tempty_bar, (ti & 1u) ^ 1u, abort_flag)) break;
                tcgen05_fence_after_sync();
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar + 8u * stage, phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t sa = base + stage * kBigStageBytes;
                    const uint64_t da0 = umma_smem_desc_sw128(sa);
                    const uint64_t da1 = umma_smem_desc_sw128(sa + kBigABytes / 2);
                    const uint64_t db = umma_smem_desc_sw128(sa + kBigABytes);
                    const uint32_t accumulate = kb > 0 ? 1u : 0u;
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k) {
                        umma_f16<2>(tmem_base, da0 + 2u * k, db + 2u * k, idesc, (accumulate | k) ? 1u : 0u);
                        umma_f16<2>(tmem_base + BN, da1 + 2u * k, db + 2u * k, idesc, (accumulate | k) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar + 8u * stage, all_mask);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar, pair_mask);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        // warp w may read tensor-memory lanes 32 * (w % 4) ..; warps 2-5 take accumulator 0
        // (rows 0-127 of the CTA's slab), warps 6-9 accumulator 1 (rows 128-255)
        const uint32_t q = warp & 3u;
        const uint32_t sub = (warp - 2u) >> 2;
        uint8_t *my_staging_ptr = staging_ptr + (warp - 2u) * 4096u;
        const uint32_t my_staging = staging + (warp - 2u) * 4096u;
        pdl_wait_prior_grids();
        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            const TileCoord tc = tile_coord(worker + ti * workers, p.m_blocks, p.n_blocks, p.group_m);
            const uint32_t m0 = tc.m_blk * 512u + half * 256u + sub * 128u;
            const uint32_t n0 = tc.n_blk * kTileN + pair * BN;
            uint32_t ready = 1;
            if (lane == 0) ready = mbar_wait(tfull_bar, ti & 1u, abort_flag) ? 1u : 0u;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + sub * BN;
            const bool warp_rows_live = (m0 + q * 32u) < p.m;
            // Drain first, store afterwards: the 32 x 256 FP32 values of this warp are read out in
            // sixteen 16-column loads (two in flight) and kept as 128 registers of packed halves, so
            // that tensor memory goes back to the MMA issuer before any store has to be waited for.
            // (Ten warps are allocated registers as twelve: 168 per thread is all there is.)
            uint32_t packed[BN / 2];
            uint32_t fa[16], fb[16];
            tmem_ld_32x32b_x16(taddr, fa);
#pragma unroll
            for (uint32_t s = 0; s < BN / 16; ++s) {
                uint32_t *cur = (s & 1u) ? fb : fa;
                tmem_ld_wait();
                if (s + 1 < BN / 16) {
                    tmem_ld_32x32b_x16(taddr + (s + 1) * 16u, (s & 1u) ? fa : fb);
                } else {
                    // this warp's part of the tile is in registers: tell the pair's MMA issuer
                    tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar, quad ? pair * 2u : 0u));
                }
                if (EPI) {
                    if (warp_rows_live) fused_epilogue<16>(p, m0 + q * 32u + lane, n0 + s * 16u, cur);
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) packed[s * 8 + j] = pack2_rn(cur[2 * j], cur[2 * j + 1], p.c_type);
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) packed[s * 8 + j] = pack_half2_rn(cur[2 * j], cur[2 * j + 1]);
                }
            }
#pragma unroll
            for (uint32_t c = 0; c < BN / 64; ++c) {
                const bool live = warp_rows_live && (n0 + c * 64u) < p.n;
                if (live) {
                    if (lane == 0) tma_store_wait_read<0>();  // one staging buffer per warp
                    __syncwarp();
                    uint8_t *row_ptr = my_staging_ptr + lane * 128u;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        uint4 v;
                        v.x = packed[c * 32 + 4 * j + 0];
                        v.y = packed[c * 32 + 4 * j + 1];
                        v.z = packed[c * 32 + 4 * j + 2];
                        v.w = packed[c * 32 + 4 * j + 3];
                        *reinterpret_cast<uint4 *>(row_ptr + ((j ^ (lane & 7u)) << 4)) = v;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&p.tm_c, my_staging, static_cast<int32_t>(n0 + c * 64u), static_cast<int32_t>(m0 + q * 32u));
                        tma_store_commit();
                    }
                }
            }
        }
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
        if (threadIdx.x == 0) atomicExch(p.error_word, static_cast<uint32_t>(kDevWaitTimeout));
        __syncthreads();
    }
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<2>(tmem_base, kBigTmemCols);
    }
}

}  // namespace b200
