// CTA-pair kernel with cluster multicast of the A operand, for single-GPU runs only.
//
// Four consecutive CTAs (two CTA pairs side by side along N) compute a 256 x 512 super-tile.
// Both pairs multiply the same 256 rows of A, so each 128-row slab of A that a CTA needs is
// also needed by the CTA at the same position of the other pair. When the four CTAs were
// launched as one cluster, each of the two loads one 64-row half of that slab with a TMA load
// that delivers it to both CTAs at once: per CTA and k-block 24 KB are read from L2 for the same
// 32 KB of operands landing in shared memory, where the plain pair kernel reads 32 KB
// (hgemm_tcgen05_kernel<256, 6, 2, kModeTiles>).
//
// Only 33 clusters of four fit the 148 SMs of a B200 (GPCs of 18 SMs hold four such clusters and
// leave two SMs over), so the kernel is launched with a regular cluster of 2 and a PREFERRED
// cluster of 4 (cudaLaunchAttributePreferredClusterDimension): the hardware forms clusters of
// four where it can and clusters of two from the rest. The kernel reads its actual cluster size
// at run time; pairs that ended up in a cluster of two load their whole A slab themselves and
// otherwise behave like the plain pair kernel. The tile assignment is the same either way.
//
// This translation unit is the only place in the repository that names a multicast TMA load.
// It is built into a library of its own (libb200_hgemm_mc.so) that the main library loads when
// it is present; runs on two or more GPUs leave both this file and that library behind and use
// the plain pair kernel. All memory the loads read is local to the GPU the kernel runs on.
//
// Everything else follows hgemm_tcgen05_kernel (../gemm_kernel.cuh): same operand layouts, same
// stage ring, tensor-memory double buffering, TMA-store epilogue, bounded waits and error word.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include <mutex>

#include "../gemm_kernel.cuh"
#include "../gemm_kernel_big.cuh"

namespace b200 {

constexpr int kMcStages = 6;
constexpr int kMcClusterCtas = 4;
constexpr uint32_t kMcABytes = 128 * kBK * 2;
constexpr uint32_t kMcBBytes = 128 * kBK * 2;
constexpr uint32_t kMcStageBytes = kMcABytes + kMcBBytes;
constexpr uint32_t kMcTmemCols = 512;
constexpr uint32_t kMcSmemBytes = 1024 + kMcStages * kMcStageBytes + kStagingBytes + 256;

// TMA tile load delivered to every CTA of `cta_mask` at the same shared-memory offset; the
// transaction bytes are counted on the barrier of each destination pair's leader.
__device__ __forceinline__ void tma_load_2d_pair_multicast(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y,
                                                           uint32_t leader_bar, uint16_t cta_mask) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster "
        "[%0], [%1, {%2, %3}], [%4], %5;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(leader_bar), "h"(cta_mask)
        : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) hgemm_tcgen05_mc_kernel(const __grid_constant__ GemmParams p) {
    constexpr int STAGES = kMcStages;
    constexpr uint32_t BN = 256;  // columns per pair

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw_addr);
    const uint32_t staging = base + STAGES * kMcStageBytes;
    uint8_t *staging_ptr = base_ptr + STAGES * kMcStageBytes;
    const uint32_t bars = staging + kStagingBytes;
    uint8_t *bars_ptr = staging_ptr + kStagingBytes;
    const uint32_t full_bar = bars;
    const uint32_t empty_bar = bars + 8u * STAGES;
    const uint32_t tfull_bar = bars + 16u * STAGES;
    const uint32_t tempty_bar = tfull_bar + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_ptr + 16u * STAGES + 32u);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_cta_rank();   // 0..3 in a cluster of four, 0..1 in a cluster of two
    const bool quad = cluster_num_ctas() == 4u;  // all four CTAs of the super-tile share one cluster
    const uint32_t pair = (blockIdx.x >> 1) & 1u;  // which 256-column half of the super-tile
    const uint32_t half = blockIdx.x & 1u;         // which 128 rows of the pair's 256 (= rank & 1)
    const uint32_t worker = blockIdx.x / kMcClusterCtas;
    const uint32_t workers = gridDim.x / kMcClusterCtas;
    const uint32_t k_blocks = p.k_blocks;
    const uint32_t my_tiles = worker < p.tiles ? (p.tiles - worker + workers - 1) / workers : 0u;

    if (warp == 0) {
        if (lane < static_cast<uint32_t>(STAGES)) {
            mbar_init(full_bar + 8u * lane, 1);
            mbar_init(empty_bar + 8u * lane, quad ? 2 : 1);  // in a cluster of four both pairs' MMA issuers release a stage
        } else if (lane < static_cast<uint32_t>(STAGES) + 2u) {
            const uint32_t a = lane - STAGES;
            mbar_init(tfull_bar + 8u * a, 1);
            mbar_init(tempty_bar + 8u * a, 8);  // four epilogue warps of each CTA of the pair
        } else if (lane == static_cast<uint32_t>(STAGES) + 2u) {
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
        tmem_alloc<2>(smem_u32(const_cast<uint32_t *>(tmem_slot)), kMcTmemCols);
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
                // this CTA's 128 rows of A; it fetches the 64-row part `pair` of them for itself and
                // for the CTA at the same position of the other pair, which fetches the other part
                const int32_t row_a0 = static_cast<int32_t>(tc.m_blk * 256u + half * 128u);
                const int32_t row_b = static_cast<int32_t>(tc.n_blk * 512u + pair * BN + half * 128u);
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar + 8u * stage, phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = base + stage * kMcStageBytes;
                    const uint32_t sb = sa + kMcABytes;
                    const int32_t kx = static_cast<int32_t>(kb * kBK);
                    if (half == 0) mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * kMcStageBytes);
                    const uint32_t leader = pair_leader_bar(full_bar + 8u * stage, rank);
                    if (quad) {
                        tma_load_2d_pair_multicast(sa + pair * (kMcABytes / 2), &p.tm_a, kx, row_a0 + static_cast<int32_t>(pair * 64u),
                                                   leader, a_mask);
                    } else {
                        tma_load_2d_pair(sa, &p.tm_a, kx, row_a0, leader);
                        tma_load_2d_pair(sa + kMcABytes / 2, &p.tm_a, kx, row_a0 + 64, leader);
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
                const uint32_t acc = ti & 1u;
                const uint32_t acc_phase = (ti >> 1) & 1u;
                if (!mbar_wait(tempty_bar + 8u * acc, acc_phase ^ 1u, abort_flag)) break;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar + 8u * stage, phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t sa = base + stage * kMcStageBytes;
                    const uint64_t da = umma_smem_desc_sw128(sa);
                    const uint64_t db = umma_smem_desc_sw128(sa + kMcABytes);
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k) {
                        umma_f16<2>(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    // in a cluster of four the CTAs write into each other's A slabs: every one of them
                    // has to learn that this pair is done with the stage
                    umma_commit_pair(empty_bar + 8u * stage, all_mask);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar + 8u * acc, pair_mask);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        const uint32_t q = warp & 3u;
        uint8_t *my_staging_ptr = staging_ptr + q * 8192u;
        const uint32_t my_staging = staging + q * 8192u;
        uint32_t store_buf = 0;
        pdl_wait_prior_grids();
        for (uint32_t ti = 0; ti < my_tiles; ++ti) {
            const uint32_t acc = ti & 1u;
            const uint32_t acc_phase = (ti >> 1) & 1u;
            const TileCoord tc = tile_coord(worker + ti * workers, p.m_blocks, p.n_blocks, p.group_m);
            const uint32_t m0 = tc.m_blk * 256u + half * 128u;
            const uint32_t n0 = tc.n_blk * 512u + pair * BN;
            uint32_t ready = 1;
            if (lane == 0) ready = mbar_wait(tfull_bar + 8u * acc, acc_phase, abort_flag) ? 1u : 0u;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * BN;
            const bool warp_rows_live = (m0 + q * 32u) < p.m;
            constexpr uint32_t kChunks = BN / 64;
            uint32_t ra[64], rb[64];
            tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(ra));
            tmem_ld_32x32b_x32(taddr + 32u, *reinterpret_cast<uint32_t(*)[32]>(ra + 32));
#pragma unroll
            for (uint32_t c = 0; c < kChunks; ++c) {
                uint32_t *cur = (c & 1u) ? rb : ra;
                uint32_t *nxt = (c & 1u) ? ra : rb;
                tmem_ld_wait();
                if (c + 1 < kChunks) {
                    tmem_ld_32x32b_x32(taddr + (c + 1) * 64u, *reinterpret_cast<uint32_t(*)[32]>(nxt));
                    tmem_ld_32x32b_x32(taddr + (c + 1) * 64u + 32u, *reinterpret_cast<uint32_t(*)[32]>(nxt + 32));
                } else {
                    // the accumulator is in registers: hand it back to the pair's MMA issuer
                    tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar + 8u * acc, quad ? pair * 2u : 0u));
                }
                const bool live = warp_rows_live && (n0 + c * 64u) < p.n;
                if (live) {
                    uint8_t *buf = my_staging_ptr + (store_buf & 1u) * 4096u;
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    uint8_t *row_ptr = buf + lane * 128u;
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        uint4 v;
                        v.x = pack_half2_rn(cur[8 * j + 0], cur[8 * j + 1]);
                        v.y = pack_half2_rn(cur[8 * j + 2], cur[8 * j + 3]);
                        v.z = pack_half2_rn(cur[8 * j + 4], cur[8 * j + 5]);
                        v.w = pack_half2_rn(cur[8 * j + 6], cur[8 * j + 7]);
                        *reinterpret_cast<uint4 *>(row_ptr + ((j ^ (lane & 7u)) << 4)) = v;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&p.tm_c, my_staging + (store_buf & 1u) * 4096u, static_cast<int32_t>(n0 + c * 64u),
                                     static_cast<int32_t>(m0 + q * 32u));
                        tma_store_commit();
                    }
                    ++store_buf;
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
        tmem_dealloc<2>(tmem_base, kMcTmemCols);
    }
}


// ------------------------------------------------------------------------------------------
// 512 x 512 super-tiles: 256 x 256 outputs per CTA
// ------------------------------------------------------------------------------------------
// The kernel body is hgemm_big_body (../gemm_kernel_big.cuh) for groups of four CTAs; this file
// adds the one thing that header may not contain, the multicast load of the A slab halves.
struct PairMulticastLoad {
    static __device__ __forceinline__ void load(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y, uint32_t leader_bar,
                                                uint16_t cta_mask) {
        tma_load_2d_pair_multicast(smem_dst, tm, x, y, leader_bar, cta_mask);
    }
};

__global__ void __launch_bounds__(kBigThreads, 1) hgemm_tcgen05_mc512_kernel(const __grid_constant__ GemmParams p) {
    hgemm_big_body<4, PairMulticastLoad>(p);
}

}  // namespace b200

using namespace b200;

namespace {
std::mutex g_mu;
bool g_attr_set[2][64] = {};
int g_max_clusters[64] = {};

// Launches one of the two kernels: groups of four CTAs, a regular cluster of 2 and a preferred
// cluster of 4, at most one group per four SMs.
int launch_groups(void (*kern)(const GemmParams), int which, uint32_t smem_bytes, uint32_t threads, const GemmParams &p,
                  void *stream, int use_pdl) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -5;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_attr_set[which][dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -5;
            g_attr_set[which][dev] = true;
        }
        if (g_max_clusters[dev] == 0) {
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < kMcClusterCtas) return -5;
            g_max_clusters[dev] = sms / kMcClusterCtas;  // groups of four CTAs, one CTA per SM
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attrs[3];
    int n_attrs = 0;
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;  // what the hardware may fall back to
    attrs[n_attrs].val.clusterDim.x = 2;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
    attrs[n_attrs].id = cudaLaunchAttributePreferredClusterDimension;  // what it forms where four SMs are free
    attrs[n_attrs].val.preferredClusterDim.x = kMcClusterCtas;
    attrs[n_attrs].val.preferredClusterDim.y = 1;
    attrs[n_attrs].val.preferredClusterDim.z = 1;
    ++n_attrs;
    if (use_pdl) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;
    uint32_t groups = static_cast<uint32_t>(g_max_clusters[dev]);
    if (groups > p.tiles) groups = p.tiles;
    cfg.gridDim = dim3(groups * kMcClusterCtas, 1, 1);
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
        cudaGetLastError();
        return -5;
    }
    return 0;
}
}  // namespace

// Launches the 256 x 512 multicast kernel on `stream`. `params` is a b200::GemmParams whose tensor
// maps use boxes of 64 rows (A), 128 rows (B) and 32 rows (C), with m_blocks / n_blocks / tiles
// counted in 256 x 512 super-tiles. Returns 0, or -5 when a CUDA call fails.
extern "C" int b200_mc_launch(const void *params, void *stream, int use_pdl) {
    return launch_groups(hgemm_tcgen05_mc_kernel, 0, kMcSmemBytes, kThreads, *static_cast<const GemmParams *>(params), stream,
                         use_pdl);
}

// Launches the 512 x 512 multicast kernel: boxes of 128 rows (A), 128 rows (B) and 32 rows (C);
// m_blocks / n_blocks / tiles counted in 512 x 512 super-tiles.
extern "C" int b200_mc512_launch(const void *params, void *stream, int use_pdl) {
    return launch_groups(hgemm_tcgen05_mc512_kernel, 1, kBigSmemBytes, kBigThreads, *static_cast<const GemmParams *>(params),
                         stream, use_pdl);
}

// How many groups of four CTAs a launch uses on this device (0 before the first launch on it).
extern "C" int b200_mc_resident_clusters(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return g_max_clusters[dev];
}
