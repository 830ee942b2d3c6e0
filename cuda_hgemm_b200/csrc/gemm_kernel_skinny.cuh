// Kernel for a short A (M <= 128 rows): the weight matrix B streams through the MMA's row operand.
//
// C[M x N] = A[M x K] * B^T with M of a decode batch (16 ... 64 rows) is bound by reading B once from
// HBM. hgemm_tcgen05_kernel puts A on the 128 rows of the MMA, so every k-block stages a 16 KB slab of
// A that is mostly padding next to 16 KB of B, six stages deep, and the thread that issues the MMAs
// needs about 0.28 us per k-block for its own instructions (a barrier test, four MMAs, a commit):
// 112 CTAs x 16 KB / 0.28 us is 6.4 TB/s, the HBM rate itself.
//
// Here the operands are swapped: 128 rows of B are the MMA's row operand, the MT >= M rows of A its
// column operand (UMMA 128 x MT x 16), and the accumulator holds C transposed: tensor-memory lane = column
// of C, tensor-memory column = row of C. A stage is two k-blocks (32 KB of B and 2 x MT x 128 B of A)
// under one barrier round trip, six stages deep for MT = 16: twice the bytes of B in flight per SM and
// 0.20 us of issue time per k-block. One CTA computes one (column tile, k-range) pair; when the tiles
// are too few to fill the GPU (N = 4096: 32) the k-range is cut into equal slices. Their FP32 partial
// results are summed either inside a thread-block cluster that holds the k-ranges of one tile (template
// parameter CK below: no workspace, no second kernel) or, for more k-ranges than a cluster takes, through a
// workspace by skinny_reduce_kernel, which follows in the stream; both give the same bits.
//
// A column tile is tile_w <= 128 columns of C wide (a multiple of 8): the TMA box of B has tile_w rows,
// the MMA still multiplies 128 rows of the stage's slab, and whatever lies in the rows the box did not
// write only reaches tensor-memory lanes that are never read. The launcher picks the width that spreads
// N over the SMs best: N = 14336 gives 112 tiles of 128 columns on 148 SMs, but 138 tiles of 104.
//
// CG = 2 runs a pair of CTAs (cta_group::2) on two neighbouring column tiles: every CTA stages its own
// tile_w rows of B but only half of the rows of A, the leader issues MMAs of 256 x MT for both, and the
// rows of A cross from L2 to an SM once per pair instead of once per CTA. With 65 ... 128 rows of A
// that traffic is as large as B's own (a 16 KB slab of A beside at most 16 KB of B per k-block) and, not
// HBM, bounds the single-CTA form; the pair form also leaves room for a deeper ring.
//
// The epilogue turns the accumulator (lane = column of C) back into rows of C in shared memory (the
// ring's first stage: every MMA has retired by then) and writes the tile with one TMA store; when C
// cannot have a tensor map (N % 8 != 0) or when FP32 partials are wanted it stores by element.
//
// Operand layouts, swizzle, bounded waits and the error word are those of hgemm_tcgen05_kernel
// (gemm_kernel.cuh); the reference has no counterpart (its kernels tile every shape alike,
// src/mma/mma_async_stage4.cu:54-70).
#pragma once

#include "gemm_kernel.cuh"

namespace b200 {

struct alignas(64) SkinnyParams {
    CUtensorMap tm_w;  // B as {K, N}, box {64, tile_w}, 128-byte swizzle
    CUtensorMap tm_x;  // A as {K, M}, box {64, MT / CG}, 128-byte swizzle
    CUtensorMap tm_c;  // C as {N, M}, box {tile_w, MT}, no swizzle (only valid when tma_store != 0)
    __half *c;
    float *partials;  // slices x MT x n_pad FP32, used when slices > 1
    uint32_t *error_word;
    uint32_t m, n, k;
    uint32_t k_blocks;
    uint32_t n_tiles;        // column tiles of C (even for pairs: a tile past N reads zeros and stores nothing)
    uint32_t tile_w;         // columns of C per tile: a multiple of 8, at most 128 (= rows of the TMA box of B)
    uint32_t slices;         // k-ranges per tile
    uint32_t kb_per_slice;   // k-blocks per k-range (the last one may be shorter, never empty)
    uint32_t n_pad;          // row pitch of the partial results, in floats
    uint32_t tma_store;      // 1: whole results leave through tm_c
    uint32_t prefetch_kb;    // k-blocks of B asked into L2 before waiting for the previous kernel
    EpilogueArgs epi;        // kernels instantiated with EPI: alpha / beta / bias / c_in and the element type of C
#ifdef B200_TIMELINE
    unsigned long long *timeline;  // profiling builds only: 32 words per CTA (see GemmParams::timeline)
#endif
};

template <int MT, int STAGES, int KPS, int CG = 1>
struct SkinnyTraits {
    static_assert(MT == 16 || MT == 32 || MT == 64 || MT == 128, "rows of A per tile");
    static_assert(KPS == 1 || KPS == 2, "k-blocks per stage");
    static_assert(CG == 1 || CG == 2, "single CTAs or CTA pairs");
    static constexpr uint32_t kWBytes = 128 * kBK * 2;
    static constexpr uint32_t kXRows = MT / CG;  // rows of A this CTA stages
    static constexpr uint32_t kXBytes = kXRows * kBK * 2;
    static constexpr uint32_t kBlockBytes = kWBytes + kXBytes;
    static constexpr uint32_t kStageBytes = KPS * kBlockBytes;
    static constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;
    static constexpr uint32_t kSmemBytes = 1024 + STAGES * kStageBytes + 256;
    static_assert((kBlockBytes % 1024) == 0, "operand slabs must keep 1024-byte alignment");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KB of shared memory");
    static_assert((2 * STAGES + 1) * 8 + 16 <= 256, "barrier area too small");
    static_assert(STAGES * kStageBytes >= MT * 128 * 2, "the ring must hold one tile of C for the epilogue");
};

// EPI: whole results get alpha * acc + beta * c_in + bias before their one rounding and leave in epi.c_type
// (FP32 partials of cut k-ranges are left as they are: skinny_reduce_kernel applies the same to their sum).
//
// CK: the k-ranges of one column tile (p.slices of them, at least two) run as one thread-block cluster and sum
// their partial results on chip. CTA `s` of the cluster owns rows [s * rows_per, (s + 1) * rows_per) of the
// tile. Every CTA first turns its accumulator into rows of C (FP32) in its own ring; when all CTAs of the cluster
// have done so (cluster barrier: every MMA has retired, every ring is free) it sends each owner that owner's
// rows with one bulk copy from shared memory to shared memory, counted on a barrier of the owner; the owner
// then adds the k-ranges in order -- the order and the arithmetic of skinny_reduce_kernel, so both forms give
// the same bits -- and stores its rows of C. No workspace, no second kernel. With CG = 2 the cluster holds
// p.slices pairs: rank = 2 * k-range + position in the pair.
template <int MT, int STAGES, int KPS, int CG = 1, bool EPI = false, bool CK = false>
__global__ void __launch_bounds__(kThreads, 1) hgemm_skinny_kernel(const __grid_constant__ SkinnyParams p) {
    using T = SkinnyTraits<MT, STAGES, KPS, CG>;
    static_assert(!CK || STAGES * T::kStageBytes >= (2 * MT + 8) * 128 * 4, "the ring must hold the accumulator and the other k-ranges' rows");
    static_assert(16 * STAGES + 24 <= 256 && STAGES + 3 <= 32, "barrier area too small");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw_addr);
    const uint32_t bars = base + STAGES * T::kStageBytes;
    uint8_t *bars_ptr = base_ptr + STAGES * T::kStageBytes;
    const uint32_t full_bar = bars;
    const uint32_t empty_bar = bars + 8u * STAGES;
    const uint32_t tfull_bar = bars + 16u * STAGES;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_ptr + 16u * STAGES + 8u);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t inbox_bar = bars + 16u * STAGES + 16u;  // CK: counts the bytes the other k-ranges send to this CTA

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    // position in the cluster, position in the pair, and the pair's leader (the even rank)
    const uint32_t cluster_rank = (CG == 2 || CK) ? cluster_cta_rank() : 0u;
    const uint32_t cta_rank = (CG == 2) ? (cluster_rank & 1u) : 0u;
    const uint32_t leader_rank = cluster_rank & ~1u;
    // consecutive CTAs take consecutive column tiles (the two CTAs of a pair: tiles 2i and 2i + 1 of one k-range);
    // with CK consecutive clusters do, and the CTAs (pairs) of a cluster take the k-ranges of one tile (pair of tiles)
    const uint32_t tile = CK ? (blockIdx.x / (p.slices * CG)) * CG + cta_rank : blockIdx.x % p.n_tiles;
    const uint32_t slice = CK ? cluster_rank / CG : blockIdx.x / p.n_tiles;
    const uint32_t kb0 = slice * p.kb_per_slice;
    const uint32_t kb1 = min(p.k_blocks, kb0 + p.kb_per_slice);
    const uint32_t n0 = tile * p.tile_w;

    if (threadIdx.x == 0) B200_STAMP(0);
    if (warp == 0) {
        if (lane < static_cast<uint32_t>(STAGES)) {
            mbar_init(full_bar + 8u * lane, 1);
            mbar_init(empty_bar + 8u * lane, 1);
        } else if (lane == static_cast<uint32_t>(STAGES)) {
            mbar_init(tfull_bar, 1);
        } else if (lane == static_cast<uint32_t>(STAGES) + 1u) {
            *abort_flag = 0;
        } else if (CK && lane == static_cast<uint32_t>(STAGES) + 2u) {
            mbar_init(inbox_bar, 1);
        }
        fence_mbar_init();
        __syncwarp();
    }
    if (warp == 2 && lane == 0) {
        tma_prefetch_desc(&p.tm_w);
        tma_prefetch_desc(&p.tm_x);
        if (p.tma_store) tma_prefetch_desc(&p.tm_c);
    }
    if (warp == 1) {
        tmem_alloc<CG>(smem_u32(const_cast<uint32_t *>(tmem_slot)), T::kTmemCols);
        tmem_relinquish<CG>();
    }
    tcgen05_fence_before_sync();
    if (CG == 2) {
        // the peer's copies and arrivals target this CTA's barriers: both CTAs must have set up
        __syncthreads();
        cluster_sync_all();
    } else {
        // The producer warp initialised the barriers itself and needs no tensor memory: it only
        // announces its arrival and starts loading while the allocation completes.
        if (warp == 0) {
            __threadfence_block();
            named_bar_arrive(2, kThreads);
        } else {
            named_bar_sync(2, kThreads);
        }
    }
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = (CG == 1 && warp == 0) ? 0u : *tmem_slot;
    pdl_launch_dependents();
    if (threadIdx.x == 0) B200_STAMP(1);
    uint32_t ready = 1;  // epilogue warps: the accumulator is complete

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            const uint32_t block_tx = p.tile_w * kBK * 2u + T::kXBytes;  // bytes one CTA stages per k-block
            const int32_t row_x = static_cast<int32_t>(cta_rank * T::kXRows);
            // While the previous kernel in the stream finishes, ask L2 for the first k-blocks of this tile's
            // rows of B: the kernel is bound by HBM and the previous one's last CTAs leave it idle. Only a
            // hint -- nothing is read into the SM before the wait below.
            for (uint32_t kb = kb0; kb < kb1 && kb < kb0 + p.prefetch_kb; ++kb) {
                tma_prefetch_l2_2d(&p.tm_w, static_cast<int32_t>(kb * kBK), static_cast<int32_t>(n0));
            }
            pdl_wait_prior_grids();  // A and B may have been written by the previous kernel
            B200_STAMP(2);
            for (uint32_t kb = kb0; kb < kb1; kb += KPS) {
                if (!mbar_wait(empty_bar + 8u * stage, phase ^ 1u, abort_flag)) break;
                const uint32_t slot = base + stage * T::kStageBytes;
                // a k-block past the end of this k-range is not loaded; its share of the stage is not waited for
                const uint32_t blocks = min(static_cast<uint32_t>(KPS), kb1 - kb);
                if (CG == 1) {
                    mbar_arrive_expect_tx(full_bar + 8u * stage, blocks * block_tx);
                    for (uint32_t j = 0; j < blocks; ++j) {
                        const uint32_t sw = slot + j * T::kBlockBytes;
                        const int32_t kx = static_cast<int32_t>((kb + j) * kBK);
                        tma_load_2d(sw, &p.tm_w, kx, static_cast<int32_t>(n0), full_bar + 8u * stage);
                        tma_load_2d(sw + T::kWBytes, &p.tm_x, kx, 0, full_bar + 8u * stage);
                    }
                } else {
                    // both CTAs' copies complete on the leader's barrier; the leader posts the byte count of the pair
                    if (cta_rank == 0) mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * blocks * block_tx);
                    const uint32_t leader_bar = map_to_cta(full_bar + 8u * stage, leader_rank);
                    for (uint32_t j = 0; j < blocks; ++j) {
                        const uint32_t sw = slot + j * T::kBlockBytes;
                        const int32_t kx = static_cast<int32_t>((kb + j) * kBK);
                        tma_load_2d_pair(sw, &p.tm_w, kx, static_cast<int32_t>(n0), leader_bar);
                        tma_load_2d_pair(sw + T::kWBytes, &p.tm_x, kx, row_x, leader_bar);
                    }
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            B200_STAMP(3);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(128 * CG, MT);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb0; kb < kb1; kb += KPS) {
                if (!mbar_wait(full_bar + 8u * stage, phase, abort_flag)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after_sync();
#ifdef B200_TIMELINE
                if (kb == kb0) B200_STAMP(4);
#endif
                const uint32_t slot = base + stage * T::kStageBytes;
                const uint32_t blocks = min(static_cast<uint32_t>(KPS), kb1 - kb);
                for (uint32_t j = 0; j < blocks; ++j) {
                    const uint64_t dw = umma_smem_desc_sw128(slot + j * T::kBlockBytes);
                    const uint64_t dx = umma_smem_desc_sw128(slot + j * T::kBlockBytes + T::kWBytes);
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k) {
                        umma_f16<CG>(tmem_base, dw + 2u * k, dx + 2u * k, idesc, (kb > kb0 || j > 0 || k > 0) ? 1u : 0u);
                    }
                }
                if (CG == 1) {
                    umma_commit(empty_bar + 8u * stage);
                } else {
                    umma_commit_pair(empty_bar + 8u * stage, static_cast<uint16_t>(0x3u << leader_rank));
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok) {
                if (CG == 1) {
                    umma_commit(tfull_bar);
                } else {
                    umma_commit_pair(tfull_bar, static_cast<uint16_t>(0x3u << leader_rank));
                }
            }
            B200_STAMP(5);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        // lane of tensor memory = column of C (n), column of tensor memory = row of C (m)
        const uint32_t q = warp & 3u;
        const uint32_t col_in_tile = q * 32u + lane;
        const uint32_t n = n0 + col_in_tile;
        const bool col_live = n < p.n && col_in_tile < p.tile_w;
        const bool staged = p.slices == 1 && p.tma_store != 0;  // whole results, through shared memory and one TMA store
        pdl_wait_prior_grids();  // C (or the workspace) may still be read by the previous kernel
        if (lane == 0) ready = mbar_wait(tfull_bar, 0, abort_flag) ? 1u : 0u;
        ready = __shfl_sync(0xffffffffu, ready, 0);
        if (ready && !CK) {
            tcgen05_fence_after_sync();
            if (threadIdx.x == 64) B200_STAMP(6);
            const uint32_t taddr = tmem_base + ((q * 32u) << 16);
            // every MMA has retired and with it every read of the ring: its first bytes now hold the tile of C,
            // row-major [MT][tile_w] halves
            __half *tile_c = reinterpret_cast<__half *>(base_ptr);
#pragma unroll
            for (uint32_t c = 0; c < MT / 16; ++c) {
                uint32_t r[16];
                tmem_ld_32x32b_x16(taddr + c * 16u, r);
                tmem_ld_wait();
                if (staged) {
                    if (col_in_tile < p.tile_w) {
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            // 32 lanes write 32 consecutive halves of one row of the tile
                            const uint32_t m = c * 16u + j;
                            float v = __uint_as_float(r[j]);
                            if (EPI) {
                                if (m < p.m && n < p.n) v = fused_value(p.epi, v, m, n, p.n);
                                store_c_elem(tile_c, m * p.tile_w + col_in_tile, v, p.epi.c_type);  // FP16 or BF16 here
                            } else {
                                tile_c[m * p.tile_w + col_in_tile] = __float2half_rn(v);
                            }
                        }
                    }
                } else if (col_live) {
                    if (p.slices == 1) {
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            const uint32_t m = c * 16u + j;
                            // 32 lanes write 32 consecutive elements of one row of C
                            if (m < p.m) {
                                if (EPI) {
                                    store_c_elem(p.c, static_cast<size_t>(m) * p.n + n,
                                                 fused_value(p.epi, __uint_as_float(r[j]), m, n, p.n), p.epi.c_type);
                                } else {
                                    p.c[static_cast<size_t>(m) * p.n + n] = __float2half_rn(__uint_as_float(r[j]));
                                }
                            }
                        }
                    } else {
                        float *ws = p.partials + static_cast<size_t>(slice) * MT * p.n_pad;
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            const uint32_t m = c * 16u + j;
                            if (m < p.m) ws[static_cast<size_t>(m) * p.n_pad + n] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
        }
        if (staged) {
            // all four warps have written their columns (a warp that gave up still arrives): one TMA store
            // of tile_w x MT; rows past M and columns past N are clipped by the tensor map
            fence_proxy_async_smem();
            named_bar_sync(3, kEpiThreads);
            if (threadIdx.x == 64 && ready && *abort_flag == 0 && n0 < p.n) {
                tma_store_2d(&p.tm_c, base, static_cast<int32_t>(n0), 0);
                tma_store_commit();
                tma_store_wait_read<0>();
            }
        }
        if (threadIdx.x == 64) B200_STAMP(8);
    }

    if (CK) {
        // ------------------------------------------------------------------ sum of the k-ranges inside the cluster
        // Every thread of the cluster passes both cluster barriers, whatever its warp did before (a CTA whose
        // wait expired still arrives; its error word is set below and the result is not to be used).
        const uint32_t rows_per = (p.m + p.slices - 1u) / p.slices;  // rows of C per owner
        const uint32_t m0 = slice * rows_per;                        // this CTA owns rows [m0, m0 + my_rows)
        const uint32_t my_rows = m0 < p.m ? min(rows_per, p.m - m0) : 0u;
        const uint32_t col_in_tile = ((warp & 3u) << 5) + lane;
        // The ring is free once this CTA's MMAs have retired. Its first MT x 128 floats take this CTA's accumulator
        // as rows of C ([row][128 columns]: an owner's rows are one contiguous block); behind them the rows this
        // CTA owns arrive from the other k-ranges ([k-range][rows_per][128]).
        const uint32_t staging = base;
        const uint32_t inbox = base + MT * 512u;
        const float *staging_f = reinterpret_cast<const float *>(base_ptr);
        if (warp >= 2) {
            if (ready) {
                tcgen05_fence_after_sync();
                if (threadIdx.x == 64) B200_STAMP(6);
                const uint32_t taddr = tmem_base + (((warp & 3u) * 32u) << 16);
#pragma unroll
                for (uint32_t c = 0; c < MT / 16; ++c) {
                    if (c * 16u < p.m) {  // uniform over the CTA
                        uint32_t r[16];
                        tmem_ld_32x32b_x16(taddr + c * 16u, r);
                        tmem_ld_wait();
                        float *row = reinterpret_cast<float *>(base_ptr) + c * 16u * 128u + col_in_tile;
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) row[j * 128u] = __uint_as_float(r[j]);  // 32 lanes: 128 consecutive bytes
                    }
                }
                fence_proxy_async_smem();  // the bulk copies below read what the threads wrote
            }
            if (threadIdx.x == 64 && my_rows > 0) mbar_arrive_expect_tx(inbox_bar, (p.slices - 1u) * my_rows * 512u);
        }
        cluster_sync_all();  // every CTA of the cluster has staged its accumulator: every ring is free to receive
        if (warp == 2 && ready) {
            // lane 4 * o + q sends the q-th quarter of owner o's rows: more copies in flight than one per owner
            const uint32_t o = lane >> 2, quarter = lane & 3u;
            const uint32_t first = o * rows_per;
            if (o < p.slices && o != slice && first < p.m) {
                const uint32_t bytes = min(rows_per, p.m - first) * 128u;  // a quarter of the rows' 512 bytes each
                const uint32_t to = o * CG + cta_rank;
                bulk_copy_to_cluster(map_to_cta(inbox + slice * rows_per * 512u + quarter * bytes, to),
                                     staging + first * 512u + quarter * bytes, bytes, map_to_cta(inbox_bar, to));
            }
        }
        uint32_t arrived = 1;
        if (my_rows > 0) {
            if (lane == 0) arrived = mbar_wait(inbox_bar, 0, abort_flag) ? 1u : 0u;  // false soon when the CTA has given up
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
        }
        // No CTA may leave (and hand its shared memory on) while a copy out of it may still be running. A CTA
        // arrives here when everything sent to it has come in, so when all have arrived every copy inside the
        // cluster is complete; the wait comes after this CTA's own additions, which the others need not see.
        cluster_arrive_relaxed();  // (nothing this CTA wrote is read by the others after this point)
        if (my_rows > 0) {
            // All six warps add (the producer and the MMA issuer have nothing else left to do). A warp takes whole
            // rows: lane l adds columns 4l ... 4l + 3 of every k-range's copy of the row -- one 16-byte load each,
            // four k-ranges' loads issued before the first addition -- and stores four results at once.
            constexpr uint32_t kSumWarps = kThreads / 32;
            const uint32_t c4 = lane * 4u;
            const uint32_t n = n0 + c4;
            const bool vec_ok = (p.n & 3u) == 0 && !EPI;  // 8-byte stores of four halves
            // where k-range u's copy of this CTA's first row starts (in floats from the start of the ring)
            uint32_t from[8];
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u) from[u] = (u == slice ? m0 * 128u : (MT + u * rows_per) * 128u) + c4;
            if (arrived && n < p.n && c4 < p.tile_w) {
                for (uint32_t i = warp; i < my_rows; i += 2u * kSumWarps) {
                    // two rows per trip: i and i + kSumWarps
                    const float *row = staging_f + i * 128u;
                    const bool second = i + kSumWarps < my_rows;
                    float4 acc[2];
                    acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (uint32_t s0 = 0; s0 < 8; s0 += 4u) {  // k-range order: the order of skinny_reduce_kernel
                        if (s0 < p.slices) {
                            float4 v[4][2];
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u) {
                                if (s0 + u < p.slices) {
                                    v[u][0] = *reinterpret_cast<const float4 *>(row + from[s0 + u]);
                                    if (second) v[u][1] = *reinterpret_cast<const float4 *>(row + from[s0 + u] + kSumWarps * 128u);
                                }
                            }
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u) {
                                if (s0 + u < p.slices) {
#pragma unroll
                                    for (uint32_t r = 0; r < 2; ++r) {
                                        if (r == 0 || second) {
                                            acc[r].x += v[u][r].x;
                                            acc[r].y += v[u][r].y;
                                            acc[r].z += v[u][r].z;
                                            acc[r].w += v[u][r].w;
                                        }
                                    }
                                }
                            }
                        }
                    }
#pragma unroll
                    for (uint32_t r = 0; r < 2; ++r) {
                        if (r == 0 || second) {
                            const uint32_t m = m0 + i + kSumWarps * r;
                            const size_t at = static_cast<size_t>(m) * p.n + n;
                            const float out[4] = {acc[r].x, acc[r].y, acc[r].z, acc[r].w};
                            if (vec_ok) {
                                uint2 packed;
                                packed.x = pack_half2_rn(__float_as_uint(out[0]), __float_as_uint(out[1]));
                                packed.y = pack_half2_rn(__float_as_uint(out[2]), __float_as_uint(out[3]));
                                *reinterpret_cast<uint2 *>(p.c + at) = packed;
                            } else {
#pragma unroll
                                for (uint32_t e = 0; e < 4; ++e) {
                                    if (n + e < p.n) {
                                        if (EPI) {
                                            store_c_elem(p.c, at + e, fused_value(p.epi, out[e], m, n + e, p.n), p.epi.c_type);
                                        } else {
                                            p.c[at + e] = __float2half_rn(out[e]);
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
            }
            if (threadIdx.x == 64) B200_STAMP(8);
        }
        cluster_wait_acquire();
    }

    // ---------------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // give copies still in flight time to land before shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
        if (threadIdx.x == 0) atomicExch(p.error_word, static_cast<uint32_t>(kDevWaitTimeout));
        __syncthreads();
    }
    if (CG == 2) cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, T::kTmemCols);
    }
    if (threadIdx.x == 32) B200_STAMP(10);
}

constexpr int kSkinnyReduceThreads = 256;

// C[m][n] = sum over the k-ranges of their FP32 partial results, in range order, rounded to FP16 once.
// With `fused` the sum gets alpha / beta / bias and leaves in epi.c_type.
__global__ void __launch_bounds__(kSkinnyReduceThreads) skinny_reduce_kernel(const float *partials, __half *c, uint32_t m,
                                                                            uint32_t n, uint32_t n_pad, uint32_t mt,
                                                                            uint32_t slices, uint32_t fused, EpilogueArgs epi) {
    pdl_wait_prior_grids();
    const uint32_t col = blockIdx.x * kSkinnyReduceThreads + threadIdx.x;
    const uint32_t row = blockIdx.y;
    if (row >= m || col >= n) return;
    float acc = 0.f;
    for (uint32_t s = 0; s < slices; ++s) {
        acc += partials[(static_cast<size_t>(s) * mt + row) * n_pad + col];
    }
    if (fused) {
        store_c_elem(c, static_cast<size_t>(row) * n + col, fused_value(epi, acc, row, col, n), epi.c_type);
    } else {
        c[static_cast<size_t>(row) * n + col] = __float2half_rn(acc);
    }
}

}  // namespace b200
