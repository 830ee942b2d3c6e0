// The sm_100a HGEMM kernel family: C[M x N] = A[M x K] * B^T, with A row-major (K
// contiguous), B stored as N rows of K contiguous halves, C row-major FP16 -- the operand
// layouts of the reference's entry points (src/main.cu:11, src/common/tester.h:117-119,
// element indexing as in src/simt_naive.cu:18-24). FP16 products are accumulated in FP32 in
// tensor memory and rounded to FP16 once.
//
// It replaces the reference's mma.sync / WMMA kernels (src/mma/*.cu, src/wmma/*.cu, e.g.
// src/mma/mma_async_stage4.cu:54-644) with one warp-specialised design:
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128 x 64 slab of A and a
//               (BN / CG) x 64 slab of B into a ring of 128B-swizzled stages
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (UMMA 128*CG x BN x 16)
//               and commits stage releases / accumulator hand-offs to mbarriers
//   warps 2-5   epilogue: tcgen05.ld -> FP32 -> FP16 -> swizzled staging -> TMA store
//               (or FP32 partials to the workspace when a tile's k-range is split; those are
//               summed by streamk_reduce_kernel, which follows in the stream)
//
// Two accumulators live in TMEM, so the epilogue of one tile overlaps the main loop of the
// next. CG = 2 runs a pair of CTAs (a 2-CTA cluster) on one 256 x BN tile: each CTA stages
// its own 128 rows of A and half of the B slab, the leader CTA issues the MMAs for both.
//
// Every wait in the kernel is time-bounded; on expiry the CTA drains, frees its tensor
// memory and raises an error word the host reads.
#pragma once

#include <cuda_bf16.h>

#include "ptx_sm100.cuh"
#include "sched.h"

namespace b200 {

constexpr int kBM = 128;          // rows of C per CTA
constexpr int kBK = 64;           // halves per k-block = one 128-byte swizzle row
constexpr int kThreads = 192;     // 6 warps
constexpr int kEpiThreads = 128;  // warps 2..5
constexpr uint32_t kStagingBytes = 4u * 2u * 4096u;  // 4 epilogue warps x 2 buffers x (32 rows x 128 B)

// Bits of the kernels' FLAVOR template parameter.
enum GemmFlavor : int {
    kFlavorBatched = 1,  // operands are stacks of matrices: three-dimensional tensor maps, tile -> (matrix, tile)
    kFlavorBkn = 2,      // B is stored K x N row-major (N contiguous): tm_b is {N, K} with box {64, 64}; the B slab of
                         // a stage is BN / CG / 64 such boxes, an MN-major operand of the MMA
};

enum GemmMode : int {
    kModeTiles = 0,    // every CTA walks whole tiles, strided by the grid
    kModeStreamK = 1,  // every CTA owns a contiguous range of (tile, k-block) units
};

// Error codes a kernel can raise in GemmParams::error_word.
enum DeviceError : uint32_t {
    kDevOk = 0,
    kDevWaitTimeout = 1,
};

// Element type of C (and of c_in) in the kernels instantiated with the fused epilogue; the plain kernels
// write FP16 only. The values are those of B200_C_* in the public header.
enum OutType : uint32_t {
    kOutF16 = 0,
    kOutBF16 = 1,
    kOutF32 = 2,
};

struct alignas(64) GemmParams {
    CUtensorMap tm_a;  // A as {K, M}, box {64, 128}
    CUtensorMap tm_b;  // B as {K, N}, box {64, BN / CG}
    CUtensorMap tm_c;  // C as {N, M}, box {64, 32} (only valid when tma_store != 0)
    __half *c;
    float4 *partials;        // stream-K: 2 slots per k-range, each 128 x BN FP32
    uint32_t *error_word;
    uint32_t m, n, k;
    uint32_t m_blocks;  // number of (128 * CG)-row blocks
    uint32_t n_blocks;
    uint32_t k_blocks;
    uint32_t tiles;
    uint32_t group_m;
    uint32_t dp_tiles;   // stream-k: the first dp_tiles tiles are walked whole, strided by the grid; the rest is cut into k-ranges
    uint32_t sk_parts;   // stream-k: workers that own a k-range (the first sk_parts; never more than there are units)
    uint32_t tma_store;  // 1: epilogue uses TMA stores (needs N % 8 == 0)
    uint32_t c_vec_ok;   // 1: 16-byte vector stores to C are aligned (N % 8 == 0)
    // fused epilogue (kernels instantiated with EPI only): C = alpha * A*B^T + beta * c_in + bias
    float alpha, beta;
    const __half *bias;  // N values, one per column of C, or nullptr
    const void *c_in;    // M x N of C's element type, row-major, read when beta != 0 (may be C itself), or nullptr
    uint32_t c_type;     // OutType of C and c_in (kernels with the fused epilogue only; 0 = FP16)
    // Tail of a launch with larger tiles (whole-tile mode only; tail_sm = 0: off). This launch's tile u is part
    // u % (tail_sm * tail_sn) of the larger tile tail_first + u / (tail_sm * tail_sn), which is located with
    // the larger tiles' own geometry and split tail_sm x tail_sn ways.
    uint32_t tail_first, tail_sm, tail_sn, tail_m_blocks, tail_n_blocks, tail_group_m;
    Raster raster;  // tile id -> block coordinates of this launch (of the larger tiles' raster when tail_sm != 0)
    // Batched kernels (FLAVOR & kFlavorBatched): `tiles` counts the tiles of all matrices, m_blocks x n_blocks
    // of them per matrix; the tensor maps are {columns, rows, matrices}.
    uint64_t batch_stride_c;  // elements between consecutive matrices of C (plain-store path)
#ifdef B200_TIMELINE
    unsigned long long *timeline;  // profiling builds only: per CTA 16 stamps of %globaltimer, then the same 16 of the SM's cycle counter
#endif
};

#ifdef B200_TIMELINE
#define B200_STAMP(slot)                                                                                  \
    do {                                                                                                  \
        if (p.timeline) {                                                                                 \
            p.timeline[blockIdx.x * 32 + (slot)] = global_timer_ns();                                     \
            p.timeline[blockIdx.x * 32 + 16 + (slot)] = static_cast<unsigned long long>(clock64());       \
        }                                                                                                 \
    } while (0)
#else
#define B200_STAMP(slot) \
    do {                 \
    } while (0)
#endif

template <int BN, int STAGES, int CG, int KPS = 1>
struct KernelTraits {
    static_assert(KPS == 1 || KPS == 2, "a stage holds one or two 64-wide k-blocks");
    static_assert(BN == 64 || BN == 128 || BN == 160 || BN == 192 || BN == 224 || BN == 256 || BN == 288 || BN == 320,
                  "tile widths the kernels are built for");
    static_assert((BN / CG) % 8 == 0 && BN % 32 == 0, "whole swizzle atoms per CTA, whole 32-column epilogue chunks");
    static_assert(CG == 1 || CG == 2, "CG is the CTA-pair size");
    // Tiles wider than one MMA (N <= 256) are two MMAs of BN / 2 columns side by side in one accumulator; pairs
    // only. Each CTA then stages two slabs of BN / 4 rows of B, one per MMA: an MMA of a pair takes its first
    // N / 2 columns from the leader's slab and the other half from the peer's, so the slabs are cut to keep the
    // accumulator's columns in the order of C's.
    static constexpr bool kWide = BN > 256;
    static_assert(!kWide || (CG == 2 && KPS == 1 && (BN / 4) % 8 == 0 && (BN / 2) % 16 == 0), "wide tiles: CTA pairs, one k-block per stage");
    static constexpr uint32_t kAccStages = 2 * BN <= 512 ? 2 : 1;  // a wide tile's accumulator leaves no room for a second
    static constexpr uint32_t kARows = kBM;
    static constexpr uint32_t kBRows = BN / CG;
    static constexpr uint32_t kABytes = kARows * kBK * 2;
    static constexpr uint32_t kBBytes = kBRows * kBK * 2;
    static constexpr uint32_t kBlockBytes = kABytes + kBBytes;   // one k-block of A and B
    static constexpr uint32_t kStageBytes = KPS * kBlockBytes;  // [A0][B0] or [A0][B0][A1][B1]
    static constexpr uint32_t kTmemCols = 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;  // two accumulators; power of two
    static constexpr uint32_t kAccStride = kTmemCols / 2;  // the second accumulator (if any) starts half way (BN columns for the widths that are powers of two times 64)
    static constexpr uint32_t kBarrierBytes = 256;
    static constexpr uint32_t kSmemBytes = 1024 + STAGES * kStageBytes + kStagingBytes + kBarrierBytes;
    static_assert((kBlockBytes % 1024) == 0, "operand slabs must keep 1024-byte alignment");
    static_assert(kSmemBytes <= 232448, "exceeds 227 KB of shared memory");
    static_assert((2 * STAGES + 4) * 8 + 16 <= kBarrierBytes, "barrier area too small");
};

// Iterates this worker's segments; all three roles walk the same sequence.
template <int MODE>
struct WorkWalker;

template <>
struct WorkWalker<kModeTiles> {
    uint32_t t, step, tiles, k_blocks;
    __device__ WorkWalker(const GemmParams &p, uint32_t worker, uint32_t workers)
        : t(worker), step(workers), tiles(p.tiles), k_blocks(p.k_blocks) {}
    __device__ bool next(Segment &s) {
        if (t >= tiles) return false;
        s.tile = t;
        s.kb0 = 0;
        s.kb1 = k_blocks;
        t += step;
        return true;
    }
};

// Stream-k, optionally behind whole tiles: a worker first takes every workers-th of the first
// dp_tiles tiles whole, then its contiguous range of the (tile, k) units of the remaining tiles.
// With dp_tiles = a whole number of waves, only the ragged last wave pays for partial tiles.
template <>
struct WorkWalker<kModeStreamK> {
    uint32_t t, step, dp_tiles, k_blocks;
    bool has_range;  // only the first sk_parts workers own a k-range (there are never more ranges than units)
    SegmentWalker w;
    __device__ WorkWalker(const GemmParams &p, uint32_t worker, uint32_t workers)
        : t(worker), step(workers), dp_tiles(p.dp_tiles), k_blocks(p.k_blocks), has_range(worker < p.sk_parts),
          w(has_range ? worker : 0u, p.sk_parts > 0 ? p.sk_parts : 1u, p.tiles - p.dp_tiles, p.k_blocks) {}
    __device__ bool next(Segment &s) {
        if (t < dp_tiles) {
            s.tile = t;
            s.kb0 = 0;
            s.kb1 = k_blocks;
            t += step;
            return true;
        }
        if (!has_range || !w.next(s)) return false;
        s.tile += dp_tiles;
        return true;
    }
};

// Linear tile id of this launch -> block coordinates in this launch's own tile size.
__device__ __forceinline__ TileCoord locate_tile(const GemmParams &p, uint32_t tile) {
    if (p.tail_sm == 0) return tile_coord_fast(tile, p.raster);
    const uint32_t per = p.tail_sm * p.tail_sn;
    const uint32_t part = tile % per;
    TileCoord c = tile_coord_fast(p.tail_first + tile / per, p.raster);
    c.m_blk = c.m_blk * p.tail_sm + part % p.tail_sm;
    c.n_blk = c.n_blk * p.tail_sn + part / p.tail_sm;
    return c;
}

// 32 FP32 accumulator columns of one row -> FP16 -> global memory.
__device__ __forceinline__ void store_row_chunk32(__half *c, uint32_t row, uint32_t col0, uint32_t m, uint32_t n,
                                                  bool vec_ok, const uint32_t (&r)[32]) {
    if (row >= m || col0 >= n) return;
    __half *dst = c + static_cast<size_t>(row) * n + col0;
    if (vec_ok && col0 + 32 <= n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_half2_rn(r[8 * j + 0], r[8 * j + 1]);
            v.y = pack_half2_rn(r[8 * j + 2], r[8 * j + 3]);
            v.z = pack_half2_rn(r[8 * j + 4], r[8 * j + 5]);
            v.w = pack_half2_rn(r[8 * j + 6], r[8 * j + 7]);
            reinterpret_cast<uint4 *>(dst)[j] = v;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < n) dst[j] = __float2half_rn(__uint_as_float(r[j]));
        }
    }
}

// Two FP32 -> two packed 16-bit values of C's type, round to nearest even.
__device__ __forceinline__ uint32_t pack2_rn(uint32_t lo_f32_bits, uint32_t hi_f32_bits, uint32_t c_type) {
    if (c_type == kOutBF16) {
        __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(lo_f32_bits), __uint_as_float(hi_f32_bits));
        return *reinterpret_cast<uint32_t *>(&b);
    }
    return pack_half2_rn(lo_f32_bits, hi_f32_bits);
}

// Element i of a row-major matrix of C's type, as FP32.
__device__ __forceinline__ float load_c_elem(const void *base, size_t i, uint32_t c_type) {
    if (c_type == kOutF32) return static_cast<const float *>(base)[i];
    if (c_type == kOutBF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(base)[i]);
    return __half2float(static_cast<const __half *>(base)[i]);
}

__device__ __forceinline__ void store_c_elem(void *base, size_t i, float v, uint32_t c_type) {
    if (c_type == kOutF32) {
        static_cast<float *>(base)[i] = v;
    } else if (c_type == kOutBF16) {
        static_cast<__nv_bfloat16 *>(base)[i] = __float2bfloat16_rn(v);
    } else {
        static_cast<__half *>(base)[i] = __float2half_rn(v);
    }
}

// What the fused epilogue needs to know, for kernels that do not carry a whole GemmParams.
struct EpilogueArgs {
    float alpha, beta;
    const __half *bias;
    const void *c_in;
    uint32_t c_type;
};

// v = alpha * v + bias[col] + beta * c_in[row][col] for one element (callers check the bounds).
__device__ __forceinline__ float fused_value(const EpilogueArgs &e, float acc, size_t row, uint32_t col, uint32_t n) {
    float v = e.alpha * acc;
    if (e.bias) v += __half2float(e.bias[col]);
    if (e.beta != 0.f && e.c_in) v = fmaf(e.beta, load_c_elem(e.c_in, row * n + col, e.c_type), v);
    return v;
}

// Fused epilogue on COUNT accumulator columns of one row, in place (FP32 bit patterns):
// v = alpha * v + bias[col] + beta * c_in[row][col]. Out-of-range rows and columns are left alone
// (they are clipped when stored).
template <int COUNT>
__device__ __forceinline__ void fused_epilogue(const GemmParams &p, uint32_t row, uint32_t col0, uint32_t *vals) {
    const bool row_ok = row < p.m;
    const bool vec_ok = p.c_vec_ok != 0 && col0 + COUNT <= p.n;
    const __half *bias = p.bias ? p.bias + col0 : nullptr;
    const bool use_cin = p.beta != 0.f && p.c_in && row_ok;
    const size_t cin_off = static_cast<size_t>(row) * p.n + col0;
#pragma unroll
    for (int j = 0; j < COUNT; j += 8) {
        float add[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (vec_ok) {
            if (bias) {
                const uint4 b = *reinterpret_cast<const uint4 *>(bias + j);
                const __half2 *h = reinterpret_cast<const __half2 *>(&b);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    add[2 * e] += f.x;
                    add[2 * e + 1] += f.y;
                }
            }
            if (use_cin) {
                if (p.c_type == kOutF32) {
                    const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(p.c_in) + cin_off + j);
                    const float4 c0 = src[0], c1 = src[1];
                    add[0] += p.beta * c0.x; add[1] += p.beta * c0.y; add[2] += p.beta * c0.z; add[3] += p.beta * c0.w;
                    add[4] += p.beta * c1.x; add[5] += p.beta * c1.y; add[6] += p.beta * c1.z; add[7] += p.beta * c1.w;
                } else {
                    const uint4 c = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.c_in) + cin_off + j);
                    if (p.c_type == kOutBF16) {
                        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&c);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(h[e]);
                            add[2 * e] += p.beta * f.x;
                            add[2 * e + 1] += p.beta * f.y;
                        }
                    } else {
                        const __half2 *h = reinterpret_cast<const __half2 *>(&c);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(h[e]);
                            add[2 * e] += p.beta * f.x;
                            add[2 * e + 1] += p.beta * f.y;
                        }
                    }
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (col0 + j + e < p.n) {
                    if (bias) add[e] += __half2float(bias[j + e]);
                    if (use_cin) add[e] += p.beta * load_c_elem(p.c_in, cin_off + j + e, p.c_type);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) vals[j + e] = __float_as_uint(fmaf(p.alpha, __uint_as_float(vals[j + e]), add[e]));
    }
}

// 32 FP32 accumulator columns of one row -> C's element type -> global memory (kernels with the fused epilogue).
__device__ __forceinline__ void store_row_chunk32_typed(void *c, uint32_t c_type, uint32_t row, uint32_t col0, uint32_t m,
                                                        uint32_t n, bool vec_ok, const uint32_t (&r)[32]) {
    if (row >= m || col0 >= n) return;
    const size_t off = static_cast<size_t>(row) * n + col0;
    if (vec_ok && col0 + 32 <= n) {
        if (c_type == kOutF32) {
            float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(c) + off);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                     __uint_as_float(r[4 * j + 3]));
            }
        } else {
            uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__half *>(c) + off);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack2_rn(r[8 * j + 0], r[8 * j + 1], c_type);
                v.y = pack2_rn(r[8 * j + 2], r[8 * j + 3], c_type);
                v.z = pack2_rn(r[8 * j + 4], r[8 * j + 5], c_type);
                v.w = pack2_rn(r[8 * j + 6], r[8 * j + 7], c_type);
                dst[j] = v;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < n) store_c_elem(c, off + j, __uint_as_float(r[j]), c_type);
        }
    }
}

// KPS = k-blocks per stage. With KPS = 2, GemmParams::k_blocks and every k index of the work
// decomposition count pairs of k-blocks (one stage each); a pair that reaches past K reads zeros there.
// EPI: apply GemmParams' alpha / beta / bias in the epilogue and write C in GemmParams::c_type (tiles whose
// k-range is cut leave FP32 partials as always; streamk_reduce_kernel applies the same epilogue to their sum).
template <int BN, int STAGES, int CG, int MODE, int KPS = 1, bool EPI = false, int FLAVOR = 0>
__global__ void __launch_bounds__(kThreads, 1) hgemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
    constexpr bool BATCHED = (FLAVOR & kFlavorBatched) != 0;
    constexpr bool BKN = (FLAVOR & kFlavorBkn) != 0;
    static_assert(!BKN || (!BATCHED && BN % (64 * CG) == 0), "K x N row-major B: whole 64-column boxes per CTA, single matrices");
    static_assert(!BATCHED || (MODE == kModeTiles && !EPI), "stacks of matrices are multiplied in whole tiles, plain epilogue");
    using T = KernelTraits<BN, STAGES, CG, KPS>;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw_addr);

    const uint32_t staging = base + STAGES * T::kStageBytes;
    uint8_t *staging_ptr = base_ptr + STAGES * T::kStageBytes;
    const uint32_t bars = staging + kStagingBytes;
    uint8_t *bars_ptr = staging_ptr + kStagingBytes;
    // barrier area: full[STAGES] | empty[STAGES] | tmem_full[2] | tmem_empty[2] | tmem base | abort
    const uint32_t full_bar = bars;
    const uint32_t empty_bar = bars + 8u * STAGES;
    const uint32_t tfull_bar = bars + 16u * STAGES;
    const uint32_t tempty_bar = tfull_bar + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars_ptr + 16u * STAGES + 32u);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t cta_rank = (CG == 2) ? cluster_cta_rank() : 0u;
    const uint32_t worker = blockIdx.x / CG;
    const uint32_t workers = gridDim.x / CG;

    if (threadIdx.x == 0) B200_STAMP(0);
    if (warp == 0) {
        // one lane per barrier: the set-up of the producer warp is a serial chain otherwise
        if (lane < static_cast<uint32_t>(STAGES)) {
            mbar_init(full_bar + 8u * lane, 1);
            mbar_init(empty_bar + 8u * lane, 1);
        } else if (lane < static_cast<uint32_t>(STAGES) + 2u) {
            const uint32_t a = lane - STAGES;
            mbar_init(tfull_bar + 8u * a, 1);
            mbar_init(tempty_bar + 8u * a, 4 * CG);  // one arrival per epilogue warp of every CTA of the pair
        } else if (lane == static_cast<uint32_t>(STAGES) + 2u) {
            *abort_flag = 0;
        }
        fence_mbar_init();
        __syncwarp();
    }
    if (warp == 2 && lane == 0) {
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_b);
        if (p.tma_store) tma_prefetch_desc(&p.tm_c);
    }
    if (warp == 3 && lane == 0) {
        // The kernel's parameters sit in constant memory and nothing on this SM has read them yet: the producer's
        // first tile would pay one cache miss after the other for them (measured: 1175 cycles from the dependency
        // wait to its first load at 256^3, most of it here). An idle epilogue lane reads them now, while the
        // barriers are set up, so that the producer finds them cached.
        const uint32_t touch = p.tiles + p.k_blocks + p.m_blocks + p.n_blocks + p.group_m + p.dp_tiles + p.sk_parts + p.tail_sm +
                               p.m + p.n + p.tma_store + p.raster.n_blocks + p.raster.tall_tiles + p.raster.tall_span.mul +
                               p.raster.short_span.mul + p.raster.tall_rows.mul + p.raster.short_rows.sh2;
        asm volatile("" ::"r"(touch));
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
        // The producer warp initialised the barriers itself and needs no tensor memory: it
        // only announces its arrival and starts loading while the allocation completes.
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

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            WorkWalker<MODE> work(p, worker, workers);
            Segment seg;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            uint32_t filled = 0;  // stages filled so far, counted up to STAGES: the first trip round the ring finds every stage free
#ifdef B200_TIMELINE
            bool stamped_first_load = false;
#endif
            B200_STAMP(11);
            pdl_wait_prior_grids();  // A and B may have been written by the previous kernel
            B200_STAMP(12);
            while (ok && work.next(seg)) {
                uint32_t zt = seg.tile;
                int32_t z = 0;  // which matrix of the stack
                if (BATCHED) {
                    z = static_cast<int32_t>(zt / (p.m_blocks * p.n_blocks));
                    zt -= static_cast<uint32_t>(z) * p.m_blocks * p.n_blocks;
                }
                const TileCoord tc = locate_tile(p, zt);
                const int32_t row_a = static_cast<int32_t>((tc.m_blk * CG + cta_rank) * kBM);
                const int32_t row_b = static_cast<int32_t>(tc.n_blk * BN + cta_rank * T::kBRows);
#ifdef B200_TIMELINE
                if (!stamped_first_load) {
                    asm volatile("" ::"r"(row_a), "r"(row_b));
                    B200_STAMP(14);
                }
#endif
                for (uint32_t kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (filled < static_cast<uint32_t>(STAGES)) {
                        ++filled;
                    } else if (!mbar_wait(empty_bar + 8u * stage, phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
#ifdef B200_TIMELINE
                    if (!stamped_first_load) B200_STAMP(13);
#endif
                    const uint32_t slot = base + stage * T::kStageBytes;
                    if (CG == 1) {
                        mbar_arrive_expect_tx(full_bar + 8u * stage, T::kStageBytes);
#pragma unroll
                        for (uint32_t j = 0; j < KPS; ++j) {
                            const uint32_t sa = slot + j * T::kBlockBytes;
                            const int32_t kx = static_cast<int32_t>((kb * KPS + j) * kBK);  // past K: zero fill
                            if (BKN) {
                                tma_load_2d(sa, &p.tm_a, kx, row_a, full_bar + 8u * stage);
#pragma unroll
                                for (uint32_t g = 0; g < T::kBRows / 64u; ++g) {  // x = column of B (of C), y = k
                                    tma_load_2d(sa + T::kABytes + g * 8192u, &p.tm_b, row_b + static_cast<int32_t>(g * 64u), kx,
                                                full_bar + 8u * stage);
                                }
                            } else if (BATCHED) {
                                tma_load_3d(sa, &p.tm_a, kx, row_a, z, full_bar + 8u * stage);
                                tma_load_3d(sa + T::kABytes, &p.tm_b, kx, row_b, z, full_bar + 8u * stage);
                            } else {
                                tma_load_2d(sa, &p.tm_a, kx, row_a, full_bar + 8u * stage);
                                tma_load_2d(sa + T::kABytes, &p.tm_b, kx, row_b, full_bar + 8u * stage);
                            }
                        }
                    } else {
                        // Both CTAs' copies complete on the leader's barrier; the leader alone
                        // posts the expected byte count for the pair.
                        if (cta_rank == 0) mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * T::kStageBytes);
                        const uint32_t leader_bar = map_to_cta(full_bar + 8u * stage, 0);
#pragma unroll
                        for (uint32_t j = 0; j < KPS; ++j) {
                            const uint32_t sa = slot + j * T::kBlockBytes;
                            const int32_t kx = static_cast<int32_t>((kb * KPS + j) * kBK);
                            if (BKN) {
                                tma_load_2d_pair(sa, &p.tm_a, kx, row_a, leader_bar);
#pragma unroll
                                for (uint32_t g = 0; g < T::kBRows / 64u; ++g) {
                                    tma_load_2d_pair(sa + T::kABytes + g * 8192u, &p.tm_b, row_b + static_cast<int32_t>(g * 64u), kx,
                                                     leader_bar);
                                }
                            } else if (BATCHED) {
                                tma_load_3d_pair(sa, &p.tm_a, kx, row_a, z, leader_bar);
                                tma_load_3d_pair(sa + T::kABytes, &p.tm_b, kx, row_b, z, leader_bar);
                            } else if (T::kWide) {
                                // two slabs of BN / 4 rows: columns [r * BN / 4, (r + 1) * BN / 4) of each half of the tile
                                tma_load_2d_pair(sa, &p.tm_a, kx, row_a, leader_bar);
                                const int32_t half0 = static_cast<int32_t>(tc.n_blk * BN + cta_rank * (BN / 4));
                                tma_load_2d_pair(sa + T::kABytes, &p.tm_b, kx, half0, leader_bar);
                                tma_load_2d_pair(sa + T::kABytes + (BN / 4) * 128u, &p.tm_b, kx, half0 + BN / 2, leader_bar);
                            } else {
                                tma_load_2d_pair(sa, &p.tm_a, kx, row_a, leader_bar);
                                tma_load_2d_pair(sa + T::kABytes, &p.tm_b, kx, row_b, leader_bar);
                            }
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
#ifdef B200_TIMELINE
                    if (!stamped_first_load) {
                        B200_STAMP(2);
                        stamped_first_load = true;
                    }
#endif
                }
            }
            B200_STAMP(3);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t kMmaN = T::kWide ? BN / 2 : BN;  // columns one MMA writes
            constexpr uint32_t idesc = BKN ? umma_idesc_f16_f32_b_mn(kBM * CG, kMmaN) : umma_idesc_f16_f32(kBM * CG, kMmaN);
            WorkWalker<MODE> work(p, worker, workers);
            Segment seg;
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            while (ok && work.next(seg)) {
                const uint32_t acc = T::kAccStages == 2 ? (it & 1u) : 0u;
                const uint32_t acc_phase = T::kAccStages == 2 ? ((it >> 1) & 1u) : (it & 1u);
                if (!mbar_wait(tempty_bar + 8u * acc, acc_phase ^ 1u, abort_flag)) break;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * T::kAccStride;
                for (uint32_t kb = seg.kb0; kb < seg.kb1; ++kb) {
                    if (!mbar_wait(full_bar + 8u * stage, phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
#ifdef B200_TIMELINE
                    if (it == 0 && kb == seg.kb0) B200_STAMP(4);
#endif
                    const uint32_t slot = base + stage * T::kStageBytes;
#pragma unroll
                    for (uint32_t j = 0; j < KPS; ++j) {
                        const uint64_t da = umma_smem_desc_sw128(slot + j * T::kBlockBytes);
                        const uint64_t db = BKN ? umma_smem_desc_sw128_mn(slot + j * T::kBlockBytes + T::kABytes, 8192u)
                                                : umma_smem_desc_sw128(slot + j * T::kBlockBytes + T::kABytes);
#pragma unroll
                        for (uint32_t k = 0; k < kBK / 16; ++k) {
                            // 16 halves = 32 bytes along K inside the swizzle atom -> +2 in the address field; for
                            // the MN-major B, 16 rows of k = two atoms of 1024 bytes -> +128
                            umma_f16<CG>(d_tmem, da + 2u * k, db + (BKN ? 128u : 2u) * k, idesc,
                                         (kb > seg.kb0 || j > 0 || k > 0) ? 1u : 0u);
                            if (T::kWide) {
                                // the tile's second half: the other slab of B (BN / 4 rows of 128 bytes further, in
                                // the descriptor's 16-byte units), the accumulator's columns BN / 2 onward
                                umma_f16<CG>(d_tmem + BN / 2, da + 2u * k, db + (BN / 4) * 8u + 2u * k, idesc,
                                             (kb > seg.kb0 || j > 0 || k > 0) ? 1u : 0u);
                            }
                        }
                    }
                    if (CG == 1) {
                        umma_commit(empty_bar + 8u * stage);
                    } else {
                        umma_commit_pair(empty_bar + 8u * stage, 0x3);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (CG == 1) {
                    umma_commit(tfull_bar + 8u * acc);
                } else {
                    umma_commit_pair(tfull_bar + 8u * acc, 0x3);
                }
                ++it;
            }
            B200_STAMP(5);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        const uint32_t q = warp & 3u;  // TMEM lane quadrant this warp may read
        [[maybe_unused]] const uint32_t epi_tid = threadIdx.x - 64u;
        uint8_t *my_staging_ptr = staging_ptr + q * 8192u;
        const uint32_t my_staging = staging + q * 8192u;
        WorkWalker<MODE> work(p, worker, workers);
        Segment seg;
        uint32_t it = 0, store_buf = 0;
        pdl_wait_prior_grids();  // C and the workspace may still be in use by the previous kernel
        while (work.next(seg)) {
            const uint32_t acc = T::kAccStages == 2 ? (it & 1u) : 0u;
            const uint32_t acc_phase = T::kAccStages == 2 ? ((it >> 1) & 1u) : (it & 1u);
            uint32_t zt = seg.tile;
            int32_t z = 0;
            if (BATCHED) {
                z = static_cast<int32_t>(zt / (p.m_blocks * p.n_blocks));
                zt -= static_cast<uint32_t>(z) * p.m_blocks * p.n_blocks;
            }
            const TileCoord tc = locate_tile(p, zt);
            const uint32_t m0 = (tc.m_blk * CG + cta_rank) * kBM;
            const uint32_t n0 = tc.n_blk * BN;
            // one lane per warp polls the barrier; the other 31 park at the warp barrier
            uint32_t ready = 1;
            if (lane == 0) ready = mbar_wait(tfull_bar + 8u * acc, acc_phase, abort_flag) ? 1u : 0u;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            tcgen05_fence_after_sync();
#ifdef B200_TIMELINE
            if (epi_tid == 0) B200_STAMP(it == 0 ? 6 : 7);
#endif
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * T::kAccStride;
            const uint32_t row_in_tile = q * 32u + lane;
            const bool whole_tile = (MODE == kModeTiles) || (seg.kb0 == 0 && seg.kb1 == p.k_blocks);

            if (whole_tile) {
                if (p.tma_store) {
                    const bool warp_rows_live = (m0 + q * 32u) < p.m;
                    constexpr uint32_t kChunks = BN / 64;
                    // Two register sets: the TMEM load of chunk c+1 is in flight while chunk c is
                    // converted, staged and handed to TMA.
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
                        }
                        const bool live = warp_rows_live && (n0 + c * 64u) < p.n;
                        if (live) {
                            if (EPI) fused_epilogue<64>(p, m0 + row_in_tile, n0 + c * 64u, cur);
                            uint8_t *buf = my_staging_ptr + (store_buf & 1u) * 4096u;
                            // the store issued two chunks ago read this buffer: wait until it has
                            if (lane == 0) tma_store_wait_read<1>();
                            __syncwarp();
                            uint8_t *row_ptr = buf + lane * 128u;
                            const uint32_t c_type = EPI ? p.c_type : static_cast<uint32_t>(kOutF16);  // FP16 or BF16 here
#pragma unroll
                            for (uint32_t j = 0; j < 8; ++j) {
                                uint4 v;
                                v.x = pack2_rn(cur[8 * j + 0], cur[8 * j + 1], c_type);
                                v.y = pack2_rn(cur[8 * j + 2], cur[8 * j + 3], c_type);
                                v.z = pack2_rn(cur[8 * j + 4], cur[8 * j + 5], c_type);
                                v.w = pack2_rn(cur[8 * j + 6], cur[8 * j + 7], c_type);
                                // 128-byte swizzle: 16-byte word j of row r lives at word j ^ (r % 8)
                                *reinterpret_cast<uint4 *>(row_ptr + ((j ^ (lane & 7u)) << 4)) = v;
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                if (BATCHED) {
                                    tma_store_3d(&p.tm_c, my_staging + (store_buf & 1u) * 4096u,
                                                 static_cast<int32_t>(n0 + c * 64u), static_cast<int32_t>(m0 + q * 32u), z);
                                } else {
                                    tma_store_2d(&p.tm_c, my_staging + (store_buf & 1u) * 4096u,
                                                 static_cast<int32_t>(n0 + c * 64u), static_cast<int32_t>(m0 + q * 32u));
                                }
                                tma_store_commit();
                            }
                            ++store_buf;
                        }
                    }
                    if (BN % 64 == 32) {
                        // a tile 160 or 224 columns wide ends in half a chunk: its 32 columns leave with plain 16-byte stores
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(taddr + kChunks * 64u, r);
                        tmem_ld_wait();
                        if (EPI) {
                            fused_epilogue<32>(p, m0 + row_in_tile, n0 + kChunks * 64u, r);
                            store_row_chunk32_typed(p.c, p.c_type, m0 + row_in_tile, n0 + kChunks * 64u, p.m, p.n, p.c_vec_ok != 0, r);
                        } else {
                            store_row_chunk32(p.c, m0 + row_in_tile, n0 + kChunks * 64u, p.m, p.n, p.c_vec_ok != 0, r);
                        }
                    }
                } else {
#pragma unroll 1
                    for (uint32_t c = 0; c < BN / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(taddr + c * 32u, r);
                        tmem_ld_wait();
                        if (EPI) {
                            fused_epilogue<32>(p, m0 + row_in_tile, n0 + c * 32u, r);
                            store_row_chunk32_typed(p.c, p.c_type, m0 + row_in_tile, n0 + c * 32u, p.m, p.n, p.c_vec_ok != 0, r);
                        } else {
                            __half *c_mat = BATCHED ? p.c + static_cast<size_t>(z) * p.batch_stride_c : p.c;
                            store_row_chunk32(c_mat, m0 + row_in_tile, n0 + c * 32u, p.m, p.n, p.c_vec_ok != 0, r);
                        }
                    }
                }
                // accumulator drained: hand it back to the MMA warp
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (CG == 1) {
                        mbar_arrive(tempty_bar + 8u * acc);
                    } else {
                        mbar_arrive_cluster(map_to_cta(tempty_bar + 8u * acc, 0));
                    }
                }
            } else {
                // ---- this tile's k-range is shared with other workers: publish an FP32 partial
                // (a pair's slot holds 256 x BN values; each CTA writes the half that belongs to its 128 rows)
                const uint32_t slot = partial_slot(worker, p.sk_parts, p.tiles - p.dp_tiles, p.k_blocks, seg.tile - p.dp_tiles);
                float4 *ws = p.partials + (static_cast<size_t>(slot) * CG + cta_rank) * (kBM * BN / 4);
                const bool row_live = (m0 + row_in_tile) < p.m;
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + c * 32u, r);
                    tmem_ld_wait();
                    if (row_live && (n0 + c * 32u) < p.n) {
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) {
                            float4 v = make_float4(__uint_as_float(r[4 * j + 0]), __uint_as_float(r[4 * j + 1]),
                                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                            // row-fastest layout: consecutive lanes write consecutive 16-byte words
                            ws[(c * 8u + j) * kBM + row_in_tile] = v;
                        }
                    }
                }
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (CG == 1) {
                        mbar_arrive(tempty_bar + 8u * acc);
                    } else {
                        mbar_arrive_cluster(map_to_cta(tempty_bar + 8u * acc, 0));
                    }
                }

                // the partial tiles of all ranges are summed by streamk_reduce_kernel, launched next
            }
            ++it;
        }
        if (epi_tid == 0) B200_STAMP(8);
        // shared memory must stay valid until the last TMA store has read it (the writes
        // themselves are complete, like any store, when the kernel has finished)
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        if (epi_tid == 0) B200_STAMP(9);
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

// ------------------------------------------------------------------------------------------
// Sums the FP32 partial tiles a stream-k launch left in the workspace and writes FP16 C.
// ------------------------------------------------------------------------------------------
// grid = (chunks, tiles): block (x, t) handles the x-th share of tile t's live 16-byte words.
// Tiles that one k-range covered completely were stored by the GEMM kernel itself and are
// skipped. The contributing ranges are added in range order, so the result does not depend on
// timing. The partials are laid out row-fastest ([16-byte column word][row]), which makes every
// load here coalesced; being a kernel of its own, the reduction runs on all SMs at once instead
// of on whichever CTA happened to finish a tile last.
struct ReduceParams {
    const float4 *partials;
    __half *c;
    uint32_t m, n;
    uint32_t m_blocks, n_blocks, k_blocks, tiles, group_m;
    uint32_t dp_tiles;  // tiles the GEMM kernel walked whole; the k-ranges cover tiles [dp_tiles, tiles)
    uint32_t parts;
    uint32_t bn;
    uint32_t cg;        // 1: tiles of 128 rows; 2: pair tiles of 256 rows (each slot holds the two CTAs' halves one after the other)
    uint32_t fused;     // 1: apply `epi` to the sums and write C in epi.c_type; 0: plain FP16
    EpilogueArgs epi;
};

constexpr int kReduceThreads = 256;

__global__ void __launch_bounds__(kReduceThreads) streamk_reduce_kernel(const ReduceParams p) {
    const uint32_t cut_tile = blockIdx.y;  // index among the tiles that are cut into k-ranges
    const uint32_t cut_tiles = p.tiles - p.dp_tiles;
    const uint32_t tile = p.dp_tiles + cut_tile;
    const uint64_t total_units = static_cast<uint64_t>(cut_tiles) * p.k_blocks;
    const uint64_t u0 = static_cast<uint64_t>(cut_tile) * p.k_blocks;
    const uint32_t part_first = part_of_unit(u0, p.parts, total_units);
    const uint32_t part_last = part_of_unit(u0 + p.k_blocks - 1, p.parts, total_units);
    pdl_wait_prior_grids();  // the partials are written by the GEMM kernel launched just before
    if (part_first == part_last) return;

    const TileCoord tc = tile_coord(tile, p.m_blocks, p.n_blocks, p.group_m);
    const uint32_t half = blockIdx.z;  // which CTA's 128 rows of a pair tile (always 0 for single-CTA tiles)
    const uint32_t m0 = (tc.m_blk * p.cg + half) * kBM, n0 = tc.n_blk * p.bn;
    if (m0 >= p.m) return;
    const uint32_t rows_live = (p.m - m0) < static_cast<uint32_t>(kBM) ? (p.m - m0) : kBM;
    const uint32_t cols_left = p.n - n0;
    const uint32_t words_per_row = ((cols_left < p.bn ? cols_left : p.bn) + 3u) / 4u;
    const uint32_t total_words = rows_live * words_per_row;
    const uint32_t n_parts = part_last - part_first + 1u;
    const size_t slot_words = static_cast<size_t>(kBM) * p.bn / 4;
    // the first contributor may have entered this tile from an earlier one (its second slot);
    // every later contributor starts inside this tile (its first slot)
    const uint32_t slot_first = partial_slot(part_first, p.parts, cut_tiles, p.k_blocks, cut_tile);
    const bool vec4_ok = (p.n % 4u) == 0;

    for (uint32_t i = blockIdx.x * kReduceThreads + threadIdx.x; i < total_words; i += gridDim.x * kReduceThreads) {
        const uint32_t w = i / rows_live, r = i - w * rows_live;
        const size_t off = static_cast<size_t>(w) * kBM + r;
        float4 acc = ld_cg_f4(p.partials + (static_cast<size_t>(slot_first) * p.cg + half) * slot_words + off);
        uint32_t k = 1;
        for (; k + 1 < n_parts; k += 2) {  // two loads in flight per step
            const float4 v0 = ld_cg_f4(p.partials + (static_cast<size_t>(2u * (part_first + k)) * p.cg + half) * slot_words + off);
            const float4 v1 = ld_cg_f4(p.partials + (static_cast<size_t>(2u * (part_first + k + 1)) * p.cg + half) * slot_words + off);
            acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
            acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
        }
        if (k < n_parts) {
            const float4 v0 = ld_cg_f4(p.partials + (static_cast<size_t>(2u * (part_first + k)) * p.cg + half) * slot_words + off);
            acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
        }
        const uint32_t col = n0 + w * 4u;
        if (p.fused) {
            const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
            const size_t row = m0 + r;
            for (uint32_t e = 0; e < 4 && col + e < p.n; ++e) {
                store_c_elem(p.c, row * p.n + col + e, fused_value(p.epi, vals[e], row, col + e, p.n), p.epi.c_type);
            }
            continue;
        }
        __half *dst = p.c + static_cast<size_t>(m0 + r) * p.n + col;
        if (vec4_ok && col + 4u <= p.n) {
            uint2 v;
            v.x = pack_half2_rn(__float_as_uint(acc.x), __float_as_uint(acc.y));
            v.y = pack_half2_rn(__float_as_uint(acc.z), __float_as_uint(acc.w));
            *reinterpret_cast<uint2 *>(dst) = v;
        } else {
            const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
            for (uint32_t e = 0; e < 4 && col + e < p.n; ++e) dst[e] = __float2half_rn(vals[e]);
        }
    }
}

}  // namespace b200
