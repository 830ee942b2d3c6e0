// Thin inline-PTX wrappers for the sm_100a features the HGEMM kernels use:
// mbarrier (with time-bounded waits), TMA tiled loads/stores, tcgen05 (TMEM
// allocation, UMMA issue, commit, TMEM loads) and the proxy fences between them.
//
// This header takes the place of the reference's PTX macro layer
// (src/common/ptx.h:9-43: ldmatrix / mma.sync / cp.async), which has no
// counterpart on the Blackwell tensor-core path.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------
// address helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Number of CTAs in the cluster this CTA was launched in.
__device__ __forceinline__ uint32_t cluster_num_ctas() {
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}

// Address of the same shared-memory offset inside CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

// One float into the shared memory of another CTA of the cluster (an address from map_to_cta).
__device__ __forceinline__ void st_shared_cluster_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// Bulk copy from this CTA's shared memory into another CTA's of the cluster; the bytes are counted on a barrier
// in the destination CTA. Both cluster addresses come from map_to_cta with the same rank; addresses and size
// are multiples of 16 bytes. The source must stay allocated and unchanged until the destination's barrier has
// seen the bytes.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t cluster_dst, uint32_t local_src, uint32_t bytes,
                                                     uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(cluster_dst),
                 "r"(local_src), "r"(bytes), "r"(cluster_bar)
                 : "memory");
}

__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
// Arrival that publishes nothing: for a barrier that only says "what was sent to me has come in".
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    cluster_arrive_release();
    cluster_wait_acquire();
}

// ---------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------
// Lets the next kernel in the stream (if it was launched with programmatic stream
// serialization) start its prologue while this grid is still running.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Blocks until every grid this one depends on has completed and its memory is visible.
// Must precede the first global-memory access that can conflict with the previous kernel.
__device__ __forceinline__ void pdl_wait_prior_grids() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Named barrier among `count` threads: arrive without waiting / arrive and wait.
__device__ __forceinline__ void named_bar_arrive(uint32_t id, uint32_t count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy and to the peer CTA.
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that lives in another CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Longest time one wait may take before the kernel gives up (nanoseconds).
// A healthy wait is microseconds; the bound only exists so that a protocol
// bug ends as an error status instead of a hung GPU.
#ifndef B200_WAIT_LIMIT_NS
#define B200_WAIT_LIMIT_NS 2000000000ull
#endif

// Bounded wait. `abort_flag` is a CTA-shared word: once any role of the CTA has
// given up, every later wait returns false at once so the CTA drains quickly.
// Returns true when the barrier phase completed.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0x3ffu) == 0) {
            if (*abort_flag != 0) return false;
            uint64_t now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, B200_WAIT_LIMIT_NS);
}

// ---------------------------------------------------------------------------
// proxy fences
// ---------------------------------------------------------------------------
// Orders generic-proxy shared-memory writes before later async-proxy (TMA) reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), 2-D tiled
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// x = innermost coordinate (elements), y = row. x * sizeof(elem) must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Asks for one box to be brought into L2 (no shared-memory destination, no barrier). A hint: data that
// is rewritten afterwards is simply read again from L2, the point of coherence, by the load that follows.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *tm, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y)
                 : "memory");
}

// Pair-CTA form: the destination is this CTA's shared memory, the barrier may live in the
// peer CTA of the pair (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y,
                                                 uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
        "%3}], [%4];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tm, uint32_t smem_src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}

// Three-dimensional forms for batched operands viewed as {columns, rows, matrices}: z picks the matrix.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y, int32_t z,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap *tm, int32_t x, int32_t y, int32_t z,
                                                 uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
        "%3, %4}], [%5];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(cluster_bar)
        : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *tm, uint32_t smem_src, int32_t x, int32_t y, int32_t z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N committed store groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Wait until at most N committed store groups are not yet complete (writes visible).
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory
// ---------------------------------------------------------------------------
// One full warp allocates `cols` (power of two, 32..512) TMEM columns; the base address
// is written to shared memory at `smem_result`.
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
    if (kCtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols)
                     : "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols)
                     : "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish() {
    if (kCtaGroup == 1) {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if (kCtaGroup == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    }
}

// ---------------------------------------------------------------------------
// tcgen05: UMMA descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes
// (64 halves) written by TMA with the 128-byte swizzle:
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4 (unused for swizzled K-major; 1)
//   bits [32,46) stride-dimension byte offset >> 4 = 1024 B between 8-row groups
//   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
// The tile base must be 1024-byte aligned. Stepping 16 halves (32 B) along K inside the
// swizzle atom adds 2 to the start-address field.
__host__ __device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// The same for an MN-major operand: 64 consecutive elements along the operand's row index are contiguous
// (one 128-byte line) and consecutive k sit 128 bytes apart, as TMA writes a box of {64 columns, 64 rows} of
// a K x N row-major matrix. An atom is 8 k-rows of 128 bytes; atoms follow each other every 1024 bytes
// along k (the stride field) and every `mn_stride_bytes` along the row index (the leading field), which is
// the size of one such box. Stepping 16 along K (two atoms) adds 2048 bytes = 128 to the address field.
__host__ __device__ __forceinline__ uint64_t umma_smem_desc_sw128_mn(uint32_t smem_addr, uint32_t mn_stride_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((mn_stride_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16: FP16 A and B (both K-major), FP32 accumulate.
//   bits [4,6)   D format (1 = F32)
//   bits [7,10)  A format (0 = F16)      bits [10,13) B format (0 = F16)
//   bit 15 / 16  A / B major (0 = K-major)
//   bits [17,23) N >> 3                  bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// The same with the B operand MN-major (bit 16).
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32_b_mn(uint32_t m, uint32_t n) {
    return umma_idesc_f16_f32(m, n) | (1u << 16);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
template <int kCtaGroup>
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    if (kCtaGroup == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Arrive on `bar` (this CTA) once every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Pair form: arrive on the barrier at the same offset in every CTA named in `cta_mask`.
// (A barrier arrive, not a data copy.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM -> registers
// ---------------------------------------------------------------------------
// Each lane reads its own TMEM lane (row): 16 consecutive FP32 columns starting at taddr.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Each lane reads its own TMEM lane (row): 32 consecutive FP32 columns starting at taddr.
// A warp can only touch TMEM lanes [32*(warp_id%4), 32*(warp_id%4)+32).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two FP32 -> packed FP16x2, round to nearest even (first argument in the low half).
__device__ __forceinline__ uint32_t pack_half2_rn(uint32_t lo_f32_bits, uint32_t hi_f32_bits) {
    __half2 h = __floats2half2_rn(__uint_as_float(lo_f32_bits), __uint_as_float(hi_f32_bits));
    return *reinterpret_cast<uint32_t *>(&h);
}

// L2-coherent (L1-bypassing) loads for data another CTA has just published.
__device__ __forceinline__ float4 ld_cg_f4(const float4 *p) {
    return __ldcg(p);
}

}  // namespace b200
