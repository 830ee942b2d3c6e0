/*
 * b200_hgemm -- C ABI of the sm_100a half-precision GEMM library.
 *
 *   C[M x N] = A[M x K] * B      FP16 in, FP32 accumulate (tensor memory), FP16 out
 *
 * Operand layouts are those of the cuda_hgemm entry points
 * `void kernel(half *A, half *B, half *C, size_t M, size_t N, size_t K)` (reference
 * src/main.cu:11-33; layouts src/common/tester.h:117-119):
 *   A  row-major, M rows of K contiguous halves            (lda = K)
 *   B  "col-major K x N": N rows of K contiguous halves    (ldb = K), element (k, n) at B[n*K + k]
 *   C  row-major, M rows of N contiguous halves            (ldc = N), fully overwritten (beta = 0)
 * alpha = 1, beta = 0, no batching and no strides, exactly like the reference kernels.
 *
 * All pointers are DEVICE pointers unless a function says otherwise. Calls are asynchronous
 * on `stream` and never synchronise; they may be issued back to back on one stream.
 * There is no CPU fallback and no alternate backend: on a device that is not sm_100 every
 * compute entry point returns B200_HGEMM_ERR_NO_SM100.
 *
 * Preconditions (checked, reported by return code): A, B, C 16-byte aligned; K % 8 == 0;
 * M, N, K >= 1. Tails in M, N and K (to a multiple of 8) are handled inside the kernels.
 */
#ifndef B200_HGEMM_H_
#define B200_HGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same type as cudaStream_t / CUstream; spelled out so that C callers need no CUDA headers. */
typedef struct CUstream_st *b200_stream_t;
/* Same type as cudaEvent_t / CUevent. */
typedef struct CUevent_st *b200_event_t;

enum {
    B200_HGEMM_OK = 0,
    B200_HGEMM_ERR_INVALID_ARG = -1,  /* null pointer or zero dimension */
    B200_HGEMM_ERR_UNSUPPORTED = -2,  /* shape or plan outside what the kernels implement */
    B200_HGEMM_ERR_MISALIGNED = -3,   /* pointer not 16-byte aligned */
    B200_HGEMM_ERR_NO_SM100 = -4,     /* current device is not compute capability 10.x */
    B200_HGEMM_ERR_CUDA = -5,         /* a CUDA runtime / driver call failed */
    B200_HGEMM_ERR_WORKSPACE = -6,    /* split-k workspace missing or too small */
    B200_HGEMM_ERR_DEVICE_WAIT = -7,  /* a kernel gave up on a bounded wait (b200_hgemm_synchronize, b200_mg_synchronize) */
    B200_HGEMM_ERR_TOO_LARGE = -8     /* size beyond a stated maximum of the entry point */
};

/* Kernel family a plan selects. */
enum {
    B200_VARIANT_CTA1 = 0,    /* tcgen05.mma cta_group::1, whole tiles, persistent */
    B200_VARIANT_CTA2 = 1,    /* tcgen05.mma cta_group::2 (CTA pair on a 256-row tile) */
    B200_VARIANT_STREAMK = 2, /* cta_group::1, k-ranges split across CTAs, FP32 workspace reduce */
    B200_VARIANT_SIMT = 3,    /* CUDA-core kernel for shapes the tensor path rejects (K % 8 != 0) */
    B200_VARIANT_CTA2_MCAST = 4, /* CTA pairs in clusters of four with the A slab delivered by TMA multicast;
                                   single-GPU processes only and off by default: it lives in libb200_hgemm_mc.so,
                                   which the library opens after b200_hgemm_enable_multicast(1)
                                   (B200_HGEMM_ERR_UNSUPPORTED otherwise); needs N % 8 == 0; A, B and C must be
                                   allocations of the GPU the call runs on */
    B200_VARIANT_SKINNY = 5,     /* M <= 128 (decode batches): B streams through the MMA's row operand and C is
                                   accumulated transposed; plan.bn = rows of A per tile (16, 32, 64 or 128, >= M),
                                   plan.parts = equal k-ranges per column tile (0 = library's choice); plan.group_m =
                                   columns of C per tile (a multiple of 8 up to 128; 0 = library's choice). More than
                                   one k-range is summed either on chip -- the k-ranges of a tile run as one
                                   thread-block cluster (at most 8 CTAs) and add their results through distributed
                                   shared memory: no workspace, no second kernel -- or from an FP32 workspace by a
                                   second kernel; both give the same bits. plan.grid = 1 asks for the cluster
                                   (B200_HGEMM_ERR_UNSUPPORTED when it would be larger than 8 CTAs), 2 for the
                                   workspace, 0 leaves it to the library (the cluster whenever it fits) */
    B200_VARIANT_HYBRID = 6,     /* as STREAMK, but every full wave of tiles (parts tiles each) is computed whole
                                   and only the tiles of the ragged last wave are cut into k-ranges */
    B200_VARIANT_SKINNY_PAIR = 7, /* as SKINNY on CTA pairs (cta_group::2): two neighbouring column tiles share
                                    the rows of A, each CTA staging half of them; same plan fields */
    B200_VARIANT_HYBRID_PAIR = 8  /* as HYBRID on CTA pairs: 256 x bn tiles (bn 128 or 256), the full waves whole, the
                                    tiles of the ragged last wave cut into k-ranges over all pairs (parts = pairs
                                    launched; 0 = one per two SMs) and summed from the FP32 workspace */
};

/* The dispatch decision for one shape. All fields are filled by b200_hgemm_select(); a
 * caller may edit them and pass the plan to b200_hgemm_ex(). */
typedef struct b200_hgemm_plan {
    int32_t variant;   /* B200_VARIANT_* */
    int32_t bn;        /* tile width in N: 64, 128, 192 or 256 (tile height is 128, or 256 per CTA pair); CTA2 also 160, 224,
                        * and 288, 320 (two MMAs side by side and a single accumulator: for shapes whose tiles then fit one wave).
                        * 512 with CTA2 or CTA2_MCAST selects the arrangement with 256 x 256 outputs per CTA
                        * instead: 512 x 256 tiles per pair (CTA2), 512 x 512 per group of four CTAs
                        * (CTA2_MCAST, which otherwise takes 256 only); both need N % 8 == 0 and tma_store = 1 */
    int32_t parts;     /* STREAMK: number of equal k-ranges = CTAs launched; 0 = one per SM */
    int32_t group_m;   /* rasterisation band height in row blocks; 0 = library default */
    int32_t tma_store; /* 1: epilogue writes C with TMA stores (needs N % 8 == 0); 0: plain stores */
    int32_t grid;      /* CTA1/CTA2: CTAs launched (0 = min(tiles, SMs)); informational for STREAMK;
                        * SKINNY/SKINNY_PAIR: how several k-ranges are summed (see B200_VARIANT_SKINNY) */
    int32_t stages;    /* CTA1/CTA2: depth of the operand ring; 0 = the kernel's default (its deepest). Shallower
                        * rings exist for measurements and the autotuner: CTA1 bn 256: 3, bn 128: 2, bn 64: 3;
                        * CTA2 bn 256: 4 or 5, bn 128: 3; anything else is B200_HGEMM_ERR_UNSUPPORTED */
} b200_hgemm_plan;

/* ---- compute entry points: each replaces one reference HGEMM_FUNC symbol ----------------
 * Reference interface replaced: src/main.cu:11 `HGEMM_FUNC(name)` and its 19 instances
 * (src/main.cu:13-33), called from src/common/tester.h:61 and :93. */

/* Auto-dispatching GEMM: picks a plan with b200_hgemm_select() and runs it.
 * Replaces the role of the reference's best kernel, mmaAsyncStage4 (src/mma/mma_async_stage4.cu:637-644). */
int b200_hgemm(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);

/* Fixed-variant entry points (log names B200-Tcgen05-1Cta / -2Cta / -SplitK / -StreamK); they
 * stand where the reference registers one symbol per kernel variant (src/main.cu:106-123). */
int b200_hgemm_cta1(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);
int b200_hgemm_cta2(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);
int b200_hgemm_splitk(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);
int b200_hgemm_streamk(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);

/* Stream-k GEMM that never allocates: its scratch (the FP32 partial tiles of split k-ranges) is a
 * static 16.06 MiB device array inside the library, held by every GPU the library is loaded on.
 * It has no counterpart in the reference, whose kernels need no scratch memory; it exists for
 * callers that may not call cudaMalloc where they need the GEMM (all device memory owned by a
 * pool, a serving loop that cannot afford an allocation's implicit synchronisation, a host
 * application that forbids allocations after start-up).
 * Limits: K % 8 == 0; ceil(M/128) * ceil(N/128) <= 16384 tiles, else B200_HGEMM_ERR_TOO_LARGE.
 * The first call on a device resolves the array's device address and should come before any
 * stream capture. Calls share the array: kernels of two calls that overlap on the GPU race.
 * A device-side wait expiry in this variant is recorded in the array's first word only, which
 * b200_hgemm_streamk_static_last_error() reads. */
int b200_hgemm_streamk_static(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                              b200_stream_t stream);
/* Synchronises the current device and returns the error word of the static array (0 = none, 1 = a
 * bounded wait expired inside b200_hgemm_streamk_static), clearing it. Allocates nothing. Like the
 * entry point it serves, it has no counterpart in the reference. */
int b200_hgemm_streamk_static_last_error(void);

/* Any-shape CUDA-core kernel with FP32 accumulation: the counterpart of the reference's
 * simtNaive (src/simt_naive.cu:9-32), with the bounds guard corrected. */
int b200_hgemm_simt(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);

/* Run an explicit plan. */
int b200_hgemm_ex(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, const b200_hgemm_plan *plan,
                  b200_stream_t stream);

/* GEMM with a fused epilogue: C = alpha * (A * B^T) + beta * c_in + bias, everything after the product in
 * FP32 on the accumulator before the one rounding to C's element type, which may be FP16, BF16 or FP32.
 * The reference fixes alpha = 1, beta = 0 and FP16 (src/cublas_tensor_op.cu:19-24) and has no counterpart;
 * this is the step either side of a GEMM in decode/prefill use. It runs on the kernel the dispatch picks for
 * the shape (short-A, single-CTA and pair tiles, k-ranges, 256 x 256 outputs per CTA) with two exceptions:
 * the multicast variants run as the same tiles on plain pairs, and FP32 output is written with plain stores
 * (the 256 x 256-per-CTA arrangement falls back to 128 x 256 per CTA for it). Needs K % 8 == 0. */
enum {
    B200_C_F16 = 0,  /* IEEE binary16, the reference's only output type */
    B200_C_BF16 = 1,
    B200_C_F32 = 2
};
typedef struct b200_hgemm_epilogue {
    float alpha;
    float beta;
    const void *bias; /* N halves (FP16), one per column of C, 16-byte aligned; or NULL */
    const void *c_in; /* M x N elements of C's type, row-major, 16-byte aligned, read when beta != 0; may be C itself; or NULL */
    int32_t c_type;   /* B200_C_*: element type of C and of c_in */
} b200_hgemm_epilogue;
int b200_hgemm_fused(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                     const b200_hgemm_epilogue *epilogue, b200_stream_t stream);
/* The same on an explicit plan (as b200_hgemm_ex). */
int b200_hgemm_fused_ex(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                        const b200_hgemm_epilogue *epilogue, const b200_hgemm_plan *plan, b200_stream_t stream);

/* The same product with B stored the other way round: B_kn is K rows of N contiguous halves (row-major K x N,
 * element (k, n) at B_kn[k*N + n]), as frameworks keep a weight matrix that is applied as x @ W. The reference
 * only has the K-contiguous form (src/common/tester.h:117-119, src/cublas_tensor_op.cu:22-24: OP_T on B). No copy
 * or transpose is made: TMA stages boxes of 64 k x 64 n and the MMA reads them as an MN-major operand. Runs on
 * the whole-tile kernels (single CTAs and CTA pairs); needs K % 8 == 0 and N % 8 == 0. */
int b200_hgemm_bkn(const void *A, const void *B_kn, void *C, size_t M, size_t N, size_t K, b200_stream_t stream);

/* `batch` products of one shape in one call: C_i = A_i * B_i with A_i = A + i * stride_a (strides in elements,
 * multiples of 8; matrices must not overlap), likewise B_i and C_i; stride_b = 0 multiplies every A_i by the
 * same B. The reference has no counterpart (no batch, no strides: src/main.cu:11, src/cublas_tensor_op.cu:22-24).
 * Stacks run as ONE launch of the whole-tile kernels over three-dimensional tensor maps, so that many small
 * products fill the GPU together; a shared B under densely stacked A and C is simply one product of
 * batch * M rows; what fits neither (K % 8 != 0, a shared B with gaps between the A_i) runs product by product. */
int b200_hgemm_batched(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, size_t batch,
                       size_t stride_a, size_t stride_b, size_t stride_c, b200_stream_t stream);

/* HOST-pointer GEMM: copies A and B to the device, runs b200_hgemm, copies C back and
 * synchronises. This is the path of reference Matrix (src/common/matrix.h:23-35 upload,
 * :83-85 moveToHost) + one kernel call, behind one entry point. Returns after C_host is complete. */
int b200_hgemm_host(const void *A_host, const void *B_host, void *C_host, size_t M, size_t N, size_t K);

/* The same with B already on the current device (complete, 16-byte aligned): only A goes up and C comes down.
 * For weights that stay resident, and for several GPUs, where each one uploads a share of B and the shares are
 * exchanged between the GPUs instead of every GPU pulling all of B over its own host link. Work queued on other
 * streams that produces B must have completed (or the caller must have synchronised) before the call. */
int b200_hgemm_host_a(const void *A_host, const void *B_device, void *C_host, size_t M, size_t N, size_t K);

/* The same for a B that is still being completed on the device when the call is made: the first upload of A waits
 * for the event `upload_after`, the first multiply for `gemm_after` (CUDA events the caller has recorded; either may
 * be NULL). With several GPUs a rank records `upload_after` behind the upload of its share of B and `gemm_after`
 * behind the exchange of the shares, and its rows of A travel over the host link while the other shares arrive
 * over NVLink. */
int b200_hgemm_host_a_after(const void *A_host, const void *B_device, void *C_host, size_t M, size_t N, size_t K,
                            b200_event_t upload_after, b200_event_t gemm_after);

/* ---- planning, workspace, status ------------------------------------------------------- */

/* Fills *plan with the library's choice for (M, N, K) on the current device. */
int b200_hgemm_select(size_t M, size_t N, size_t K, b200_hgemm_plan *plan);

/* Tuned plans. b200_hgemm_select() (and so b200_hgemm) first looks the shape up in a table of measured
 * plans, a text file with one "M N K variant bn parts group_m tma_store [stages]" line per shape that
 * `python -m cuda_hgemm_b200.autotune` writes: B200_HGEMM_PLAN_TABLE if set, else plan_table.txt in the
 * directory above the library's; B200_HGEMM_NO_PLAN_TABLE=1 disables it. This call replaces the table at run
 * time (NULL: empty table) and returns the number of entries read, or a negative status.
 * b200_hgemm_select_untuned() answers from the rules alone. */
int b200_hgemm_load_plan_table(const char *path);
int b200_hgemm_select_untuned(size_t M, size_t N, size_t K, b200_hgemm_plan *plan);

/* Bytes of device workspace `plan` needs for this shape (0 for whole-tile variants). */
size_t b200_hgemm_workspace_bytes(size_t M, size_t N, size_t K, const b200_hgemm_plan *plan);

/* Hands the library a caller-owned device workspace for the current device (256-byte aligned);
 * every stream-k call on that device then uses it, so such calls must be ordered with respect to
 * each other. With no workspace set the library keeps one workspace per stream, allocated and
 * grown on first need (cudaMalloc outside any stream capture), and calls on different streams
 * may overlap freely. Pass (NULL, 0) to go back to that. */
int b200_hgemm_set_workspace(void *workspace, size_t bytes);

/* The library keeps at most 64 of those per-stream workspaces on a device (32 MiB or more each); when
 * a 65th stream needs one, the workspace used longest ago changes hands (after a device synchronisation,
 * so that its previous owner's kernels are done with it). This call frees all of them on the current device, e.g.
 * after a burst of short-lived streams; returns how many were freed, or a negative status. */
int b200_hgemm_release_workspaces(void);

/* Synchronises the current device and returns the device-side error word (0 = none,
 * 1 = a bounded wait expired), clearing it. */
int b200_hgemm_last_device_error(void);

/* Waits for `stream` and reports what the kernels on it left in the device-side error word:
 * B200_HGEMM_OK, or B200_HGEMM_ERR_DEVICE_WAIT when a kernel gave up on a bounded wait (the word is
 * cleared). Unlike b200_hgemm_last_device_error() it waits for this stream only. The reference has
 * no counterpart: its launches are never checked (src/mma/mma_async_stage4.cu:643). */
int b200_hgemm_synchronize(b200_stream_t stream);

/* Whether `plan` can run for this shape in this process (B200_HGEMM_OK) or why not; no device is touched. */
int b200_hgemm_plan_supported(size_t M, size_t N, size_t K, const b200_hgemm_plan *plan);

/* The kernels that share operand loads between the CTAs of a cluster (B200_VARIANT_CTA2_MCAST, in
 * libb200_hgemm_mc.so) are OFF unless the process switches them on here (or starts with
 * B200_HGEMM_MULTICAST=1 in its environment). They are for processes that own ONE GPU, the
 * reference's model (its only device knob is -gpu_rank, src/main.cu:45,51): in a process that is one
 * rank of several (WORLD_SIZE or LOCAL_WORLD_SIZE > 1) or that has called b200_mg_create() with two or
 * more devices the switch is locked off for good, b200_hgemm_enable_multicast(1) returns
 * B200_HGEMM_ERR_UNSUPPORTED, b200_hgemm_select() never picks the variant and an explicit plan that
 * names it is refused. Also B200_HGEMM_ERR_UNSUPPORTED when the companion library is absent.
 * b200_hgemm_multicast_state(): 0 = off, 1 = on, 2 = locked off. */
int b200_hgemm_enable_multicast(int on);
int b200_hgemm_multicast_state(void);

const char *b200_hgemm_status_string(int status);
const char *b200_hgemm_version(void);

/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t b200_hgemm_launch_count(void);

/* ---- several GPUs from one process: row slabs of C, B replicated --------------------------
 * The reference is single-GPU (its only device knob is -gpu_rank, src/main.cu:45,51); these have no
 * counterpart there. C (and A) are cut into contiguous row slabs, one per device, with boundaries on
 * multiples of 128 rows (b200_mg_slab); every device multiplies its slab by its own copy of B with the
 * single-GPU dispatch, on a stream the handle owns; no data crosses GPUs during the multiply. The
 * launching thread loops over the devices (cudaSetDevice) and restores the device that was current. */
typedef struct b200_mg b200_mg;

/* `devices`: n distinct CUDA device ordinals, 1 <= n <= 64, every one an sm_100 GPU. */
int b200_mg_create(const int *devices, int n, b200_mg **out);
int b200_mg_destroy(b200_mg *mg);
int b200_mg_device_count(const b200_mg *mg);
/* Rows [*row0, *row0 + *rows) of C and A that device `index` (position in `devices`) owns; *rows may be 0. */
int b200_mg_slab(const b200_mg *mg, size_t M, int index, size_t *row0, size_t *rows);
/* A_slabs[i], B_replicas[i], C_slabs[i]: device pointers on devices[i] (A and C slabs as b200_mg_slab says,
 * B complete). Launches on every device and returns without synchronising. M is the row count of the whole C. */
int b200_mg_hgemm(b200_mg *mg, const void *const *A_slabs, const void *const *B_replicas, void *const *C_slabs, size_t M,
                  size_t N, size_t K);
/* Copies every slab of C into C_full[i] (M x N on devices[i]) for each i with C_full[i] != NULL, by peer copies
 * ordered after the multiply on the owning device's stream: a gather when one entry is set, an all-gather
 * when all are. */
int b200_mg_gather_c(b200_mg *mg, void *const *C_slabs, void *const *C_full, size_t M, size_t N);
/* Waits for everything launched through the handle; B200_HGEMM_ERR_DEVICE_WAIT when a kernel on any of
 * the devices gave up on a bounded wait (the error words are cleared). */
int b200_mg_synchronize(b200_mg *mg);
/* After b200_mg_synchronize: device time of the last b200_mg_hgemm, the maximum over the devices (ms). */
int b200_mg_elapsed_ms_max(b200_mg *mg, float *ms);

/* ---- host-side helpers exposed for tests (no GPU needed) -------------------------------- */

/* The row slab of device `index` of `n` for a C of M rows: the rule b200_mg_slab applies (no handle needed). */
int b200_partition_slab(size_t M, int n, int index, size_t *row0, size_t *rows);
/* Tile rasterisation: linear tile id -> (m_blk, n_blk). */
void b200_sched_tile_coord(uint32_t tile, uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m, uint32_t *m_blk,
                           uint32_t *n_blk);
/* The same through the kernels' own path: the launch's raster constants worked out once, divisions by
 * multiplication (must agree with b200_sched_tile_coord everywhere). And that division on its own: n / d, d >= 1. */
void b200_sched_tile_coord_fast(uint32_t tile, uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m, uint32_t *m_blk,
                                uint32_t *n_blk);
uint32_t b200_debug_fast_div(uint32_t n, uint32_t d);
/* Stream-K: writes up to `cap` segments {tile, kb0, kb1} of part `part` to out[3*i..]; returns the count. */
uint32_t b200_sched_segments(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t *out,
                             uint32_t cap);
/* Stream-K: first and last part contributing to `tile`, and the workspace slot of (part, tile). */
void b200_sched_contributors(uint32_t tile, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t *first,
                             uint32_t *last);
uint32_t b200_sched_partial_slot(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t tile);
/* Needs a GPU: launches one CTA that waits, for at most `limit_ms` (1..1000), on a barrier nothing
 * arrives on -- the way a kernel of this library would notice a protocol failure -- and raises the
 * device error word. b200_hgemm_last_device_error() then returns 1 and the device stays usable. */
int b200_debug_wait_expiry(uint32_t limit_ms, b200_stream_t stream);
/* The same, reported where b200_hgemm_streamk_static reports: in the first word of its static array
 * (b200_hgemm_streamk_static_last_error() then returns 1). Allocates nothing. */
int b200_debug_wait_expiry_static(uint32_t limit_ms, b200_stream_t stream);
/* For tests of the short-A kernels' fall-back: with clusters > 0 the library behaves as if the device could hold
 * only that many thread-block clusters at once, whatever their size, so its own choice of summing k-ranges inside
 * clusters gives way to the workspace form when there are more clusters than that; 0 restores what the device says. */
void b200_debug_cluster_capacity(int clusters);
/* tcgen05 descriptor encoders (instruction descriptor; shared-memory matrix descriptor). */
uint32_t b200_debug_idesc(uint32_t m, uint32_t n);
uint64_t b200_debug_smem_desc(uint32_t smem_addr);

#ifdef __cplusplus
}
#endif

#endif /* B200_HGEMM_H_ */
