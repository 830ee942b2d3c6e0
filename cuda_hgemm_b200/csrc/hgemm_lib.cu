// Host side of the library: per-device state, tensor-map cache, shape -> plan selection,
// kernel launches and the extern "C" entry points declared in include/b200_hgemm.h.
//
// What it stands in for in the reference: the per-kernel launchers with their one-time
// shared-memory opt-in (e.g. src/mma/mma_async_stage4.cu:619-644) and the kernel table of
// src/main.cu:11-33. Unlike those, nothing here exits the process: errors are return codes.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <math.h>
#include <string.h>

#include <atomic>
#include <initializer_list>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200_hgemm.h"
#include "gemm_kernel.cuh"
#include "gemm_kernel_big.cuh"
#include "gemm_kernel_skinny.cuh"

namespace b200 {

// ------------------------------------------------------------------------------------------
// per-device state
// ------------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
constexpr size_t kMaxOwnedWorkspace = size_t(1) << 30;  // the library never grows its own workspace past 1 GiB
constexpr size_t kCounterBytes = 64 * 1024;             // reserved header at the front of the workspace (no kernel uses it now)
constexpr uint32_t kMaxCountedTiles = kCounterBytes / 4;  // most tiles the allocation-free stream-k entry point accepts

struct TensorMapKey {
    const void *ptr;
    uint64_t rows, cols;
    uint32_t box_rows, box_cols;
    bool swizzle;
    uint64_t batch, batch_stride;  // stacks of matrices: how many, and elements from one to the next (1, 0: a single matrix)
    bool operator==(const TensorMapKey &o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
               swizzle == o.swizzle && batch == o.batch && batch_stride == o.batch_stride;
    }
};

struct TensorMapSlot {
    bool used = false;
    uint64_t last_use = 0;
    TensorMapKey key{};
    CUtensorMap map{};
};
constexpr size_t kTensorMapWays = 4;

struct DeviceState {
    std::mutex mu;
    bool probed = false;       // attributes known and the error word allocated
    bool attrs_known = false;  // sm100 / sm_count filled in (no allocation needed for that)
    bool sm100 = false;
    int sm_count = 0;
    uint32_t *error_word = nullptr;
    // stream-k workspace [64 KiB header | FP32 partial slots]: either one the caller handed over
    // (ws), or one per stream that the library allocates and grows itself, so that GEMMs running
    // on different streams at the same time never share partial-tile slots
    void *ws = nullptr;
    size_t ws_bytes = 0;
    struct StreamWorkspace {
        cudaStream_t stream;
        void *ptr;
        size_t bytes;
        uint64_t last_use;
    };
    std::vector<StreamWorkspace> owned_ws;
    uint64_t ws_clock = 0;
    // staging buffers of the host-pointer entry point
    void *host_a = nullptr, *host_b = nullptr, *host_c = nullptr;
    size_t host_a_bytes = 0, host_b_bytes = 0, host_c_bytes = 0;
    cudaStream_t host_stream[3] = {nullptr, nullptr, nullptr};  // upload, GEMMs, download
    cudaEvent_t host_event[2] = {nullptr, nullptr};
    bool attr_set[96] = {};
    int max_clusters[96] = {};
    int ck_clusters[16][9] = {};  // short-A kernels that sum inside clusters: clusters of each size the device holds at once (-1: none)  // CTA pairs the device can keep resident at once, per pair kernel
    TensorMapSlot tm_cache[64 * kTensorMapWays];
    uint64_t tm_clock = 0;
};

static DeviceState g_dev[kMaxDevices];
#ifdef B200_TIMELINE
// profiling builds only: device buffer of per-CTA time stamps, set through b200_debug_set_timeline
static unsigned long long *g_timeline = nullptr;
extern "C" void b200_debug_set_timeline(unsigned long long *buf) { g_timeline = buf; }
#endif
static std::atomic<uint64_t> g_launches{0};

// With B200_HGEMM_DEBUG set in the environment, every failing CUDA call is named on stderr
// (the C ABI itself only returns B200_HGEMM_ERR_CUDA).
static bool cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    static const bool verbose = (getenv("B200_HGEMM_DEBUG") != nullptr);
    if (verbose) fprintf(stderr, "[b200_hgemm] %s failed: %s\n", what, cudaGetErrorString(e));
    cudaGetLastError();
    return false;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess) {
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Compute capability and SM count of `dev`, asked for once; allocates nothing. Call with st.mu held.
static int probe_attributes_locked(DeviceState &st, int dev) {
    if (st.attrs_known) return B200_HGEMM_OK;
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return B200_HGEMM_ERR_CUDA;
    }
    st.sm100 = (major == 10);
    st.sm_count = sms;
    st.attrs_known = true;
    return B200_HGEMM_OK;
}

static int current_state(DeviceState **out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return B200_HGEMM_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return B200_HGEMM_ERR_CUDA;
    // The tensor-map encoder is a driver call and wants a context current on the calling thread; a
    // thread that has made no runtime call yet has none. Binding the device's primary context
    // once per thread (and again when the thread switches device) costs nothing afterwards.
    static thread_local int bound_dev = -1;
    if (bound_dev != dev) {
        if (!cuda_ok(cudaSetDevice(dev), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaFree(nullptr), "cudaFree(nullptr)")) return B200_HGEMM_ERR_CUDA;
        bound_dev = dev;
    }
    DeviceState &st = g_dev[dev];
    std::lock_guard<std::mutex> lock(st.mu);
    if (!st.probed) {
        const int rc = probe_attributes_locked(st, dev);
        if (rc != B200_HGEMM_OK) return rc;
        if (st.sm100) {
            if (!cuda_ok(cudaMalloc(&st.error_word, 256), "cudaMalloc")) return B200_HGEMM_ERR_CUDA;
            if (!cuda_ok(cudaMemset(st.error_word, 0, 256), "cudaMemset")) return B200_HGEMM_ERR_CUDA;
        }
        st.probed = true;
    }
    *out = &st;
    return B200_HGEMM_OK;
}

// A 2-D FP16 tensor of `rows` x `cols` (cols contiguous) viewed through boxes of
// box_rows x box_cols, with the 128-byte swizzle (box_cols = 64) or, for plain row-major staging
// tiles, without. Out-of-range elements read as zero and are dropped on store. The cache is 4-way
// set-associative (64 sets): a handful of operands in rotation never evict each other.
static int get_tensor_map(DeviceState &st, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
                          uint32_t box_cols, CUtensorMap *out, bool swizzle = true, uint64_t batch = 1, uint64_t batch_stride = 0) {
    TensorMapKey key{ptr, rows, cols, box_rows, box_cols, swizzle, batch, batch_stride};
    size_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
    h ^= rows * 0xC2B2AE3D27D4EB4Full + cols * 0x165667B19E3779F9ull + box_rows * 131u + box_cols + (swizzle ? 0u : 77u) +
         batch * 0x9E3779B1ull + batch_stride * 0x85EBCA77ull;
    const size_t set = ((h >> 20) & 63u) * kTensorMapWays;
    std::lock_guard<std::mutex> lock(st.mu);
    TensorMapSlot *slot = nullptr;
    for (size_t w = 0; w < kTensorMapWays; ++w) {
        TensorMapSlot &cand = st.tm_cache[set + w];
        if (cand.used && cand.key == key) {
            cand.last_use = ++st.tm_clock;
            *out = cand.map;
            return B200_HGEMM_OK;
        }
        // the victim, should there be no hit: a free way, else the one used longest ago
        if (!slot || (slot->used && (!cand.used || cand.last_use < slot->last_use))) slot = &cand;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return B200_HGEMM_ERR_CUDA;
    // a stack of matrices is a third dimension; a stack of one with stride 0 stays two-dimensional
    const bool stacked = batch > 1 || batch_stride != 0;
    cuuint64_t dims[3] = {cols, rows, batch};
    cuuint64_t strides[2] = {cols * sizeof(__half), (batch_stride ? batch_stride : rows * cols) * sizeof(__half)};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t elem_strides[3] = {1, 1, 1};
    CUresult r = enc(&slot->map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, stacked ? 3 : 2, const_cast<void *>(ptr), dims, strides, box,
                     elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        slot->used = false;
        if (getenv("B200_HGEMM_DEBUG")) fprintf(stderr, "[b200_hgemm] cuTensorMapEncodeTiled failed: CUresult %d\n", static_cast<int>(r));
        return B200_HGEMM_ERR_CUDA;
    }
    slot->used = true;
    slot->key = key;
    slot->last_use = ++st.tm_clock;
    *out = slot->map;
    return B200_HGEMM_OK;
}

// ------------------------------------------------------------------------------------------
// optional single-GPU companion library (the kernel variants whose operand loads are shared
// between the CTAs of a cluster)
// ------------------------------------------------------------------------------------------
// It is a separate shared object next to this one so that it can be left out wholesale, and it is
// OFF unless the process asks for it (b200_hgemm_enable_multicast(1), or B200_HGEMM_MULTICAST=1 in
// the environment). A process that drives two or more GPUs can never switch it on: the kernels'
// tensor maps must cover the memory of the one GPU they run on, and a process that owns one GPU
// is the one setting in which that holds by construction (the reference's model: one device per
// process, src/main.cu:45,51). Such a process is recognised by
//   * WORLD_SIZE or LOCAL_WORLD_SIZE > 1 in the environment (one rank of several), or
//   * a b200_mg_create() call that names two or more devices,
// and either locks the switch in the off position for the rest of the process's life.
typedef int (*McLaunchFn)(const void *params, void *stream, int use_pdl);

struct McEntryPoints {
    McLaunchFn launch256 = nullptr;  // 256 x 512 super-tiles, 128 x 256 per CTA
    McLaunchFn launch512 = nullptr;  // 512 x 512 super-tiles, 256 x 256 per CTA
};

enum : int { kMcOff = 0, kMcOn = 1, kMcLocked = 2 };
static std::atomic<int> g_mc_state{kMcOff};
static std::once_flag g_mc_env_once;

static bool env_int_above_one(const char *name) {
    const char *v = getenv(name);
    return v && atol(v) > 1;
}

// The companion's entry points; the library is opened on first request only.
static const McEntryPoints &mc_entry_points() {
    static McEntryPoints ep = []() -> McEntryPoints {
        McEntryPoints e;
        Dl_info info;
        if (!dladdr(reinterpret_cast<const void *>(&g_launches), &info) || !info.dli_fname) return e;
        std::string path(info.dli_fname);
        const size_t slash = path.rfind('/');
        path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/libb200_hgemm_mc.so";
        void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!h) return e;
        e.launch256 = reinterpret_cast<McLaunchFn>(dlsym(h, "b200_mc_launch"));
        e.launch512 = reinterpret_cast<McLaunchFn>(dlsym(h, "b200_mc512_launch"));
        return e;
    }();
    return ep;
}

static void mc_lock_off() {
    g_mc_state.store(kMcLocked, std::memory_order_release);
}

static int mc_enable(bool on) {
    if (g_mc_state.load(std::memory_order_acquire) == kMcLocked) return on ? B200_HGEMM_ERR_UNSUPPORTED : B200_HGEMM_OK;
    if (!on) {
        int expected = kMcOn;
        g_mc_state.compare_exchange_strong(expected, kMcOff);
        return B200_HGEMM_OK;
    }
    if (getenv("B200_HGEMM_NO_MULTICAST")) return B200_HGEMM_ERR_UNSUPPORTED;
    const McEntryPoints &ep = mc_entry_points();
    if (!ep.launch256 || !ep.launch512) return B200_HGEMM_ERR_UNSUPPORTED;
    int expected = kMcOff;
    g_mc_state.compare_exchange_strong(expected, kMcOn);  // loses against a lock taken meanwhile
    return g_mc_state.load(std::memory_order_acquire) == kMcOn ? B200_HGEMM_OK : B200_HGEMM_ERR_UNSUPPORTED;
}

// The switch as the environment sets it, read once: ranks of a multi-process job lock it off,
// B200_HGEMM_MULTICAST=1 asks for it.
static int mc_state() {
    std::call_once(g_mc_env_once, []() {
        if (env_int_above_one("WORLD_SIZE") || env_int_above_one("LOCAL_WORLD_SIZE")) {
            mc_lock_off();
        } else if (const char *v = getenv("B200_HGEMM_MULTICAST")) {
            if (atoi(v) != 0) mc_enable(true);
        }
    });
    return g_mc_state.load(std::memory_order_acquire);
}

// The launcher of the multicast kernel for this arrangement, or null when the process may not use it.
static McLaunchFn mc_launch_fn(int bn = 256) {
    if (mc_state() != kMcOn) return nullptr;
    return bn == 512 ? mc_entry_points().launch512 : mc_entry_points().launch256;
}

// ------------------------------------------------------------------------------------------
// plans
// ------------------------------------------------------------------------------------------
static inline uint32_t ceil_div_u32(uint64_t a, uint64_t b) {
    return static_cast<uint32_t>((a + b - 1) / b);
}

// STREAMK and HYBRID run the same kernel; HYBRID walks the full waves of tiles whole first. HYBRID_PAIR is
// HYBRID on CTA pairs (256-row tiles).
static bool plan_cuts_k(const b200_hgemm_plan &pl) {
    return pl.variant == B200_VARIANT_STREAMK || pl.variant == B200_VARIANT_HYBRID || pl.variant == B200_VARIANT_HYBRID_PAIR;
}

// CTAs that work on one tile together.
static int plan_cg(const b200_hgemm_plan &pl) {
    return (pl.variant == B200_VARIANT_CTA2 || pl.variant == B200_VARIANT_HYBRID_PAIR) ? 2 : 1;
}

static bool plan_is_tensor(const b200_hgemm_plan &pl) {
    return pl.variant == B200_VARIANT_CTA1 || pl.variant == B200_VARIANT_CTA2 || plan_cuts_k(pl) ||
           pl.variant == B200_VARIANT_CTA2_MCAST || pl.variant == B200_VARIANT_SKINNY ||
           pl.variant == B200_VARIANT_SKINNY_PAIR;
}

static int validate_plan(const b200_hgemm_plan &pl, size_t N, size_t K) {
    if (pl.variant == B200_VARIANT_SIMT) return B200_HGEMM_OK;
    if (!plan_is_tensor(pl)) return B200_HGEMM_ERR_UNSUPPORTED;
    if (pl.variant == B200_VARIANT_SKINNY || pl.variant == B200_VARIANT_SKINNY_PAIR) {
        // bn is the number of rows of A a tile holds (M may not exceed it; checked where M is known)
        if (pl.bn != 16 && pl.bn != 32 && pl.bn != 64 && pl.bn != 128) return B200_HGEMM_ERR_UNSUPPORTED;
        // group_m is the width of a column tile here: a multiple of 8 from 8 to 128, or 0 for the library's choice
        if (pl.group_m != 0 && (pl.group_m < 8 || pl.group_m > 128 || pl.group_m % 8 != 0)) return B200_HGEMM_ERR_UNSUPPORTED;
        // grid names how several k-ranges are summed: 0 the library's choice, 1 inside clusters, 2 through the workspace
        if (pl.grid > 2) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.variant == B200_VARIANT_CTA2_MCAST) {
        // bn names the CTA arrangement here: 256 = 128 x 256 per CTA, 512 = 256 x 256 per CTA
        if ((pl.bn != 256 && pl.bn != 512) || N % 8 != 0 || !mc_launch_fn(pl.bn)) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.variant == B200_VARIANT_CTA2 && pl.bn == 512) {
        // 256 x 256 outputs per CTA, 512 x 256 per pair; its epilogue is TMA stores only
        if (N % 8 != 0 || !pl.tma_store) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.bn == 192) {
        // whole tiles only: between 128 and 256 for shapes whose tile count would leave a wave ragged
        if (plan_cuts_k(pl)) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.bn == 160 || pl.bn == 224) {
        // two more widths for the same purpose, on CTA pairs only
        if (pl.variant != B200_VARIANT_CTA2) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.bn == 288 || pl.bn == 320) {
        // wider than one MMA: two MMAs side by side in one accumulator that fills tensor memory alone; CTA pairs,
        // the default ring only
        if (pl.variant != B200_VARIANT_CTA2 || pl.stages != 0) return B200_HGEMM_ERR_UNSUPPORTED;
    } else if (pl.bn != 64 && pl.bn != 128 && pl.bn != 256) {
        return B200_HGEMM_ERR_UNSUPPORTED;
    }
    if (pl.variant == B200_VARIANT_CTA2 && pl.bn == 64) return B200_HGEMM_ERR_UNSUPPORTED;
    if (pl.variant == B200_VARIANT_HYBRID_PAIR && pl.bn != 128 && pl.bn != 256) return B200_HGEMM_ERR_UNSUPPORTED;
    if (K % 8 != 0) return B200_HGEMM_ERR_UNSUPPORTED;  // TMA row pitch must be a multiple of 16 bytes
    const bool short_a = pl.variant == B200_VARIANT_SKINNY || pl.variant == B200_VARIANT_SKINNY_PAIR;
    if (pl.tma_store && N % 8 != 0 && !short_a) return B200_HGEMM_ERR_UNSUPPORTED;  // (the short-A kernels then store by element)
    if (pl.parts < 0 || pl.group_m < 0 || pl.grid < 0 || pl.stages < 0) return B200_HGEMM_ERR_INVALID_ARG;
    if (pl.stages != 0) {
        // ring depths other than the default exist for the whole-tile kernels only: the default or one or two less
        const int def = pl.variant == B200_VARIANT_CTA1 ? (pl.bn == 128 ? 3 : pl.bn == 192 ? 0 : 4)
                        : pl.variant == B200_VARIANT_CTA2 ? (pl.bn == 256 ? 6 : pl.bn == 128 ? 4 : 0) : 0;
        const int least = (pl.variant == B200_VARIANT_CTA2 && pl.bn == 256) ? 4 : def - 1;
        if (def == 0 || pl.stages > def || pl.stages < least) return B200_HGEMM_ERR_UNSUPPORTED;
    }
    return B200_HGEMM_OK;
}

// k-blocks per pipeline stage of the kernel a plan runs. Tiles narrower than 256 columns take two:
// the thread that issues the MMAs spends about 0.28 us per stage on its own instructions (a
// barrier wait, four MMAs, a commit; measured with one CTA alone on the GPU, the same for every
// tile width), which the four MMAs of a 256-column slab cover and those of a narrower slab do not;
// one wait and one commit per two k-blocks brought 128 x 64 tiles from 0.28 to 0.20 us per k-block
// and the M = 128 decode shape from 3.8 to 4.2 TB/s. The kernels count k in stages, so everything
// that cuts k-ranges (stream-k ranges, workspace sizes) counts the same units.
static uint32_t plan_kps(const b200_hgemm_plan &pl) {
    if (pl.variant == B200_VARIANT_HYBRID_PAIR) return pl.bn == 128 ? 2u : 1u;
    if (pl.variant == B200_VARIANT_CTA1 || plan_cuts_k(pl)) return (pl.bn == 128 || pl.bn == 64) ? 2u : 1u;
    if (pl.variant == B200_VARIANT_CTA2) return (pl.bn == 128 || pl.bn == 160 || pl.bn == 192 || pl.bn == 224) ? 2u : 1u;
    return 1u;
}

static uint32_t plan_k_units(const b200_hgemm_plan &pl, size_t K) {
    return ceil_div_u32(K, 64u * plan_kps(pl));
}

static uint32_t streamk_parts(const b200_hgemm_plan &pl, const DeviceState &st, uint32_t tiles, uint32_t k_blocks) {
    uint64_t units = static_cast<uint64_t>(tiles) * k_blocks;
    uint64_t parts = pl.parts > 0 ? static_cast<uint64_t>(pl.parts) : static_cast<uint64_t>(st.sm_count / plan_cg(pl));
    if (parts > units) parts = units;
    if (parts < 1) parts = 1;
    return static_cast<uint32_t>(parts);
}

// ------------------------------------------------------------------------------------------
// tuned plans: shapes whose best plan was measured (autotune.py) override the rules below
// ------------------------------------------------------------------------------------------
// A text file, one line per shape: "M N K variant bn parts group_m tma_store [stages]"; '#' starts a comment.
// It is read once, from B200_HGEMM_PLAN_TABLE if that is set, else from plan_table.txt in the
// directory above the one this library lies in (the package directory); B200_HGEMM_NO_PLAN_TABLE
// turns it off; b200_hgemm_load_plan_table() replaces it at run time. An entry that the
// running configuration cannot serve (the multicast companion is absent) is skipped at look-up.
struct TunedPlan {
    uint64_t m, n, k;
    b200_hgemm_plan plan;
};
static std::mutex g_table_mu;
static std::vector<TunedPlan> g_table;
static bool g_table_loaded = false;

static int read_plan_table(const char *path, std::vector<TunedPlan> *out) {
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    char line[256];
    int entries = 0;
    while (fgets(line, sizeof(line), f)) {
        char *hash = strchr(line, '#');
        if (hash) *hash = 0;
        unsigned long long m, n, k;
        int variant, bn, parts, group_m, tma_store, stages = 0;
        if (sscanf(line, "%llu %llu %llu %d %d %d %d %d %d", &m, &n, &k, &variant, &bn, &parts, &group_m, &tma_store, &stages) < 8) continue;
        TunedPlan t;
        t.m = m;
        t.n = n;
        t.k = k;
        memset(&t.plan, 0, sizeof(t.plan));
        t.plan.variant = variant;
        t.plan.bn = bn;
        t.plan.parts = parts;
        t.plan.group_m = group_m;
        t.plan.tma_store = tma_store;
        t.plan.stages = stages;
        out->push_back(t);
        ++entries;
    }
    fclose(f);
    return entries;
}

static void load_default_plan_table_locked() {
    g_table_loaded = true;
    if (getenv("B200_HGEMM_NO_PLAN_TABLE")) return;
    if (const char *env = getenv("B200_HGEMM_PLAN_TABLE")) {
        read_plan_table(env, &g_table);
        return;
    }
    Dl_info info;
    if (!dladdr(reinterpret_cast<const void *>(&g_launches), &info) || !info.dli_fname) return;
    std::string path(info.dli_fname);
    size_t slash = path.rfind('/');
    path = slash == std::string::npos ? std::string(".") : path.substr(0, slash);
    read_plan_table((path + "/../plan_table.txt").c_str(), &g_table);
}

static bool tuned_plan(size_t M, size_t N, size_t K, b200_hgemm_plan *pl) {
    std::lock_guard<std::mutex> lock(g_table_mu);
    if (!g_table_loaded) load_default_plan_table_locked();
    for (const TunedPlan &t : g_table) {
        if (t.m == M && t.n == N && t.k == K) {
            if (validate_plan(t.plan, N, K) != B200_HGEMM_OK) return false;
            if ((t.plan.variant == B200_VARIANT_SKINNY || t.plan.variant == B200_VARIANT_SKINNY_PAIR) &&
                M > static_cast<size_t>(t.plan.bn)) {
                return false;
            }
            *pl = t.plan;
            return true;
        }
    }
    return false;
}

// Shape -> plan, from measurements on B200 (square sizes 256..16384 in both timing protocols of
// abtest.py, the decode shapes, the prefill shape):
//  * M <= 64: the short-A kernel (B on the MMA's row operand);
//  * 65 <= M <= 128 (decode-like, HBM-bound): the short-A kernel on CTA pairs when B is large; for small
//    problems whole 128-wide tiles when they cover most SMs, else equal k-ranges over all SMs with the
//    FP32 workspace reduce;
//  * two or more full waves of CTA pairs on 256 x 256 tiles: those pairs, or - for long runs with long
//    k - 256 x 256 outputs per CTA (pairs on 512 x 256, groups of four on 512 x 512 with A multicast),
//    whichever fills its waves best after what the larger tiles gain under the power cap;
//  * in between: the candidate with the smallest estimated time among single-CTA tiles of three
//    widths, pairs on 256 x 256, 256 x 224 and 256 x 192, and stream-k.
static void select_plan(const DeviceState &st, size_t M, size_t N, size_t K, b200_hgemm_plan *pl, bool use_table = true) {
    memset(pl, 0, sizeof(*pl));
    if (K % 8 != 0) {
        pl->variant = B200_VARIANT_SIMT;
        return;
    }
    if (use_table && tuned_plan(M, N, K, pl)) return;
    const uint32_t sms = st.sm_count > 0 ? static_cast<uint32_t>(st.sm_count) : 148u;
    pl->tma_store = (N % 8 == 0) ? 1 : 0;
    pl->group_m = 0;
    const uint64_t m_blocks = ceil_div_u32(M, 128);
    const uint64_t k_blocks = ceil_div_u32(K, 64);
    const uint64_t tiles256 = m_blocks * ceil_div_u32(N, 256);
    const uint64_t tiles128 = m_blocks * ceil_div_u32(N, 128);

    if (M <= 64) {
        // decode batches: B through the MMA's row operand, deeper ring, k cut only when the column tiles
        // are few (measured against the 128-row tiles below at N = 14336, K = 4096 and the transpose:
        // +18 % at M = 16, +10 % at M = 64)
        pl->variant = B200_VARIANT_SKINNY;
        pl->bn = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        return;
    }
    if (M <= 128 && N >= 2048 && K >= 1024) {
        // 65 ... 128 rows against a large weight matrix: the short-A kernel on CTA pairs, which fetch the rows
        // of A once per pair (measured at N = 14336, K = 4096, M = 128: 26.3 us against 28.0 for 128-row tiles
        // of single CTAs; at N = 4096, K = 14336 with four k-ranges: 30.6 against 33.7 for stream-k)
        // Where the column tiles are so few that k would be cut into three or more ranges, single CTAs instead:
        // (at most) four k-ranges of a tile are one cluster that sums on chip (pairs would need clusters of six
        // or eight, which the GPU cannot hold all at once). Measured at N = 4096, K = 14336, M = 128: 28.4 us against 30.7 for pairs with the workspace.
        const uint32_t col_tiles = ceil_div_u32(N, 128);
        const uint32_t k_ranges = static_cast<uint64_t>(col_tiles) * 5 < 3ull * sms ? sms / col_tiles : 1u;
        pl->variant = k_ranges >= 3 ? B200_VARIANT_SKINNY : B200_VARIANT_SKINNY_PAIR;
        pl->bn = 128;
        return;
    }
    if (M <= 128) {
        if (tiles128 * 4 >= 3ull * sms) {  // e.g. N = 14336: 112 tiles on 148 SMs
            pl->variant = B200_VARIANT_CTA1;
            pl->bn = 128;
        } else if (k_blocks >= 8) {
            pl->variant = B200_VARIANT_STREAMK;
            pl->bn = (tiles128 * k_blocks >= 4ull * sms) ? 128 : 64;
        } else {
            pl->variant = B200_VARIANT_CTA1;
            pl->bn = 64;
        }
        return;
    }

    const uint64_t pairs256 = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 256);
    const uint64_t pair_slots = sms / 2;
    const double kb = static_cast<double>(k_blocks);
    auto waves = [](uint64_t work, uint64_t slots) { return static_cast<double>((work + slots - 1) / slots); };

    if (pairs256 >= 2 * pair_slots) {
        // Two or more full waves of CTA pairs: the tensor-bound regime. 256 x 256 tiles on pairs, unless
        // the arrangements with 256 x 256 outputs per CTA apply: 512 x 256 tiles on pairs, or 512 x 512
        // tiles on groups of four CTAs when the single-GPU companion library with the multicast kernel
        // is there. Those move fewer bytes per flop, which under the power cap means a higher clock:
        // +10 % at 16384^3, +4 % at 8192 x 8192 x 2048, level at 4096^3, and behind below that (the run
        // is over before the cap bites), at K < 1536 (the tensor pipe waits about a microsecond per tile
        // for the epilogue to drain tensor memory) and wherever their last wave is emptier (3840^3,
        // 7168^3). Their epilogue is TMA stores only (N % 8 == 0). Measured with abtest.py, both protocols.
        pl->variant = B200_VARIANT_CTA2;
        pl->bn = 256;
        const double flops = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
        if (N % 8 == 0 && k_blocks >= 24 && flops >= 2.0 * 4096.0 * 4096.0 * 4096.0) {
            // share of the launched tile area that is output, last wave included
            auto fill = [&](uint64_t tiles, uint64_t slots, double tile_area) {
                return static_cast<double>(M) * static_cast<double>(N) / (waves(tiles, slots) * static_cast<double>(slots) * tile_area);
            };
            const uint64_t tiles_big = static_cast<uint64_t>(ceil_div_u32(M, 512)) * ceil_div_u32(N, 256);
            const uint64_t tiles_mc = static_cast<uint64_t>(ceil_div_u32(M, 512)) * ceil_div_u32(N, 512);
            const double f256 = fill(pairs256, pair_slots, 256.0 * 256.0);
            // left-over tiles that fit one wave as 256 x 256 halves run on the 128 x 256-per-CTA kernel behind the
            // full waves (launch_big_with_tail): a little over half a wave's time instead of a whole one
            const uint64_t big_rest = tiles_big % pair_slots;
            const bool big_tail = tiles_big >= pair_slots && big_rest != 0 && 2 * big_rest <= pair_slots;
            const double big_waves = big_tail ? static_cast<double>(tiles_big / pair_slots) + 0.55 : waves(tiles_big, pair_slots);
            const double fbig = static_cast<double>(M) * static_cast<double>(N) /
                                (big_waves * static_cast<double>(pair_slots) * 512.0 * 256.0);
            const double fmc = mc_launch_fn(512) ? fill(tiles_mc, sms / 4, 512.0 * 512.0) : 0.0;
            // what the larger tiles gain at equal fill grows with the length of the run (measured:
            // pairs +0.5 % at 4096^3, +4 % at 8192^3, +7 % at 16384^3; groups of four 2 % more)
            const double doublings = log2(flops / (2.0 * 4096.0 * 4096.0 * 4096.0));
            const double gain_big = 0.005 + 0.012 * doublings;
            const double gain_mc = gain_big + 0.02;
            const double s256 = f256, sbig = fbig * (1.0 + gain_big), smc = fmc * (1.0 + gain_mc);
            if (smc > s256 && smc >= sbig) {
                pl->variant = B200_VARIANT_CTA2_MCAST;
                pl->bn = 512;
            } else if (sbig > s256) {
                pl->bn = 512;
            }
        }
        return;
    }

    // Fewer tiles than that: pick by estimated time. Microseconds per 64-wide k-block of one
    // tile (measured on B200 at 1024..3072: these sizes are bound by the rate at which one SM can
    // pull operand slabs from L2, not by the tensor pipe), plus a fixed cost per kernel; the
    // stream-k estimates carry the cost of writing and summing the partial tiles (measured at
    // 2304 and 2560: 660 and 775 TFLOP/s against 850 and 1030 for whole tiles).
    struct Candidate {
        int variant, bn;
        double us;
    };
    const uint64_t tiles64 = m_blocks * ceil_div_u32(N, 64);
    // every range leaves up to two FP32 partial tiles, each written once and read once through L2
    // (about 4 TB/s for this pattern): with full-height tiles that costs more than a ragged last
    // wave does, so stream-k only wins here when the tiles are few and k is long
    auto partial_us = [&](int bn) { return 2.0 * sms * 2.0 * (128.0 * bn * 4.0) / 4.0e6; };
    constexpr int kCands = 10;
    const uint64_t pairs288 = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 288);
    const uint64_t pairs320 = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 320);
    const uint64_t pairs192 = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 192);
    const uint64_t pairs224 = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 224);
    // Waves of pair tiles, the last one counted by how full it is: behind at least one full wave a nearly empty
    // wave costs about three quarters of a full one (its tiles have L2 and the memory system to themselves).
    // Measured in the driver's burst protocol at 2304 ... 3840: pairs on 256 x 224 beat 256 x 256 at 2816^3
    // (1260 against 1163 TFLOP/s) and 3328^3 (1300 against 1245), 256 x 192 wins 2304^3 and 2560^3, and 256 x 160
    // (built, a plan option) wins nowhere.
    auto pair_waves = [&](uint64_t tiles) {
        if (tiles <= pair_slots) return 1.0;
        const uint64_t rest = tiles % pair_slots;
        if (rest == 0) return static_cast<double>(tiles / pair_slots);
        return static_cast<double>(tiles / pair_slots) + 0.75 + 0.25 * static_cast<double>(rest) / static_cast<double>(pair_slots);
    };
    Candidate cands[kCands] = {
        {B200_VARIANT_CTA1, 256, waves(tiles256, sms) * kb * 0.35 + 2.0},
        {B200_VARIANT_CTA1, 128, waves(tiles128, sms) * kb * 0.33 + 1.5},
        {B200_VARIANT_CTA1, 64, waves(tiles64, sms) * kb * 0.30 + 1.2},
        // pairs: less L2 traffic per k-block than single CTAs, a costlier launch (measured: single
        // CTAs ahead at 1792 and 2048, pairs from 2304 up)
        {B200_VARIANT_CTA2, 256, pair_waves(pairs256) * kb * 0.335 + 2.5},
        {B200_VARIANT_STREAMK, 256, static_cast<double>(tiles256) * kb / sms * 0.35 + 4.0 + partial_us(256)},
        {B200_VARIANT_STREAMK, 128, static_cast<double>(tiles128) * kb / sms * 0.33 + 4.0 + partial_us(128)},
        // pairs on 256 x 192 tiles (two k-blocks per stage): three quarters of the time of a 256-wide tile,
        // so two ragged waves of them beat two ragged waves of those (measured: 2304^3 950 against 810
        // TFLOP/s, 2560^3 1160 against 990; no gain where 256-wide tiles fit one wave, as at 1792^3)
        {B200_VARIANT_CTA2, 192, pairs256 > pair_slots ? pair_waves(pairs192) * kb * 0.27 + 2.5 : 1e30},
        {B200_VARIANT_CTA2, 224, pairs256 > pair_slots ? pair_waves(pairs224) * kb * 0.308 + 2.5 : 1e30},
        // pairs on tiles wider than one MMA (two MMAs of 144 or 160 columns side by side, each with the fixed part
        // of an MMA's time: about 0.49 us per k-block against 0.335 for 256 columns): only where they turn
        // two ragged waves into one. Measured at 2304 x 2304 x K (72 tiles of 256 x 288 on 74 pairs), burst
        // protocol, against the best of the narrower pair tiles (two waves of 256 x 160): K = 1536 18.6 / 19.3 us,
        // 2304 23.9 / 24.6, 4096 36.1 / 37.8, 8192 65.3 / 73.3; 2304 x 2560 x 2304 on 256 x 320: 24.5 / 25.0;
        // 4608 x 1152 x 2048: 22.0 / 23.3. With several tiles per pair they lose (one accumulator: no overlap of
        // epilogue and MMAs). The factors below are set under the narrower tiles' so that one wave wins.
        {B200_VARIANT_CTA2, 288, (pairs256 > pair_slots && pairs288 <= pair_slots && N % 8 == 0) ? kb * 0.44 + 2.5 : 1e30},
        {B200_VARIANT_CTA2, 320, (pairs256 > pair_slots && pairs320 <= pair_slots && N % 8 == 0) ? kb * 0.455 + 2.5 : 1e30},
    };
    if (M % 256 != 0) cands[8].us *= 1.0 + 128.0 / static_cast<double>(M);
    if (M % 256 != 0) cands[9].us *= 1.0 + 128.0 / static_cast<double>(M);
    if (M % 256 != 0) cands[7].us *= 1.0 + 128.0 / static_cast<double>(M);
    if (M % 256 != 0) cands[6].us *= 1.0 + 128.0 / static_cast<double>(M);
    if (M % 256 != 0) cands[3].us *= 1.0 + 128.0 / static_cast<double>(M);  // the pair's second CTA idles on the last rows
    if (k_blocks < 16) cands[4].us = cands[5].us = 1e30;                    // too little k to split
    int best = 0;
    for (int i = 1; i < kCands; ++i) {
        if (cands[i].us < cands[best].us * 0.98) best = i;  // earlier entries win ties: fewer moving parts
    }
    pl->variant = cands[best].variant;
    pl->bn = cands[best].bn;
}

// ------------------------------------------------------------------------------------------
// launch
// ------------------------------------------------------------------------------------------
// Programmatic dependent launch is on unless B200_HGEMM_NO_PDL is set in the environment (for
// A/B measurements; without the launch attribute the kernels' griddepcontrol instructions do nothing).
static bool pdl_enabled() {
    static const bool on = (getenv("B200_HGEMM_NO_PDL") == nullptr);
    return on;
}

template <int BN, int STAGES, int CG, int MODE, int KPS = 1, bool EPI = false, int FLAVOR = 0>
static int launch_kernel(DeviceState &st, int attr_slot, const GemmParams &p, uint32_t grid, cudaStream_t stream) {
    using T = KernelTraits<BN, STAGES, CG, KPS>;
    auto kern = hgemm_tcgen05_kernel<BN, STAGES, CG, MODE, KPS, EPI, FLAVOR>;
    if (!st.attr_set[attr_slot]) {
        std::lock_guard<std::mutex> lock(st.mu);
        if (!st.attr_set[attr_slot]) {
            if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes), "cudaFuncSetAttribute")) {
                return B200_HGEMM_ERR_CUDA;
            }
            st.attr_set[attr_slot] = true;
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = T::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n_attrs = 0;
    // programmatic dependent launch: the kernel's prologue (barrier set-up, tensor-memory
    // allocation) may overlap the tail of the previous kernel in the stream; every global
    // access inside the kernel comes after griddepcontrol.wait
    if (pdl_enabled()) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    if (CG == 2) {
        attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[n_attrs].val.clusterDim.x = 2;
        attrs[n_attrs].val.clusterDim.y = 1;
        attrs[n_attrs].val.clusterDim.z = 1;
        ++n_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;
    if (CG == 2) {
        // A persistent grid must be fully resident: ask how many pairs fit (GPC boundaries can
        // leave fewer than SMs / 2) and never launch more.
        if (st.max_clusters[attr_slot] == 0) {
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
                cudaGetLastError();
                return B200_HGEMM_ERR_CUDA;
            }
            std::lock_guard<std::mutex> lock(st.mu);
            st.max_clusters[attr_slot] = n;
        }
        // (k-ranges are handed out by CTA index: that grid is launched as it is; none of its CTAs waits for another)
        if (MODE == kModeTiles && grid / 2 > static_cast<uint32_t>(st.max_clusters[attr_slot])) {
            grid = 2u * static_cast<uint32_t>(st.max_clusters[attr_slot]);
            cfg.gridDim = dim3(grid, 1, 1);
        }
    }
    if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, p), "cudaLaunchKernelEx")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

// The pair kernel with 256 x 256 outputs per CTA (gemm_kernel_big.cuh), 512 x 256 per pair.
__global__ void __launch_bounds__(kBigThreads, 1) hgemm_tcgen05_big_kernel(const __grid_constant__ GemmParams p) {
    hgemm_big_body<2, NoMulticastLoad>(p);
}

__global__ void __launch_bounds__(kBigThreads, 1) hgemm_tcgen05_big_epi_kernel(const __grid_constant__ GemmParams p) {
    hgemm_big_body<2, NoMulticastLoad, true>(p);
}

// Launch configuration of the kernel with 256 x 256 outputs per CTA (shared-memory opt-in done once).
static int big_kernel_config(DeviceState &st, bool fused, cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attrs) {
    auto kern = fused ? hgemm_tcgen05_big_epi_kernel : hgemm_tcgen05_big_kernel;
    const int slot = fused ? 15 : 8;
    if (!st.attr_set[slot]) {
        std::lock_guard<std::mutex> lock(st.mu);
        if (!st.attr_set[slot]) {
            if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBigSmemBytes), "cudaFuncSetAttribute")) {
                return B200_HGEMM_ERR_CUDA;
            }
            st.attr_set[slot] = true;
        }
    }
    memset(cfg, 0, sizeof(*cfg));
    cfg->blockDim = dim3(kBigThreads, 1, 1);
    cfg->dynamicSmemBytes = kBigSmemBytes;
    int n_attrs = 0;
    if (pdl_enabled()) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 2;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
    cfg->attrs = attrs;
    cfg->numAttrs = n_attrs;
    return B200_HGEMM_OK;
}

// CTA pairs of that kernel the device keeps resident at once (74 on a B200), asked for once.
static int big_kernel_pair_slots(DeviceState &st, bool fused, uint32_t *slots) {
    const int slot = fused ? 15 : 8;
    if (st.max_clusters[slot] == 0) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attrs[2];
        const int rc = big_kernel_config(st, fused, &cfg, attrs);
        if (rc != B200_HGEMM_OK) return rc;
        cfg.gridDim = dim3(2u * static_cast<uint32_t>(st.sm_count > 1 ? st.sm_count / 2 : 1), 1, 1);
        int n = 0;
        auto kern = fused ? hgemm_tcgen05_big_epi_kernel : hgemm_tcgen05_big_kernel;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            return B200_HGEMM_ERR_CUDA;
        }
        std::lock_guard<std::mutex> lock(st.mu);
        st.max_clusters[slot] = n;
    }
    *slots = static_cast<uint32_t>(st.max_clusters[slot]);
    return B200_HGEMM_OK;
}

static int launch_big_kernel(DeviceState &st, const GemmParams &p, uint32_t grid, cudaStream_t stream, bool fused = false) {
    auto kern = fused ? hgemm_tcgen05_big_epi_kernel : hgemm_tcgen05_big_kernel;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attrs[2];
    int rc = big_kernel_config(st, fused, &cfg, attrs);
    if (rc != B200_HGEMM_OK) return rc;
    uint32_t slots = 0;
    if ((rc = big_kernel_pair_slots(st, fused, &slots)) != B200_HGEMM_OK) return rc;
    if (grid / 2 > slots) grid = 2u * slots;  // a persistent grid must be fully resident
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.stream = stream;
    if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, p), "cudaLaunchKernelEx")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

static size_t plan_workspace_bytes(const DeviceState &st, size_t M, size_t N, size_t K, const b200_hgemm_plan &pl) {
    if (!plan_cuts_k(pl)) return 0;
    const uint32_t cg = static_cast<uint32_t>(plan_cg(pl));
    const uint32_t tiles = ceil_div_u32(M, 128u * cg) * ceil_div_u32(N, pl.bn);
    const uint32_t parts = streamk_parts(pl, st, tiles, plan_k_units(pl, K));
    return kCounterBytes + static_cast<size_t>(parts) * 2u * (128u * cg * pl.bn * sizeof(float));
}

constexpr size_t kMaxStreamWorkspaces = 64;

// The workspace a stream-k launch on `stream` may use: the caller's when one was handed over,
// else this stream's own, allocated or grown here (cudaMalloc / cudaFree: never during capture).
// At most kMaxStreamWorkspaces streams hold one at a time; when a further stream asks, the
// workspace used longest ago is given up (its cudaFree waits for the work that still uses it).
static int workspace_for(DeviceState &st, cudaStream_t stream, size_t need, uint8_t **out) {
    std::lock_guard<std::mutex> lock(st.mu);
    if (st.ws) {
        if (st.ws_bytes < need) return B200_HGEMM_ERR_WORKSPACE;  // caller-provided and too small
        *out = static_cast<uint8_t *>(st.ws);
        return B200_HGEMM_OK;
    }
    if (need > kMaxOwnedWorkspace) return B200_HGEMM_ERR_WORKSPACE;
    DeviceState::StreamWorkspace *slot = nullptr;
    for (auto &w : st.owned_ws) {
        if (w.stream == stream) slot = &w;
    }
    if (!slot) {
        if (st.owned_ws.size() >= kMaxStreamWorkspaces) {
            size_t oldest = 0;
            for (size_t i = 1; i < st.owned_ws.size(); ++i) {
                if (st.owned_ws[i].last_use < st.owned_ws[oldest].last_use) oldest = i;
            }
            slot = &st.owned_ws[oldest];
            // the previous owner's kernels may still be using the buffer (and its stream handle may be
            // gone by now): wait for the device once; this path is rare
            if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return B200_HGEMM_ERR_CUDA;
            slot->stream = stream;  // the buffer itself is kept when it is large enough
        } else {
            st.owned_ws.push_back({stream, nullptr, 0, 0});
            slot = &st.owned_ws.back();
        }
    }
    slot->last_use = ++st.ws_clock;
    if (slot->bytes < need) {
        if (slot->ptr) {
            if (!cuda_ok(cudaFree(slot->ptr), "cudaFree")) return B200_HGEMM_ERR_CUDA;  // synchronises the device
            slot->ptr = nullptr;
            slot->bytes = 0;
        }
        const size_t bytes = need < (size_t(32) << 20) ? (size_t(32) << 20) : need;
        if (!cuda_ok(cudaMalloc(&slot->ptr, bytes), "cudaMalloc")) {
            cudaGetLastError();
            return B200_HGEMM_ERR_WORKSPACE;
        }
        slot->bytes = bytes;
    }
    *out = static_cast<uint8_t *>(slot->ptr);
    return B200_HGEMM_OK;
}

// One CTA waits on an mbarrier that nothing ever arrives on, with a short limit: the expiry
// path of the kernels' bounded waits (abort flag, error word), exercised without hanging anything.
__global__ void wait_expiry_probe_kernel(uint32_t *error_word, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    // parity 0 of a fresh barrier completes only after an arrival, and none is ever made
    const bool done = mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && !done && abort_flag != 0) atomicExch(error_word, static_cast<uint32_t>(kDevWaitTimeout));
}

// Any-shape CUDA-core kernel: one thread per C element, FP32 accumulate.
__global__ void hgemm_simt_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ c,
                                  size_t m, size_t n, size_t k) {
    const size_t col = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t row = blockIdx.y * static_cast<size_t>(blockDim.y) + threadIdx.y;
    if (row >= m || col >= n) return;
    const __half *ar = a + row * k;
    const __half *br = b + col * k;
    float acc = 0.f;
    for (size_t i = 0; i < k; ++i) acc = fmaf(__half2float(ar[i]), __half2float(br[i]), acc);
    c[row * n + col] = __float2half_rn(acc);
}

static int run_simt(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid(static_cast<unsigned>((N + block.x - 1) / block.x), static_cast<unsigned>((M + block.y - 1) / block.y));
    if (grid.y > 65535u) return B200_HGEMM_ERR_UNSUPPORTED;
    hgemm_simt_kernel<<<grid, block, 0, stream>>>(static_cast<const __half *>(A), static_cast<const __half *>(B),
                                                  static_cast<__half *>(C), M, N, K);
    if (!cuda_ok(cudaGetLastError(), "cudaGetLastError")) return B200_HGEMM_ERR_CUDA;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

// The fused epilogue a caller asked for, checked and in the kernels' terms.
static int epilogue_args(const b200_hgemm_epilogue &epi, EpilogueArgs *out) {
    if (epi.c_type != B200_C_F16 && epi.c_type != B200_C_BF16 && epi.c_type != B200_C_F32) return B200_HGEMM_ERR_INVALID_ARG;
    if (epi.beta != 0.f && !epi.c_in) return B200_HGEMM_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(epi.bias) | reinterpret_cast<uintptr_t>(epi.c_in)) & 15u) return B200_HGEMM_ERR_MISALIGNED;
    out->alpha = epi.alpha;
    out->beta = epi.beta;
    out->bias = static_cast<const __half *>(epi.bias);
    out->c_in = epi.c_in;
    out->c_type = static_cast<uint32_t>(epi.c_type);
    return B200_HGEMM_OK;
}

// ---- short A (M <= 128): B streams through the MMA's row operand (gemm_kernel_skinny.cuh) ----
// Width of a column tile, in columns of C. Every CTA streams the tile's rows of B over its whole
// k-range, so the kernel takes as long as its busiest SM: waves x width is what to minimise. 128
// columns give N = 14336 112 tiles for 148 SMs; 104 give it 138. Below 64 columns the MMAs (always
// 128 rows tall) would cost more issue time than the narrower tile saves; when k is cut into slices
// the tiles stay 128 wide.
static uint32_t skinny_tile_w(const b200_hgemm_plan &pl, const DeviceState &st, size_t N) {
    if (pl.group_m > 0) return static_cast<uint32_t>(pl.group_m);
    const uint32_t sms = st.sm_count > 0 ? static_cast<uint32_t>(st.sm_count) : 148u;
    if (pl.parts > 1 || ceil_div_u32(N, 128) * 5 < sms * 3) return 128u;  // few tiles: k is cut instead
    uint32_t best_w = 128u;
    uint64_t best_cost = static_cast<uint64_t>(ceil_div_u32(ceil_div_u32(N, 128), sms)) * 128u;
    for (uint32_t w = 120; w >= 64; w -= 8) {
        const uint64_t cost = static_cast<uint64_t>(ceil_div_u32(ceil_div_u32(N, w), sms)) * w;
        if (cost < best_cost) {
            best_cost = cost;
            best_w = w;
        }
    }
    return best_w;
}

// B200_HGEMM_SKINNY_WORKSPACE_SUM (any value): the library never chooses the sum inside clusters by itself (for
// measurements; a plan that asks for it with grid = 1 still gets it).
static bool skinny_workspace_sum_forced() {
    static const bool on = (getenv("B200_HGEMM_SKINNY_WORKSPACE_SUM") != nullptr);
    return on;
}

static uint32_t skinny_slices(const b200_hgemm_plan &pl, const DeviceState &st, size_t N, size_t K) {
    const uint32_t tiles = ceil_div_u32(N, skinny_tile_w(pl, st, N));
    const uint32_t k_blocks = ceil_div_u32(K, 64);
    const uint32_t sms = st.sm_count > 0 ? static_cast<uint32_t>(st.sm_count) : 148u;
    uint32_t slices = pl.parts > 0 ? static_cast<uint32_t>(pl.parts) : 0u;
    if (slices == 0) {
        // cut k only when the column tiles leave most of the GPU idle, and keep 8 k-blocks per slice
        slices = (tiles * 5 >= sms * 3) ? 1u : sms / tiles;
        const uint32_t most = k_blocks / 8 > 0 ? k_blocks / 8 : 1u;
        if (slices > most) slices = most;
        // Four k-ranges summed inside a cluster beat more of them summed through the workspace as long as they
        // still occupy two fifths of the SMs (measured at N = 2048 and 3072, K = 8192: 16 and 24 tiles, 11.0
        // against 13.0 us and 12.8 against 13.6); single CTAs only -- pairs would be left with two k-ranges.
        if (slices > 4 && pl.variant == B200_VARIANT_SKINNY && pl.grid != 2 && !skinny_workspace_sum_forced() &&
            tiles * 4u * 5u >= sms * 2u) {
            slices = 4;
        }
    }
    if (slices > k_blocks) slices = k_blocks;
    if (slices < 1) slices = 1;
    const uint32_t per = ceil_div_u32(k_blocks, slices);
    return ceil_div_u32(k_blocks, per);  // no empty slice
}

// How the k-ranges of a column tile are summed. plan.grid says: 1 = inside a thread-block cluster (the k-ranges of a
// tile, times two CTAs for pairs, are one cluster of at most 8 CTAs: no workspace, no second kernel), 2 = through the
// FP32 workspace and skinny_reduce_kernel, 0 = the library's choice: the cluster when it is at most four CTAs.
// Returns 1 / 0, or -1 when the plan asks for a cluster that would be larger than 8 CTAs.
static int skinny_sums_on_chip(const b200_hgemm_plan &pl, uint32_t slices) {
    const uint32_t cg = pl.variant == B200_VARIANT_SKINNY_PAIR ? 2u : 1u;
    if (slices < 2) return 0;
    const bool fits = slices * cg <= 8u;
    if (pl.grid == 1) return fits ? 1 : -1;
    if (pl.grid == 2) return 0;
    // left to the library: clusters of up to four CTAs (148 SMs hold far fewer clusters of eight than 148 / 8:
    // measured, 16 of them ran as two waves)
    return (slices * cg <= 4u && !skinny_workspace_sum_forced()) ? 1 : 0;
}

static size_t skinny_workspace_bytes(const b200_hgemm_plan &pl, const DeviceState &st, size_t N, size_t K) {
    const uint32_t slices = skinny_slices(pl, st, N, K);
    if (slices <= 1 || skinny_sums_on_chip(pl, slices) == 1) return 0;
    const size_t n_pad = (N + 31) / 32 * 32;
    return static_cast<size_t>(slices) * pl.bn * n_pad * sizeof(float);
}

// k-blocks of B a short-A CTA asks into L2 before it waits for the previous kernel (B200_HGEMM_SKINNY_PREFETCH
// overrides it for measurements; 0 switches the prefetch off). Without programmatic dependent launch there
// is no previous kernel to overlap with. Measured inside CUDA graphs, B from HBM: tiles of 16 and 32 rows of A
// are fastest with 6 ... 8 k-blocks (M = 16: -4 % against none; 32 and more lose), tiles of 64 and 128 rows
// with 4 (against 8: 22.5 / 22.8 us at M = 64 and 24.7 / 25.2 at M = 128 for N = 14336, 23.0 / 23.8 and
// 26.0 / 26.6 for N = 4096, K = 14336).
static uint32_t skinny_prefetch_kb(int rows_per_tile) {
    static const int forced = []() -> int {
        const char *v = getenv("B200_HGEMM_SKINNY_PREFETCH");
        return v ? atoi(v) : -1;
    }();
    if (!pdl_enabled()) return 0u;
    if (forced >= 0) return static_cast<uint32_t>(forced);
    return rows_per_tile >= 64 ? 4u : 8u;
}

static std::atomic<int> g_debug_cluster_capacity{0};  // b200_debug_cluster_capacity(): > 0 overrides what the device reports

template <int MT, int STAGES, int KPS, int CG, bool EPI, bool CK>
static int launch_skinny_kernel(DeviceState &st, int attr_slot, const SkinnyParams &p, cudaStream_t stream, bool whole_wave_only);

// The kernel for this tile height and CTA grouping, plain or with the fused epilogue (attribute slots 32 up), its
// k-ranges summed through the workspace or (on_chip) inside clusters (attribute slots 64 up: eight plain, eight fused).
template <int MT, int STAGES, int KPS, int CG = 1>
// whole_wave_only (with on_chip): B200_HGEMM_ERR_UNSUPPORTED, and nothing launched, unless the device can hold all the
// clusters at once (the caller then takes the workspace form).
static int launch_skinny(DeviceState &st, int attr_slot, const SkinnyParams &p, cudaStream_t stream, bool fused, bool on_chip,
                         bool whole_wave_only) {
    if (on_chip) {
        const int ck_slot = 64 + (CG == 2 ? 4 + attr_slot - 25 : attr_slot - 11);
        if (fused) return launch_skinny_kernel<MT, STAGES, KPS, CG, true, true>(st, ck_slot + 8, p, stream, whole_wave_only);
        return launch_skinny_kernel<MT, STAGES, KPS, CG, false, true>(st, ck_slot, p, stream, whole_wave_only);
    }
    if (fused) return launch_skinny_kernel<MT, STAGES, KPS, CG, true, false>(st, attr_slot + 21, p, stream, false);
    return launch_skinny_kernel<MT, STAGES, KPS, CG, false, false>(st, attr_slot, p, stream, false);
}

template <int MT, int STAGES, int KPS, int CG, bool EPI, bool CK>
static int launch_skinny_kernel(DeviceState &st, int attr_slot, const SkinnyParams &p, cudaStream_t stream, bool whole_wave_only) {
    using T = SkinnyTraits<MT, STAGES, KPS, CG>;
    auto kern = hgemm_skinny_kernel<MT, STAGES, KPS, CG, EPI, CK>;
    if (!st.attr_set[attr_slot]) {
        std::lock_guard<std::mutex> lock(st.mu);
        if (!st.attr_set[attr_slot]) {
            if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes), "cudaFuncSetAttribute")) {
                return B200_HGEMM_ERR_CUDA;
            }
            st.attr_set[attr_slot] = true;
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(p.n_tiles * p.slices, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = T::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n_attrs = 0;
    if (pdl_enabled()) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    if (CG == 2 || CK) {  // the grid is a whole number of pairs (n_tiles is even), or of clusters of one tile's k-ranges
        attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[n_attrs].val.clusterDim.x = CK ? p.slices * CG : 2;
        attrs[n_attrs].val.clusterDim.y = 1;
        attrs[n_attrs].val.clusterDim.z = 1;
        ++n_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;
    if (CK && whole_wave_only) {
        // clusters that wait for a second wave would double the kernel's time: ask once per cluster size
        const uint32_t size = p.slices * CG;
        const int idx = attr_slot - 64;
        if (idx < 0 || idx >= 16 || size > 8) return B200_HGEMM_ERR_UNSUPPORTED;
        int known;
        {
            std::lock_guard<std::mutex> lock(st.mu);
            if (st.ck_clusters[idx][size] == 0) {
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
                    cudaGetLastError();
                    n = -1;
                }
                st.ck_clusters[idx][size] = n;
            }
            known = st.ck_clusters[idx][size];
        }
        const int pretend = g_debug_cluster_capacity.load(std::memory_order_relaxed);
        if (pretend > 0) known = pretend;
        if (known < 0 || static_cast<uint64_t>(known) * size < cfg.gridDim.x) return B200_HGEMM_ERR_UNSUPPORTED;
    }
    if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, p), "cudaLaunchKernelEx")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

static int run_skinny(DeviceState &st, const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                      const b200_hgemm_plan &pl, cudaStream_t stream, void *ws_override, size_t ws_override_bytes,
                      uint32_t *error_word, const b200_hgemm_epilogue *epi) {
    if (M > static_cast<size_t>(pl.bn)) return B200_HGEMM_ERR_UNSUPPORTED;
    SkinnyParams p;
    memset(&p, 0, sizeof(p));
    const bool fused = epi != nullptr;
    if (fused) {
        const int erc = epilogue_args(*epi, &p.epi);
        if (erc != B200_HGEMM_OK) return erc;
    }
    p.c = static_cast<__half *>(C);
    p.error_word = error_word;
    p.m = static_cast<uint32_t>(M);
    p.n = static_cast<uint32_t>(N);
    p.k = static_cast<uint32_t>(K);
    p.k_blocks = ceil_div_u32(K, 64);
    const bool pairs = pl.variant == B200_VARIANT_SKINNY_PAIR;
    p.tile_w = skinny_tile_w(pl, st, N);
    p.n_tiles = ceil_div_u32(N, p.tile_w);
    if (pairs) p.n_tiles += p.n_tiles & 1u;  // a pair's second tile may lie past N: it reads zeros and stores nothing
    p.slices = skinny_slices(pl, st, N, K);
    p.kb_per_slice = ceil_div_u32(p.k_blocks, p.slices);
    p.n_pad = static_cast<uint32_t>((N + 31) / 32 * 32);
    p.prefetch_kb = skinny_prefetch_kb(pl.bn);
#ifdef B200_TIMELINE
    p.timeline = g_timeline;
#endif
    if (static_cast<uint64_t>(p.n_tiles) * p.slices > 0x7fffffffull) return B200_HGEMM_ERR_UNSUPPORTED;
    int rc = get_tensor_map(st, B, N, K, p.tile_w, 64, &p.tm_w);
    if (rc != B200_HGEMM_OK) return rc;
    rc = get_tensor_map(st, A, M, K, static_cast<uint32_t>(pl.bn) / (pairs ? 2u : 1u), 64, &p.tm_x);
    if (rc != B200_HGEMM_OK) return rc;
    // whole results leave through one TMA store per tile (a plain row-major box of tile_w x bn) when C can
    // have a tensor map: rows of N halves must be a multiple of 16 bytes
    p.tma_store = (pl.tma_store && N % 8 == 0 && p.slices == 1 && p.epi.c_type != kOutF32) ? 1u : 0u;  // FP32 leaves by element
    const int sum_on_chip = skinny_sums_on_chip(pl, p.slices);
    if (sum_on_chip < 0) return B200_HGEMM_ERR_UNSUPPORTED;
    const bool on_chip = sum_on_chip == 1;
    if (p.tma_store) {
        rc = get_tensor_map(st, C, M, N, static_cast<uint32_t>(pl.bn), p.tile_w, &p.tm_c, false);
        if (rc != B200_HGEMM_OK) return rc;
    }
    // the kernel for this tile height and CTA grouping, summing inside clusters or not
    auto launch = [&](bool in_clusters, bool whole_wave_only) -> int {
        if (pairs) {
            if (pl.bn == 16) return launch_skinny<16, 6, 2, 2>(st, 25, p, stream, fused, in_clusters, whole_wave_only);
            if (pl.bn == 32) return launch_skinny<32, 6, 2, 2>(st, 26, p, stream, fused, in_clusters, whole_wave_only);
            if (pl.bn == 64) return launch_skinny<64, 5, 2, 2>(st, 27, p, stream, fused, in_clusters, whole_wave_only);
            return launch_skinny<128, 4, 2, 2>(st, 28, p, stream, fused, in_clusters, whole_wave_only);
        }
        if (pl.bn == 16) return launch_skinny<16, 6, 2>(st, 11, p, stream, fused, in_clusters, whole_wave_only);
        if (pl.bn == 32) return launch_skinny<32, 5, 2>(st, 12, p, stream, fused, in_clusters, whole_wave_only);
        if (pl.bn == 64) return launch_skinny<64, 4, 2>(st, 13, p, stream, fused, in_clusters, whole_wave_only);
        return launch_skinny<128, 3, 2>(st, 14, p, stream, fused, in_clusters, whole_wave_only);
    };
    if (on_chip) {
        // The library's own choice must fit the device in one wave of clusters; where it does not (a device with
        // fewer SMs per GPC than a B200's), the same k-ranges go through the workspace instead. A plan that asks
        // for the clusters gets them, or the launch's error.
        rc = launch(true, pl.grid != 1);
        if (rc != B200_HGEMM_ERR_UNSUPPORTED || pl.grid == 1) return rc;
    }
    if (p.slices > 1) {
        const size_t need = static_cast<size_t>(p.slices) * pl.bn * p.n_pad * sizeof(float);
        uint8_t *ws = nullptr;
        if (ws_override) {
            if (ws_override_bytes < need) return B200_HGEMM_ERR_WORKSPACE;
            ws = static_cast<uint8_t *>(ws_override);
        } else {
            rc = workspace_for(st, stream, need, &ws);
            if (rc != B200_HGEMM_OK) return rc;
        }
        p.partials = reinterpret_cast<float *>(ws);
    }
    rc = launch(false, false);
    if (rc != B200_HGEMM_OK || p.slices == 1) return rc;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(ceil_div_u32(N, kSkinnyReduceThreads), static_cast<unsigned>(M), 1);
    cfg.blockDim = dim3(kSkinnyReduceThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (!cuda_ok(cudaLaunchKernelEx(&cfg, skinny_reduce_kernel, static_cast<const float *>(p.partials), p.c, p.m, p.n, p.n_pad,
                                    static_cast<uint32_t>(pl.bn), p.slices, fused ? 1u : 0u, p.epi),
                 "cudaLaunchKernelEx")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

static int check_args(const void *A, const void *B, const void *C, size_t M, size_t N, size_t K) {
    if (!A || !B || !C || M == 0 || N == 0 || K == 0) return B200_HGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return B200_HGEMM_ERR_UNSUPPORTED;
    return B200_HGEMM_OK;
}

// 512 x 256 tiles on CTA pairs, and what is left of them after the full waves.
//
// With T tiles on S resident pairs the last wave holds T % S tiles and costs as much as a full one. When
// those left-over tiles, cut into two 256 x 256 halves each, fit one wave of the 128 x 256-per-CTA pair
// kernel (2 * (T % S) <= S), that kernel takes them in a second launch right behind the first: half a
// wave's time instead of a whole one. A row slab of 2048 x 16384 (one of eight GPUs' share of 16384^3)
// has 256 tiles on 74 pairs: 3 full waves and 34 tiles, i.e. 3.5 waves' time instead of 4. The second
// launch reads the same tensor maps (its boxes are the same) and finds its tiles through the larger
// tiles' raster (GemmParams::tail_*), so both launches together write every element of C exactly once.
static int launch_big_with_tail(DeviceState &st, const GemmParams &p, uint32_t grid, cudaStream_t stream, bool fused,
                                bool fixed_grid) {
    uint32_t slots = 0;
    int rc = big_kernel_pair_slots(st, fused, &slots);
    if (rc != B200_HGEMM_OK) return rc;
    const uint32_t full = (p.tiles / slots) * slots, rest = p.tiles - full;
    static const bool tail_off = (getenv("B200_HGEMM_NO_TAIL_SPLIT") != nullptr);
    if (tail_off || fixed_grid || full == 0 || rest == 0 || 2u * rest > slots) return launch_big_kernel(st, p, grid, stream, fused);
    GemmParams head = p;
    head.tiles = full;
    if ((rc = launch_big_kernel(st, head, grid, stream, fused)) != B200_HGEMM_OK) return rc;
    GemmParams tail = p;
    tail.tail_first = full;
    tail.tail_sm = 2;
    tail.tail_sn = 1;
    tail.tail_m_blocks = p.m_blocks;
    tail.tail_n_blocks = p.n_blocks;
    tail.tail_group_m = p.group_m;
    tail.m_blocks = ceil_div_u32(p.m, 256);
    tail.tiles = 2u * rest;
    const uint32_t tail_grid = 2u * tail.tiles;
    if (fused) return launch_kernel<256, 6, 2, kModeTiles, 1, true>(st, 19, tail, tail_grid, stream);
    return launch_kernel<256, 6, 2, kModeTiles>(st, 3, tail, tail_grid, stream);
}

static int run_plan(DeviceState &st, const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                    const b200_hgemm_plan &pl, cudaStream_t stream, void *ws_override, size_t ws_override_bytes,
                    uint32_t *error_word_override = nullptr, const b200_hgemm_epilogue *epi = nullptr) {
    int rc = validate_plan(pl, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    if (pl.variant == B200_VARIANT_SIMT) return run_simt(A, B, C, M, N, K, stream);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) {
        return B200_HGEMM_ERR_MISALIGNED;
    }
    if (pl.variant == B200_VARIANT_SKINNY || pl.variant == B200_VARIANT_SKINNY_PAIR) {
        return run_skinny(st, A, B, C, M, N, K, pl, stream, ws_override, ws_override_bytes,
                          error_word_override ? error_word_override : st.error_word, epi);
    }
    if (pl.variant == B200_VARIANT_CTA2_MCAST) {
        // the multicast loads may only ever read this GPU's own memory: every operand must be an
        // allocation of the device the kernel is launched on (not a peer's, not host memory)
        int cur_dev = -1;
        if (!cuda_ok(cudaGetDevice(&cur_dev), "cudaGetDevice")) return B200_HGEMM_ERR_CUDA;
        for (const void *ptr : {A, B, static_cast<const void *>(C)}) {
            cudaPointerAttributes pa;
            if (!cuda_ok(cudaPointerGetAttributes(&pa, ptr), "cudaPointerGetAttributes")) return B200_HGEMM_ERR_CUDA;
            if (pa.type != cudaMemoryTypeDevice || pa.device != cur_dev) return B200_HGEMM_ERR_UNSUPPORTED;
        }
        GemmParams mp;
        memset(&mp, 0, sizeof(mp));
        mp.c = static_cast<__half *>(C);
        mp.error_word = st.error_word;
        mp.m = static_cast<uint32_t>(M);
        mp.n = static_cast<uint32_t>(N);
        mp.k = static_cast<uint32_t>(K);
        const bool big = pl.bn == 512;           // 256 rows per CTA instead of 128
        mp.m_blocks = ceil_div_u32(M, big ? 512 : 256);  // super-tiles of 256 x 512 or 512 x 512: two pairs side by side
        mp.n_blocks = ceil_div_u32(N, 512);
        mp.k_blocks = ceil_div_u32(K, 64);
        if (static_cast<uint64_t>(mp.m_blocks) * mp.n_blocks > 0x7fffffffull) return B200_HGEMM_ERR_UNSUPPORTED;
        mp.tiles = mp.m_blocks * mp.n_blocks;
        mp.group_m = pl.group_m > 0 ? static_cast<uint32_t>(pl.group_m) : (big ? 6u : 8u);
        if (mp.group_m > mp.m_blocks) mp.group_m = mp.m_blocks;
        mp.tma_store = 1;
        mp.c_vec_ok = 1;
        if ((rc = get_tensor_map(st, A, M, K, big ? 128 : 64, 64, &mp.tm_a)) != B200_HGEMM_OK) return rc;
        if ((rc = get_tensor_map(st, B, N, K, 128, 64, &mp.tm_b)) != B200_HGEMM_OK) return rc;
        if ((rc = get_tensor_map(st, C, M, N, 32, 64, &mp.tm_c)) != B200_HGEMM_OK) return rc;
        rc = mc_launch_fn(pl.bn)(&mp, stream, pdl_enabled() ? 1 : 0);
        if (rc != 0) return B200_HGEMM_ERR_CUDA;
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return B200_HGEMM_OK;
    }
    const int cg = plan_cg(pl);
    const bool big = pl.variant == B200_VARIANT_CTA2 && pl.bn == 512;  // 512 x 256 per pair
    const int bn = big ? 256 : pl.bn;

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.c = static_cast<__half *>(C);
    p.error_word = error_word_override ? error_word_override : st.error_word;
    p.m = static_cast<uint32_t>(M);
    p.n = static_cast<uint32_t>(N);
    p.k = static_cast<uint32_t>(K);
    p.m_blocks = ceil_div_u32(M, big ? 512u : 128u * cg);
    p.n_blocks = ceil_div_u32(N, bn);
    p.k_blocks = plan_k_units(pl, K);  // pipeline stages per tile: k-blocks, or pairs of them
    const uint64_t tiles64 = static_cast<uint64_t>(p.m_blocks) * p.n_blocks;
    if (tiles64 > 0x7fffffffull) return B200_HGEMM_ERR_UNSUPPORTED;
    p.tiles = static_cast<uint32_t>(tiles64);
    p.group_m = pl.group_m > 0 ? static_cast<uint32_t>(pl.group_m) : (big ? 6u : cg == 2 ? 8u : 16u);
    if (p.group_m > p.m_blocks) p.group_m = p.m_blocks;
    p.raster = make_raster(p.m_blocks, p.n_blocks, p.group_m);
    p.tma_store = pl.tma_store ? 1u : 0u;
    p.c_vec_ok = (N % 8 == 0) ? 1u : 0u;
    EpilogueArgs ea;
    memset(&ea, 0, sizeof(ea));
    if (epi) {
        // c_vec_ok also covers the 16-byte loads of bias and c_in
        if ((rc = epilogue_args(*epi, &ea)) != B200_HGEMM_OK) return rc;
        if (big && ea.c_type == kOutF32) return B200_HGEMM_ERR_UNSUPPORTED;  // that kernel packs 16-bit outputs only
        p.alpha = ea.alpha;
        p.beta = ea.beta;
        p.bias = ea.bias;
        p.c_in = ea.c_in;
        p.c_type = ea.c_type;
        if (ea.c_type == kOutF32) p.tma_store = 0;  // FP32 rows leave with plain 16-byte stores
    }
#ifdef B200_TIMELINE
    p.timeline = g_timeline;
#endif

    rc = get_tensor_map(st, A, M, K, 128, 64, &p.tm_a);
    if (rc != B200_HGEMM_OK) return rc;
    // (tiles wider than 256 columns stage two slabs of bn / 4 rows per CTA, one per MMA)
    rc = get_tensor_map(st, B, N, K, static_cast<uint32_t>(bn > 256 ? bn / 4 : bn / cg), 64, &p.tm_b);
    if (rc != B200_HGEMM_OK) return rc;
    if (p.tma_store) {
        rc = get_tensor_map(st, C, M, N, 32, 64, &p.tm_c);
        if (rc != B200_HGEMM_OK) return rc;
    }

    uint32_t grid = 0;
    if (plan_cuts_k(pl)) {
        const uint32_t parts = streamk_parts(pl, st, p.tiles, p.k_blocks);
        // HYBRID: every full wave of tiles is walked whole; only the rest is cut into k-ranges
        if (pl.variant == B200_VARIANT_HYBRID || pl.variant == B200_VARIANT_HYBRID_PAIR) p.dp_tiles = (p.tiles / parts) * parts;
        if (p.tiles - p.dp_tiles > 65535u) return B200_HGEMM_ERR_UNSUPPORTED;  // the summing kernel's grid has one row per cut tile
        const uint64_t cut_units = static_cast<uint64_t>(p.tiles - p.dp_tiles) * p.k_blocks;
        p.sk_parts = cut_units < parts ? static_cast<uint32_t>(cut_units) : parts;  // no empty k-range
        const size_t need = kCounterBytes + static_cast<size_t>(parts) * 2u * (128u * cg * bn * sizeof(float));
        uint8_t *ws = nullptr;
        if (ws_override) {
            if (ws_override_bytes < need) return B200_HGEMM_ERR_WORKSPACE;
            ws = static_cast<uint8_t *>(ws_override);
        } else {
            rc = workspace_for(st, stream, need, &ws);
            if (rc != B200_HGEMM_OK) return rc;
        }
        p.partials = reinterpret_cast<float4 *>(ws + kCounterBytes);
        grid = parts * cg;
    } else {
        const uint32_t max_workers = (cg == 2) ? static_cast<uint32_t>(st.sm_count / 2) : static_cast<uint32_t>(st.sm_count);
        uint32_t workers = pl.grid > 0 ? static_cast<uint32_t>(pl.grid) / cg : max_workers;
        if (workers > p.tiles) workers = p.tiles;
        if (workers < 1) workers = 1;
        grid = workers * cg;
    }

    if (epi && !plan_cuts_k(pl)) {
        if (pl.variant == B200_VARIANT_CTA1) {
            if (bn == 256) return launch_kernel<256, 4, 1, kModeTiles, 1, true>(st, 16, p, grid, stream);
            if (bn == 192) return launch_kernel<192, 4, 1, kModeTiles, 1, true>(st, 21, p, grid, stream);
            if (bn == 128) return launch_kernel<128, 3, 1, kModeTiles, 2, true>(st, 17, p, grid, stream);
            return launch_kernel<64, 4, 1, kModeTiles, 2, true>(st, 18, p, grid, stream);
        }
        if (big) return launch_big_with_tail(st, p, grid, stream, true, pl.grid > 0);
        if (bn == 256) return launch_kernel<256, 6, 2, kModeTiles, 1, true>(st, 19, p, grid, stream);
        if (bn == 192) return launch_kernel<192, 3, 2, kModeTiles, 2, true>(st, 22, p, grid, stream);
        if (bn == 160) return launch_kernel<160, 3, 2, kModeTiles, 2, true>(st, 39, p, grid, stream);
        if (bn == 224) return launch_kernel<224, 3, 2, kModeTiles, 2, true>(st, 40, p, grid, stream);
        if (bn == 288) return launch_kernel<288, 5, 2, kModeTiles, 1, true>(st, 82, p, grid, stream);
        if (bn == 320) return launch_kernel<320, 5, 2, kModeTiles, 1, true>(st, 83, p, grid, stream);
        return launch_kernel<128, 4, 2, kModeTiles, 2, true>(st, 20, p, grid, stream);
    }
    if (pl.variant == B200_VARIANT_CTA1) {
        // a plan may ask for a shallower ring than the default (plan.stages; the autotuner's knob)
        if (bn == 256 && pl.stages == 3) return launch_kernel<256, 3, 1, kModeTiles>(st, 59, p, grid, stream);
        if (bn == 128 && pl.stages == 2) return launch_kernel<128, 2, 1, kModeTiles, 2>(st, 60, p, grid, stream);
        if (bn == 64 && pl.stages == 3) return launch_kernel<64, 3, 1, kModeTiles, 2>(st, 61, p, grid, stream);
        if (bn == 256) return launch_kernel<256, 4, 1, kModeTiles>(st, 0, p, grid, stream);
        if (bn == 192) return launch_kernel<192, 4, 1, kModeTiles>(st, 9, p, grid, stream);
        if (bn == 128) return launch_kernel<128, 3, 1, kModeTiles, 2>(st, 1, p, grid, stream);
        return launch_kernel<64, 4, 1, kModeTiles, 2>(st, 2, p, grid, stream);
    }
    if (big) return launch_big_with_tail(st, p, grid, stream, false, pl.grid > 0);
    if (pl.variant == B200_VARIANT_CTA2) {
        if (bn == 256 && pl.stages == 4) return launch_kernel<256, 4, 2, kModeTiles>(st, 62, p, grid, stream);
        if (bn == 256 && pl.stages == 5) return launch_kernel<256, 5, 2, kModeTiles>(st, 63, p, grid, stream);
        if (bn == 128 && pl.stages == 3) return launch_kernel<128, 3, 2, kModeTiles, 2>(st, 30, p, grid, stream);
        if (bn == 256) return launch_kernel<256, 6, 2, kModeTiles>(st, 3, p, grid, stream);
        if (bn == 192) return launch_kernel<192, 3, 2, kModeTiles, 2>(st, 10, p, grid, stream);
        if (bn == 160) return launch_kernel<160, 3, 2, kModeTiles, 2>(st, 37, p, grid, stream);
        if (bn == 224) return launch_kernel<224, 3, 2, kModeTiles, 2>(st, 38, p, grid, stream);
        if (bn == 288) return launch_kernel<288, 5, 2, kModeTiles>(st, 80, p, grid, stream);
        if (bn == 320) return launch_kernel<320, 5, 2, kModeTiles>(st, 81, p, grid, stream);
        return launch_kernel<128, 4, 2, kModeTiles, 2>(st, 4, p, grid, stream);
    }
    if (pl.variant == B200_VARIANT_HYBRID_PAIR) {
        if (epi) return B200_HGEMM_ERR_UNSUPPORTED;
        if (bn == 256) {
            rc = launch_kernel<256, 6, 2, kModeStreamK>(st, 31, p, grid, stream);
        } else {
            rc = launch_kernel<128, 4, 2, kModeStreamK, 2>(st, 36, p, grid, stream);
        }
    } else if (epi) {  // whole tiles get the epilogue in the kernel, cut tiles in the reduction below
        if (bn == 256) {
            rc = launch_kernel<256, 4, 1, kModeStreamK, 1, true>(st, 23, p, grid, stream);
        } else if (bn == 128) {
            rc = launch_kernel<128, 3, 1, kModeStreamK, 2, true>(st, 24, p, grid, stream);
        } else {
            rc = launch_kernel<64, 4, 1, kModeStreamK, 2, true>(st, 29, p, grid, stream);
        }
    } else if (bn == 256) {
        rc = launch_kernel<256, 4, 1, kModeStreamK>(st, 5, p, grid, stream);
    } else if (bn == 128) {
        rc = launch_kernel<128, 3, 1, kModeStreamK, 2>(st, 6, p, grid, stream);
    } else {
        rc = launch_kernel<64, 4, 1, kModeStreamK, 2>(st, 7, p, grid, stream);
    }
    if (rc != B200_HGEMM_OK) return rc;

    // Tiles whose k-range was cut across ranges left FP32 partials behind: sum them. Nothing to do
    // when every range boundary falls on a tile boundary.
    const uint32_t parts = p.sk_parts;
    const uint32_t cut_tiles = p.tiles - p.dp_tiles;
    if (cut_tiles == 0) return B200_HGEMM_OK;
    const uint64_t total_units = static_cast<uint64_t>(cut_tiles) * p.k_blocks;
    bool any_split = false;
    for (uint32_t part = 1; part < parts && !any_split; ++part) {
        any_split = (unit_begin(part, parts, total_units) % p.k_blocks) != 0;
    }
    if (!any_split) return B200_HGEMM_OK;
    ReduceParams rp;
    rp.partials = p.partials;
    rp.c = p.c;
    rp.m = p.m;
    rp.n = p.n;
    rp.m_blocks = p.m_blocks;
    rp.n_blocks = p.n_blocks;
    rp.k_blocks = p.k_blocks;
    rp.tiles = p.tiles;
    rp.dp_tiles = p.dp_tiles;
    rp.group_m = p.group_m;
    rp.parts = parts;
    rp.bn = static_cast<uint32_t>(bn);
    rp.cg = static_cast<uint32_t>(cg);
    rp.fused = epi ? 1u : 0u;
    rp.epi = ea;
    // One or two 16-byte words per thread: the sum over ranges is a chain of dependent-latency
    // loads, so the kernel gets its bandwidth from many resident threads, not from long loops.
    const uint32_t words = 128u * static_cast<uint32_t>(bn) / 4u;
    uint32_t chunks = (words + 2u * kReduceThreads - 1) / (2u * kReduceThreads);
    if (chunks < 1) chunks = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(chunks, cut_tiles, static_cast<unsigned>(cg));
    cfg.blockDim = dim3(kReduceThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (!cuda_ok(cudaLaunchKernelEx(&cfg, streamk_reduce_kernel, rp), "cudaLaunchKernelEx")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_HGEMM_OK;
}

static int entry(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, const b200_hgemm_plan *fixed,
                 int force_variant, cudaStream_t stream) {
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    b200_hgemm_plan pl;
    if (fixed) {
        pl = *fixed;
    } else {
        select_plan(*st, M, N, K, &pl);
        if (force_variant >= 0 && pl.variant != B200_VARIANT_SIMT) {
            if (force_variant == B200_VARIANT_SIMT) {
                pl.variant = B200_VARIANT_SIMT;
            } else if (force_variant == B200_VARIANT_CTA1) {
                if (pl.variant != B200_VARIANT_CTA1) pl.bn = 256;
                pl.variant = B200_VARIANT_CTA1;
                pl.parts = 0;
            } else if (force_variant == B200_VARIANT_CTA2) {
                pl.variant = B200_VARIANT_CTA2;
                pl.bn = 256;
                pl.parts = 0;
            } else if (force_variant == B200_VARIANT_STREAMK) {
                if (pl.variant != B200_VARIANT_STREAMK) pl.bn = 128;
                pl.variant = B200_VARIANT_STREAMK;
                pl.parts = 0;
            }
        } else if (force_variant == B200_VARIANT_SIMT) {
            pl.variant = B200_VARIANT_SIMT;
        }
    }
    return run_plan(*st, A, B, C, M, N, K, pl, stream, nullptr, 0);
}

// ------------------------------------------------------------------------------------------
// allocation-free stream-k: scratch in a static device array
// ------------------------------------------------------------------------------------------
// Layout: [256 B error word | 64 KiB reserved | 16 MiB FP32 partial-tile slots].
// 16 MiB holds 2 slots of 128 x 128 floats for each of 128 k-ranges, which is the most the
// entry point launches. Every GPU on which this library is loaded keeps these 16.06 MiB
// reserved until the process exits, whether or not the entry point is ever called.
constexpr size_t kStaticHeaderBytes = 256;
constexpr size_t kStaticPartialBytes = size_t(16) << 20;
constexpr size_t kStaticScratchBytes = kStaticHeaderBytes + kCounterBytes + kStaticPartialBytes;
constexpr int kStaticBn = 128;
constexpr uint32_t kStaticMaxParts = kStaticPartialBytes / (2u * 128u * kStaticBn * sizeof(float));  // 128

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// What the allocation-free entry point knows about a device. In host code the name
// g_static_scratch is only the runtime's handle for the array, not an address a kernel can
// use: the device address is asked for once per device, while that device is current.
struct StaticDevice {
    bool ready = false;
    bool sm100 = false;
    int sm_count = 0;
    unsigned char *scratch = nullptr;
};
static std::mutex g_static_mu;
static StaticDevice g_static_dev[kMaxDevices];

static int static_device(int dev, StaticDevice *out) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDevice &sd = g_static_dev[dev];
    if (!sd.ready) {
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            return B200_HGEMM_ERR_CUDA;
        }
        sd.sm100 = (major == 10);
        sd.sm_count = sms;
        if (sd.sm100) {
            void *ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return B200_HGEMM_ERR_CUDA;
            }
            sd.scratch = static_cast<unsigned char *>(ptr);
        }
        sd.ready = true;
    }
    *out = sd;
    return B200_HGEMM_OK;
}

}  // namespace b200

using namespace b200;

// ------------------------------------------------------------------------------------------
// extern "C"
// ------------------------------------------------------------------------------------------
extern "C" {

int b200_hgemm(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    return entry(A, B, C, M, N, K, nullptr, -1, reinterpret_cast<cudaStream_t>(stream));
}

int b200_hgemm_cta1(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    return entry(A, B, C, M, N, K, nullptr, B200_VARIANT_CTA1, reinterpret_cast<cudaStream_t>(stream));
}

int b200_hgemm_cta2(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    return entry(A, B, C, M, N, K, nullptr, B200_VARIANT_CTA2, reinterpret_cast<cudaStream_t>(stream));
}

int b200_hgemm_streamk(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    return entry(A, B, C, M, N, K, nullptr, B200_VARIANT_STREAMK, reinterpret_cast<cudaStream_t>(stream));
}

// Split-k with a fixed number of k-slices per tile: the stream-k kernel launched with
// tiles x slices equal ranges, so that every CTA owns exactly one slice of one tile.
int b200_hgemm_splitk(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    b200_hgemm_plan pl;
    select_plan(*st, M, N, K, &pl);
    const uint64_t tiles128 = static_cast<uint64_t>(ceil_div_u32(M, 128)) * ceil_div_u32(N, 128);
    if (pl.variant != B200_VARIANT_SIMT && tiles128 >= static_cast<uint64_t>(st->sm_count)) {
        // every SM has a tile of its own already: one slice per tile, i.e. whole 128 x 128 tiles and no workspace
        // (two slices of a 16384^2 output would want 4 GiB of partial tiles)
        memset(&pl, 0, sizeof(pl));
        pl.variant = B200_VARIANT_CTA1;
        pl.bn = 128;
        pl.tma_store = (N % 8 == 0) ? 1 : 0;
    } else if (pl.variant != B200_VARIANT_SIMT) {
        pl.variant = B200_VARIANT_STREAMK;
        pl.bn = 128;
        const uint32_t tiles = ceil_div_u32(M, 128) * ceil_div_u32(N, 128);
        const uint32_t k_blocks = plan_k_units(pl, K);  // the kernel's own unit of k: one pipeline stage
        uint32_t slices = (static_cast<uint32_t>(st->sm_count) + tiles - 1) / tiles;
        if (slices < 2) slices = 2;
        while (slices > 1 && k_blocks % slices != 0) --slices;  // equal slices only
        if (slices > k_blocks) slices = k_blocks;
        pl.parts = static_cast<int32_t>(tiles * slices);
    }
    return run_plan(*st, A, B, C, M, N, K, pl, reinterpret_cast<cudaStream_t>(stream), nullptr, 0);
}


// Stream-k GEMM that allocates nothing. It is meant for callers that cannot call cudaMalloc at
// the point where they need a GEMM: code running under a memory pool that owns all device
// memory, a latency-critical serving loop in which an allocation (which may synchronise the
// device) is not acceptable, or a plugin whose host forbids allocations after start-up. The
// other entry points create or grow a workspace on first use; this one keeps its scratch in
// the static device array above and calls no allocating routine.
//
//  * Limits: K % 8 == 0 (as for every tensor-core variant) and at most 16384 output tiles of
//    128 x 128, i.e. ceil(M/128) * ceil(N/128) <= 16384; beyond that the call returns
//    B200_HGEMM_ERR_TOO_LARGE. The k-ranges are capped at 128 so that their partial tiles fit
//    the 16 MiB array.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress),
//    sets the kernel's shared-memory attribute and encodes tensor maps. Make that first call
//    outside any stream capture.
//  * All calls on a device share the one array, which keeps whatever the last call left in it.
//    Each call clears the error word and the reserved header, stream-ordered, before its kernel;
//    partial tiles are always written before they are read. Two calls whose kernels overlap on
//    the GPU (different streams with no dependency between them) race on the array: serialise them.
//  * A bounded wait that expires inside this variant is recorded in the first word of the
//    array, not in the word b200_hgemm_last_device_error() reads: b200_hgemm_streamk_static_last_error()
//    reads and clears it (it allocates nothing either).
int b200_hgemm_streamk_static(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                              b200_stream_t stream) {
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    if (K % 8 != 0) return B200_HGEMM_ERR_UNSUPPORTED;
    const uint64_t tiles = static_cast<uint64_t>(ceil_div_u32(M, 128)) * ceil_div_u32(N, kStaticBn);
    if (tiles > kMaxCountedTiles) return B200_HGEMM_ERR_TOO_LARGE;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_HGEMM_ERR_CUDA;
    StaticDevice sd;
    rc = static_device(dev, &sd);
    if (rc != B200_HGEMM_OK) return rc;
    if (!sd.sm100) return B200_HGEMM_ERR_NO_SM100;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // the error word has to start at zero (the reserved header is cleared with it)
    if (!cuda_ok(cudaMemsetAsync(sd.scratch, 0, kStaticHeaderBytes + kCounterBytes, s), "cudaMemsetAsync")) return B200_HGEMM_ERR_CUDA;

    b200_hgemm_plan pl;
    memset(&pl, 0, sizeof(pl));
    pl.variant = B200_VARIANT_STREAMK;
    pl.bn = kStaticBn;
    pl.tma_store = (N % 8 == 0) ? 1 : 0;
    uint32_t parts = static_cast<uint32_t>(sd.sm_count);
    if (parts > kStaticMaxParts) parts = kStaticMaxParts;
    pl.parts = static_cast<int32_t>(parts);
    // g_dev[dev] serves as the cache of tensor maps and kernel attributes; its attributes are filled
    // in here if no other entry point has yet, and nothing in it is allocated on this path
    {
        std::lock_guard<std::mutex> lock(g_dev[dev].mu);
        rc = probe_attributes_locked(g_dev[dev], dev);
        if (rc != B200_HGEMM_OK) return rc;
    }
    return run_plan(g_dev[dev], A, B, C, M, N, K, pl, s, sd.scratch + kStaticHeaderBytes,
                    kCounterBytes + kStaticPartialBytes, reinterpret_cast<uint32_t *>(sd.scratch));
}

int b200_hgemm_simt(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    return entry(A, B, C, M, N, K, nullptr, B200_VARIANT_SIMT, reinterpret_cast<cudaStream_t>(stream));
}

// ---- stacks of matrices -------------------------------------------------------------------
// One launch for `batch` products of the same shape: the whole-tile kernels with three-dimensional
// tensor maps ({columns, rows, matrices}) and tile ids that run over all matrices, so that small
// products fill the GPU together. The tile is chosen by the shape of one product and by how many
// tiles the stack has in total.
static int run_batched(DeviceState &st, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, size_t batch,
                       size_t stride_a, size_t stride_b, size_t stride_c, cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) {
        return B200_HGEMM_ERR_MISALIGNED;
    }
    if ((stride_a | stride_b | stride_c) % 8 != 0) return B200_HGEMM_ERR_MISALIGNED;  // every matrix 16-byte aligned
    const uint32_t sms = st.sm_count > 0 ? static_cast<uint32_t>(st.sm_count) : 148u;
    const uint64_t m_blocks128 = ceil_div_u32(M, 128);
    // pairs on 256 x 256 when one product alone has rows for them and the stack fills the pairs twice over;
    // else single CTAs on the widest tile that still gives every SM one
    const uint64_t pair_tiles = static_cast<uint64_t>(ceil_div_u32(M, 256)) * ceil_div_u32(N, 256) * batch;
    int cg = 1, bn = 256;
    if (M > 128 && N > 128 && pair_tiles >= sms) {
        cg = 2;
    } else {
        while (bn > 64 && (N <= static_cast<size_t>(bn) / 2 || m_blocks128 * ceil_div_u32(N, bn) * batch < sms)) bn /= 2;
    }
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.c = static_cast<__half *>(C);
    p.error_word = st.error_word;
    p.m = static_cast<uint32_t>(M);
    p.n = static_cast<uint32_t>(N);
    p.k = static_cast<uint32_t>(K);
    p.m_blocks = ceil_div_u32(M, 128u * cg);
    p.n_blocks = ceil_div_u32(N, bn);
    const uint32_t kps = (cg == 1 && bn != 256) ? 2u : 1u;
    p.k_blocks = ceil_div_u32(K, 64u * kps);
    const uint64_t tiles = static_cast<uint64_t>(p.m_blocks) * p.n_blocks * batch;
    if (tiles > 0x7fffffffull || batch > 0x7fffffffull) return B200_HGEMM_ERR_UNSUPPORTED;
    p.tiles = static_cast<uint32_t>(tiles);
    p.group_m = p.m_blocks < 16u ? p.m_blocks : 16u;
    p.raster = make_raster(p.m_blocks, p.n_blocks, p.group_m);
    p.tma_store = (N % 8 == 0) ? 1u : 0u;
    p.c_vec_ok = p.tma_store;
    p.batch_stride_c = stride_c;
    int rc = get_tensor_map(st, A, M, K, 128, 64, &p.tm_a, true, batch, stride_a);
    if (rc != B200_HGEMM_OK) return rc;
    if ((rc = get_tensor_map(st, B, N, K, static_cast<uint32_t>(bn / cg), 64, &p.tm_b, true, batch, stride_b)) != B200_HGEMM_OK) return rc;
    if (p.tma_store && (rc = get_tensor_map(st, C, M, N, 32, 64, &p.tm_c, true, batch, stride_c)) != B200_HGEMM_OK) return rc;
    const uint32_t max_workers = static_cast<uint32_t>(st.sm_count) / cg;
    const uint32_t grid = (p.tiles < max_workers ? p.tiles : max_workers) * cg;
    if (cg == 2) return launch_kernel<256, 6, 2, kModeTiles, 1, false, kFlavorBatched>(st, 50, p, grid, stream);
    if (bn == 256) return launch_kernel<256, 4, 1, kModeTiles, 1, false, kFlavorBatched>(st, 51, p, grid, stream);
    if (bn == 128) return launch_kernel<128, 3, 1, kModeTiles, 2, false, kFlavorBatched>(st, 52, p, grid, stream);
    return launch_kernel<64, 4, 1, kModeTiles, 2, false, kFlavorBatched>(st, 53, p, grid, stream);
}

// ---- B stored K x N row-major -----------------------------------------------------------------
// The whole-tile kernels with B as an MN-major operand of the MMA (FLAVOR kFlavorBkn): the tile is the
// dispatch's choice for the shape mapped onto single CTAs of 64 / 128 / 256 columns or pairs on 256 x 128 /
// 256 x 256.
static int run_bkn(DeviceState &st, const void *A, const void *B, void *C, size_t M, size_t N, size_t K, cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) {
        return B200_HGEMM_ERR_MISALIGNED;
    }
    if (K % 8 != 0 || N % 8 != 0) return B200_HGEMM_ERR_UNSUPPORTED;  // row pitches of A (K halves) and of B, C (N halves)
    b200_hgemm_plan pl;
    select_plan(st, M, N, K, &pl, false);
    int cg = 1, bn = 256;
    if (pl.variant == B200_VARIANT_CTA2 || pl.variant == B200_VARIANT_CTA2_MCAST) {
        cg = 2;
        bn = pl.bn == 128 ? 128 : 256;
    } else if (pl.variant == B200_VARIANT_CTA1 || plan_cuts_k(pl)) {
        bn = pl.bn == 192 ? 256 : pl.bn;
    } else {  // decode-like shapes: narrow single-CTA tiles spread N over the SMs
        bn = ceil_div_u32(N, 128) * 2 >= static_cast<uint32_t>(st.sm_count) ? 128 : 64;
    }
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.c = static_cast<__half *>(C);
    p.error_word = st.error_word;
    p.m = static_cast<uint32_t>(M);
    p.n = static_cast<uint32_t>(N);
    p.k = static_cast<uint32_t>(K);
    p.m_blocks = ceil_div_u32(M, 128u * cg);
    p.n_blocks = ceil_div_u32(N, bn);
    const uint32_t kps = ((cg == 1 && bn != 256) || (cg == 2 && bn == 128)) ? 2u : 1u;
    p.k_blocks = ceil_div_u32(K, 64u * kps);
    const uint64_t tiles = static_cast<uint64_t>(p.m_blocks) * p.n_blocks;
    if (tiles > 0x7fffffffull) return B200_HGEMM_ERR_UNSUPPORTED;
    p.tiles = static_cast<uint32_t>(tiles);
    p.group_m = cg == 2 ? 8u : 16u;
    if (p.group_m > p.m_blocks) p.group_m = p.m_blocks;
    p.raster = make_raster(p.m_blocks, p.n_blocks, p.group_m);
    p.tma_store = 1;
    p.c_vec_ok = 1;
    int rc = get_tensor_map(st, A, M, K, 128, 64, &p.tm_a);
    if (rc != B200_HGEMM_OK) return rc;
    if ((rc = get_tensor_map(st, B, K, N, 64, 64, &p.tm_b)) != B200_HGEMM_OK) return rc;  // K rows of N halves, boxes of 64 x 64
    if ((rc = get_tensor_map(st, C, M, N, 32, 64, &p.tm_c)) != B200_HGEMM_OK) return rc;
    const uint32_t max_workers = static_cast<uint32_t>(st.sm_count) / cg;
    const uint32_t grid = (p.tiles < max_workers ? p.tiles : max_workers) * cg;
    if (cg == 2) {
        if (bn == 256) return launch_kernel<256, 6, 2, kModeTiles, 1, false, kFlavorBkn>(st, 54, p, grid, stream);
        return launch_kernel<128, 4, 2, kModeTiles, 2, false, kFlavorBkn>(st, 55, p, grid, stream);
    }
    if (bn == 256) return launch_kernel<256, 4, 1, kModeTiles, 1, false, kFlavorBkn>(st, 56, p, grid, stream);
    if (bn == 128) return launch_kernel<128, 3, 1, kModeTiles, 2, false, kFlavorBkn>(st, 57, p, grid, stream);
    return launch_kernel<64, 4, 1, kModeTiles, 2, false, kFlavorBkn>(st, 58, p, grid, stream);
}

int b200_hgemm_bkn(const void *A, const void *B_kn, void *C, size_t M, size_t N, size_t K, b200_stream_t stream) {
    int rc = check_args(A, B_kn, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    return run_bkn(*st, A, B_kn, C, M, N, K, reinterpret_cast<cudaStream_t>(stream));
}

int b200_hgemm_batched(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, size_t batch, size_t stride_a,
                       size_t stride_b, size_t stride_c, b200_stream_t stream) {
    if (batch == 0) return B200_HGEMM_ERR_INVALID_ARG;
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    // matrices of a stack may share B (stride 0) but must not overlap otherwise
    if (stride_a < M * K || stride_c < M * N || (stride_b != 0 && stride_b < N * K)) {
        if (batch > 1) return B200_HGEMM_ERR_INVALID_ARG;
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (batch == 1) return entry(A, B, C, M, N, K, nullptr, -1, s);
    // one B for the whole stack and A, C densely stacked: that is one product with batch * M rows
    if (stride_b == 0 && stride_a == M * K && stride_c == M * N) return entry(A, B, C, batch * M, N, K, nullptr, -1, s);
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    if (K % 8 != 0 || stride_b == 0) {
        // no tensor map for these rows (K % 8 != 0), or a shared B under A and C that are not densely stacked:
        // one product after the other on the stream
        for (size_t i = 0; i < batch; ++i) {
            rc = entry(static_cast<const __half *>(A) + i * stride_a, static_cast<const __half *>(B) + i * stride_b,
                       static_cast<__half *>(C) + i * stride_c, M, N, K, nullptr, -1, s);
            if (rc != B200_HGEMM_OK) return rc;
        }
        return B200_HGEMM_OK;
    }
    return run_batched(*st, A, B, C, M, N, K, batch, stride_a, stride_b, stride_c, s);
}

int b200_hgemm_ex(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, const b200_hgemm_plan *plan,
                  b200_stream_t stream) {
    if (!plan) return B200_HGEMM_ERR_INVALID_ARG;
    return entry(A, B, C, M, N, K, plan, -1, reinterpret_cast<cudaStream_t>(stream));
}

// The dispatch's plan for the shape, as the fused epilogue can run it: every kernel family carries it; the
// multicast variants run as the same tiles on plain pairs, and FP32 output leaves the 256 x 256-per-CTA
// arrangement (whose epilogue packs 16-bit values) for 128 x 256 per CTA.
static int fused_plan(const DeviceState &st, size_t M, size_t N, size_t K, int c_type, b200_hgemm_plan *pl) {
    select_plan(st, M, N, K, pl);
    if (pl->variant == B200_VARIANT_SIMT) return B200_HGEMM_ERR_UNSUPPORTED;  // K % 8 != 0
    if (pl->variant == B200_VARIANT_CTA2_MCAST || pl->variant == B200_VARIANT_HYBRID_PAIR) pl->variant = B200_VARIANT_CTA2;
    if (pl->variant == B200_VARIANT_CTA2 && pl->bn == 512 && c_type == B200_C_F32) pl->bn = 256;
    return B200_HGEMM_OK;
}

int b200_hgemm_fused(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, const b200_hgemm_epilogue *epilogue,
                     b200_stream_t stream) {
    if (!epilogue) return B200_HGEMM_ERR_INVALID_ARG;
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    b200_hgemm_plan pl;
    rc = fused_plan(*st, M, N, K, epilogue->c_type, &pl);
    if (rc != B200_HGEMM_OK) return rc;
    return run_plan(*st, A, B, C, M, N, K, pl, reinterpret_cast<cudaStream_t>(stream), nullptr, 0, nullptr, epilogue);
}

int b200_hgemm_fused_ex(const void *A, const void *B, void *C, size_t M, size_t N, size_t K, const b200_hgemm_epilogue *epilogue,
                        const b200_hgemm_plan *plan, b200_stream_t stream) {
    if (!epilogue || !plan) return B200_HGEMM_ERR_INVALID_ARG;
    int rc = check_args(A, B, C, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    if (plan->variant == B200_VARIANT_SIMT || plan->variant == B200_VARIANT_CTA2_MCAST) return B200_HGEMM_ERR_UNSUPPORTED;
    return run_plan(*st, A, B, C, M, N, K, *plan, reinterpret_cast<cudaStream_t>(stream), nullptr, 0, nullptr, epilogue);
}

int b200_hgemm_select(size_t M, size_t N, size_t K, b200_hgemm_plan *plan) {
    if (!plan || M == 0 || N == 0 || K == 0) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) {
        // no usable device: still answer, for a nominal 148-SM part, so that planning can be tested on the host
        cudaGetLastError();
        static DeviceState nominal;
        nominal.sm_count = 148;
        select_plan(nominal, M, N, K, plan);
        return B200_HGEMM_OK;
    }
    select_plan(*st, M, N, K, plan);
    return B200_HGEMM_OK;
}

int b200_hgemm_enable_multicast(int on) {
    mc_state();  // what the environment says comes first (it may lock the switch)
    return mc_enable(on != 0);
}

int b200_hgemm_multicast_state(void) {
    return mc_state();
}

int b200_hgemm_plan_supported(size_t M, size_t N, size_t K, const b200_hgemm_plan *plan) {
    if (!plan || M == 0 || N == 0 || K == 0) return B200_HGEMM_ERR_INVALID_ARG;
    const int rc = validate_plan(*plan, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    if (plan->variant == B200_VARIANT_SKINNY || plan->variant == B200_VARIANT_SKINNY_PAIR) {
        if (M > static_cast<size_t>(plan->bn)) return B200_HGEMM_ERR_UNSUPPORTED;
        if (plan->grid == 1) {
            // the k-ranges of a tile must fit one cluster of at most eight CTAs (no device is asked: where the
            // plan leaves the number of k-ranges to the library, a B200's 148 SMs are assumed)
            DeviceState nominal;
            nominal.sm_count = 148;
            if (skinny_sums_on_chip(*plan, skinny_slices(*plan, nominal, N, K)) < 0) return B200_HGEMM_ERR_UNSUPPORTED;
        }
    }
    return B200_HGEMM_OK;
}

int b200_hgemm_load_plan_table(const char *path) {
    std::vector<TunedPlan> fresh;
    int entries = 0;
    if (path && (entries = read_plan_table(path, &fresh)) < 0) return B200_HGEMM_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_table_mu);
    g_table.swap(fresh);
    g_table_loaded = true;
    return entries;
}

int b200_hgemm_select_untuned(size_t M, size_t N, size_t K, b200_hgemm_plan *plan) {
    if (!plan || M == 0 || N == 0 || K == 0) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceState *st = nullptr;
    if (current_state(&st) != B200_HGEMM_OK) {
        cudaGetLastError();
        DeviceState nominal;
        nominal.sm_count = 148;
        select_plan(nominal, M, N, K, plan, false);
        return B200_HGEMM_OK;
    }
    select_plan(*st, M, N, K, plan, false);
    return B200_HGEMM_OK;
}

size_t b200_hgemm_workspace_bytes(size_t M, size_t N, size_t K, const b200_hgemm_plan *plan) {
    if (!plan || M == 0 || N == 0 || K == 0) return 0;
    if (plan->variant == B200_VARIANT_SKINNY || plan->variant == B200_VARIANT_SKINNY_PAIR) {
        if (validate_plan(*plan, N, K) != B200_HGEMM_OK) return 0;
        DeviceState *st = nullptr;
        if (current_state(&st) != B200_HGEMM_OK) {
            cudaGetLastError();
            DeviceState nominal;
            nominal.sm_count = 148;
            return skinny_workspace_bytes(*plan, nominal, N, K);
        }
        return skinny_workspace_bytes(*plan, *st, N, K);
    }
    if (!plan_cuts_k(*plan)) return 0;
    if (plan->bn != 64 && plan->bn != 128 && plan->bn != 256) return 0;
    DeviceState *st = nullptr;
    if (current_state(&st) != B200_HGEMM_OK) {
        cudaGetLastError();
        static DeviceState nominal;
        nominal.sm_count = 148;
        return plan_workspace_bytes(nominal, M, N, K, *plan);
    }
    return plan_workspace_bytes(*st, M, N, K, *plan);
}

int b200_hgemm_set_workspace(void *workspace, size_t bytes) {
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (workspace && ((reinterpret_cast<uintptr_t>(workspace) & 255u) || bytes < kCounterBytes)) {
        return B200_HGEMM_ERR_WORKSPACE;
    }
    std::lock_guard<std::mutex> lock(st->mu);
    st->ws = workspace;
    st->ws_bytes = workspace ? bytes : 0;
    return B200_HGEMM_OK;
}

int b200_hgemm_release_workspaces(void) {
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    std::lock_guard<std::mutex> lock(st->mu);
    int freed = 0;
    for (auto &w : st->owned_ws) {
        if (w.ptr && cuda_ok(cudaFree(w.ptr), "cudaFree")) ++freed;  // waits for work that still uses it
    }
    st->owned_ws.clear();
    return freed;
}

// Reads the error word behind work already complete on `stream` (4 bytes, ordered on that stream).
static int read_error_word(uint32_t *word_dev, cudaStream_t stream, uint32_t *word) {
    *word = 0;
    if (!cuda_ok(cudaMemcpyAsync(word, word_dev, sizeof(*word), cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync")) return B200_HGEMM_ERR_CUDA;
    if (!cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    if (*word != 0) {
        if (!cuda_ok(cudaMemsetAsync(word_dev, 0, sizeof(*word), stream), "cudaMemsetAsync")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    }
    return B200_HGEMM_OK;
}

int b200_hgemm_synchronize(b200_stream_t stream) {
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    uint32_t word = 0;
    rc = read_error_word(st->error_word, reinterpret_cast<cudaStream_t>(stream), &word);
    if (rc != B200_HGEMM_OK) return rc;
    return word != 0 ? B200_HGEMM_ERR_DEVICE_WAIT : B200_HGEMM_OK;
}

int b200_hgemm_streamk_static_last_error(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_HGEMM_ERR_CUDA;
    StaticDevice sd;
    int rc = static_device(dev, &sd);
    if (rc != B200_HGEMM_OK) return rc;
    if (!sd.sm100) return B200_HGEMM_ERR_NO_SM100;
    if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return B200_HGEMM_ERR_CUDA;
    uint32_t word = 0;
    if (!cuda_ok(cudaMemcpy(&word, sd.scratch, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy")) return B200_HGEMM_ERR_CUDA;
    if (word != 0) cudaMemset(sd.scratch, 0, sizeof(word));
    return static_cast<int>(word);
}

int b200_hgemm_last_device_error(void) {
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return B200_HGEMM_ERR_CUDA;
    uint32_t word = 0;
    if (!cuda_ok(cudaMemcpy(&word, st->error_word, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy")) {
        return B200_HGEMM_ERR_CUDA;
    }
    if (word != 0) cudaMemset(st->error_word, 0, sizeof(word));
    return static_cast<int>(word);
}

const char *b200_hgemm_status_string(int status) {
    switch (status) {
        case B200_HGEMM_OK: return "ok";
        case B200_HGEMM_ERR_INVALID_ARG: return "invalid argument (null pointer or zero dimension)";
        case B200_HGEMM_ERR_UNSUPPORTED: return "unsupported shape or plan";
        case B200_HGEMM_ERR_MISALIGNED: return "pointer not 16-byte aligned";
        case B200_HGEMM_ERR_NO_SM100: return "current device is not an sm_100 GPU (no fallback exists)";
        case B200_HGEMM_ERR_CUDA: return "CUDA call failed";
        case B200_HGEMM_ERR_WORKSPACE: return "split-k workspace missing or too small";
        case B200_HGEMM_ERR_DEVICE_WAIT: return "a kernel gave up on a bounded wait";
        case B200_HGEMM_ERR_TOO_LARGE: return "size beyond the entry point's stated maximum";
        default: return "unknown status";
    }
}

const char *b200_hgemm_version(void) {
    return "b200_hgemm 0.1 (sm_100a, tcgen05/TMEM/TMA)";
}

uint64_t b200_hgemm_launch_count(void) {
    return g_launches.load(std::memory_order_relaxed);
}

// ---- host-pointer entry point -----------------------------------------------------------
static int grow(void **ptr, size_t *have, size_t need) {
    if (*have >= need) return B200_HGEMM_OK;
    if (*ptr) {
        if (!cuda_ok(cudaFree(*ptr), "cudaFree")) return B200_HGEMM_ERR_CUDA;
        *ptr = nullptr;
        *have = 0;
    }
    if (!cuda_ok(cudaMalloc(ptr, need), "cudaMalloc")) {
        cudaGetLastError();
        return B200_HGEMM_ERR_CUDA;
    }
    *have = need;
    return B200_HGEMM_OK;
}

// A and C on the host; B on the host (b_on_device = false: uploaded first) or already on the device.
// upload_after / gemm_after (b_on_device only, either may be null): events the caller recorded; A's first upload
// waits for the one, the first multiply for the other, so that the uploads of A can run while B is still being
// completed on the device (e.g. by an exchange between GPUs).
static int host_pipeline(const void *A_host, const void *B_any, void *C_host, size_t M, size_t N, size_t K, bool b_on_device,
                         cudaEvent_t upload_after = nullptr, cudaEvent_t gemm_after = nullptr) {
    const void *B_host = B_any;
    int rc = check_args(A_host, B_any, C_host, M, N, K);
    if (rc != B200_HGEMM_OK) return rc;
    DeviceState *st = nullptr;
    rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    const size_t a_bytes = M * K * sizeof(__half), b_bytes = N * K * sizeof(__half), c_bytes = M * N * sizeof(__half);
    // one host-pointer GEMM per device at a time: the staging buffers and the two streams are shared
    static std::mutex host_call_mu[kMaxDevices];
    int host_dev = 0;
    if (cudaGetDevice(&host_dev) != cudaSuccess || host_dev < 0 || host_dev >= kMaxDevices) return B200_HGEMM_ERR_CUDA;
    std::lock_guard<std::mutex> host_lock(host_call_mu[host_dev]);
    {
        std::lock_guard<std::mutex> lock(st->mu);
        if ((rc = grow(&st->host_a, &st->host_a_bytes, a_bytes)) != B200_HGEMM_OK) return rc;
        if (!b_on_device && (rc = grow(&st->host_b, &st->host_b_bytes, b_bytes)) != B200_HGEMM_OK) return rc;
        if ((rc = grow(&st->host_c, &st->host_c_bytes, c_bytes)) != B200_HGEMM_OK) return rc;
        for (int i = 0; i < 3; ++i) {
            if (!st->host_stream[i] && cudaStreamCreateWithFlags(&st->host_stream[i], cudaStreamNonBlocking) != cudaSuccess)
                return B200_HGEMM_ERR_CUDA;
        }
        for (int i = 0; i < 2; ++i) {
            if (!st->host_event[i] && cudaEventCreateWithFlags(&st->host_event[i], cudaEventDisableTiming) != cudaSuccess)
                return B200_HGEMM_ERR_CUDA;
        }
    }
    // B first (every row slab needs all of it), then A and C move in row slabs on three streams:
    // the upload of slab i+1, the GEMM of slab i and the download of slab i-1 run at the same
    // time. The link carries both directions at once (measured: 1 GiB up and 0.5 GiB down together
    // take 20.5 ms, 19.3 ms the upload alone), so what the call adds to the upload of A and B is the
    // GEMM and the download of the last slab: slabs of about 1024 rows keep that under a millisecond
    // at N = K = 16384.
    cudaStream_t s_up = st->host_stream[0], s_run = st->host_stream[1], s_down = st->host_stream[2];
    // Whatever ends the call, it returns only when nothing it queued is still running: the caller
    // may free or reuse its host buffers at once, and the staging buffers are free for the next call.
    struct Drain {
        cudaStream_t s[3];
        ~Drain() {
            for (cudaStream_t x : s) cudaStreamSynchronize(x);
            cudaGetLastError();
        }
    } drain{{s_up, s_run, s_down}};
    const void *b_dev = B_any;
    if (!b_on_device) {
        if (!cuda_ok(cudaMemcpyAsync(st->host_b, B_host, b_bytes, cudaMemcpyHostToDevice, s_up), "cudaMemcpyAsync")) return B200_HGEMM_ERR_CUDA;
        b_dev = st->host_b;
    }
    if (upload_after && !cuda_ok(cudaStreamWaitEvent(s_up, upload_after, 0), "cudaStreamWaitEvent")) return B200_HGEMM_ERR_CUDA;
    if (gemm_after && !cuda_ok(cudaStreamWaitEvent(s_run, gemm_after, 0), "cudaStreamWaitEvent")) return B200_HGEMM_ERR_CUDA;
    size_t slabs = 1;
    if (M >= 2048 && M % 128 == 0) {
        slabs = M >= 16384 ? 16 : M >= 8192 ? 8 : 4;
        while (slabs > 1 && (M / 128) % slabs != 0) --slabs;
    }
    const size_t rows = M / slabs;
    // What the call adds to the uploads is the GEMM and the download of the last slab: the last slab is
    // cut into four once more (when its quarters are still whole 128-row blocks).
    const size_t tail_parts = (slabs > 1 && rows % 512 == 0) ? 4 : 1;
    const size_t pieces = slabs - 1 + tail_parts;
    size_t row0 = 0;
    for (size_t s = 0; s < pieces; ++s) {
        const size_t rows_here = (s < slabs - 1) ? rows : rows / tail_parts;
        const char *a_src = static_cast<const char *>(A_host) + row0 * K * sizeof(__half);
        char *a_dst = static_cast<char *>(st->host_a) + row0 * K * sizeof(__half);
        char *c_dev = static_cast<char *>(st->host_c) + row0 * N * sizeof(__half);
        char *c_dst = static_cast<char *>(C_host) + row0 * N * sizeof(__half);
        if (!cuda_ok(cudaMemcpyAsync(a_dst, a_src, rows_here * K * sizeof(__half), cudaMemcpyHostToDevice, s_up), "cudaMemcpyAsync"))
            return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaEventRecord(st->host_event[0], s_up), "cudaEventRecord")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaStreamWaitEvent(s_run, st->host_event[0], 0), "cudaStreamWaitEvent")) return B200_HGEMM_ERR_CUDA;
        rc = entry(a_dst, b_dev, c_dev, rows_here, N, K, nullptr, -1, s_run);
        if (rc != B200_HGEMM_OK) return rc;
        if (!cuda_ok(cudaEventRecord(st->host_event[1], s_run), "cudaEventRecord")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaStreamWaitEvent(s_down, st->host_event[1], 0), "cudaStreamWaitEvent")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaMemcpyAsync(c_dst, c_dev, rows_here * N * sizeof(__half), cudaMemcpyDeviceToHost, s_down), "cudaMemcpyAsync"))
            return B200_HGEMM_ERR_CUDA;
        row0 += rows_here;
    }
    if (!cuda_ok(cudaStreamSynchronize(s_down), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    if (!cuda_ok(cudaStreamSynchronize(s_run), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    if (!cuda_ok(cudaStreamSynchronize(s_up), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    return B200_HGEMM_OK;
}

int b200_hgemm_host(const void *A_host, const void *B_host, void *C_host, size_t M, size_t N, size_t K) {
    return host_pipeline(A_host, B_host, C_host, M, N, K, false);
}

int b200_hgemm_host_a(const void *A_host, const void *B_device, void *C_host, size_t M, size_t N, size_t K) {
    if (reinterpret_cast<uintptr_t>(B_device) & 15u) return B200_HGEMM_ERR_MISALIGNED;
    return host_pipeline(A_host, B_device, C_host, M, N, K, true);
}

int b200_hgemm_host_a_after(const void *A_host, const void *B_device, void *C_host, size_t M, size_t N, size_t K,
                            b200_event_t upload_after, b200_event_t gemm_after) {
    if (reinterpret_cast<uintptr_t>(B_device) & 15u) return B200_HGEMM_ERR_MISALIGNED;
    return host_pipeline(A_host, B_device, C_host, M, N, K, true, reinterpret_cast<cudaEvent_t>(upload_after),
                         reinterpret_cast<cudaEvent_t>(gemm_after));
}

// ---- several GPUs from one process ----------------------------------------------------------
struct b200_mg {
    int n = 0;
    int devices[kMaxDevices] = {};
    cudaStream_t streams[kMaxDevices] = {};
    cudaEvent_t start[kMaxDevices] = {};
    cudaEvent_t stop[kMaxDevices] = {};
    bool timed[kMaxDevices] = {};  // whether the last b200_mg_hgemm launched anything on the device
};

// Keeps the calling thread's current device across a loop over devices.
struct DeviceRestore {
    int prev = -1;
    DeviceRestore() {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    }
    ~DeviceRestore() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Row blocks of 128 dealt out evenly over n devices, the first ones a block more.
static void partition_slab(size_t M, int n, int index, size_t *row0, size_t *rows) {
    const size_t blocks = (M + 127) / 128;
    const size_t base = blocks / n, extra = blocks % n;
    const size_t idx = static_cast<size_t>(index);
    const size_t begin = idx * base + (idx < extra ? idx : extra);
    const size_t count = base + (idx < extra ? 1 : 0);
    const size_t lo = begin * 128 < M ? begin * 128 : M;
    const size_t hi = (begin + count) * 128 < M ? (begin + count) * 128 : M;
    *row0 = lo;
    *rows = hi - lo;
}

static void mg_slab(const b200_mg *mg, size_t M, int index, size_t *row0, size_t *rows) {
    partition_slab(M, mg->n, index, row0, rows);
}

int b200_partition_slab(size_t M, int n, int index, size_t *row0, size_t *rows) {
    if (!row0 || !rows || n < 1 || index < 0 || index >= n) return B200_HGEMM_ERR_INVALID_ARG;
    partition_slab(M, n, index, row0, rows);
    return B200_HGEMM_OK;
}

int b200_mg_create(const int *devices, int n, b200_mg **out) {
    if (!devices || !out || n < 1 || n > kMaxDevices) return B200_HGEMM_ERR_INVALID_ARG;
    // A process that sets out to drive several GPUs never runs the kernels with multicast loads;
    // the switch is locked before anything else can fail.
    if (n >= 2) mc_lock_off();
    int count = 0;
    if (!cuda_ok(cudaGetDeviceCount(&count), "cudaGetDeviceCount")) return B200_HGEMM_ERR_CUDA;
    for (int i = 0; i < n; ++i) {
        if (devices[i] < 0 || devices[i] >= count) return B200_HGEMM_ERR_INVALID_ARG;
        for (int j = 0; j < i; ++j) {
            if (devices[j] == devices[i]) return B200_HGEMM_ERR_INVALID_ARG;
        }
    }
    DeviceRestore restore;
    b200_mg *mg = new b200_mg();
    mg->n = n;
    int rc = B200_HGEMM_OK;
    for (int i = 0; i < n && rc == B200_HGEMM_OK; ++i) {
        mg->devices[i] = devices[i];
        DeviceState *st = nullptr;
        if (!cuda_ok(cudaSetDevice(devices[i]), "cudaSetDevice")) {
            rc = B200_HGEMM_ERR_CUDA;
        } else if ((rc = current_state(&st)) == B200_HGEMM_OK && !st->sm100) {
            rc = B200_HGEMM_ERR_NO_SM100;
        } else if (rc == B200_HGEMM_OK &&
                   (cudaStreamCreateWithFlags(&mg->streams[i], cudaStreamNonBlocking) != cudaSuccess ||
                    cudaEventCreate(&mg->start[i]) != cudaSuccess || cudaEventCreate(&mg->stop[i]) != cudaSuccess)) {
            rc = B200_HGEMM_ERR_CUDA;
        }
    }
    if (rc != B200_HGEMM_OK) {
        b200_mg_destroy(mg);
        return rc;
    }
    *out = mg;
    return B200_HGEMM_OK;
}

int b200_mg_destroy(b200_mg *mg) {
    if (!mg) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceRestore restore;
    for (int i = 0; i < mg->n; ++i) {
        if (cudaSetDevice(mg->devices[i]) != cudaSuccess) continue;
        if (mg->streams[i]) {
            cudaStreamSynchronize(mg->streams[i]);
            cudaStreamDestroy(mg->streams[i]);
        }
        if (mg->start[i]) cudaEventDestroy(mg->start[i]);
        if (mg->stop[i]) cudaEventDestroy(mg->stop[i]);
    }
    cudaGetLastError();
    delete mg;
    return B200_HGEMM_OK;
}

int b200_mg_device_count(const b200_mg *mg) {
    return mg ? mg->n : B200_HGEMM_ERR_INVALID_ARG;
}

int b200_mg_slab(const b200_mg *mg, size_t M, int index, size_t *row0, size_t *rows) {
    if (!mg || !row0 || !rows || index < 0 || index >= mg->n) return B200_HGEMM_ERR_INVALID_ARG;
    mg_slab(mg, M, index, row0, rows);
    return B200_HGEMM_OK;
}

int b200_mg_hgemm(b200_mg *mg, const void *const *A_slabs, const void *const *B_replicas, void *const *C_slabs, size_t M,
                  size_t N, size_t K) {
    if (!mg || !A_slabs || !B_replicas || !C_slabs || M == 0 || N == 0 || K == 0) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceRestore restore;
    // check everything before anything is launched
    for (int i = 0; i < mg->n; ++i) {
        size_t row0 = 0, rows = 0;
        mg_slab(mg, M, i, &row0, &rows);
        if (rows == 0) continue;
        const int rc = check_args(A_slabs[i], B_replicas[i], C_slabs[i], rows, N, K);
        if (rc != B200_HGEMM_OK) return rc;
    }
    for (int i = 0; i < mg->n; ++i) {
        size_t row0 = 0, rows = 0;
        mg_slab(mg, M, i, &row0, &rows);
        mg->timed[i] = false;
        if (rows == 0) continue;
        if (!cuda_ok(cudaSetDevice(mg->devices[i]), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaEventRecord(mg->start[i], mg->streams[i]), "cudaEventRecord")) return B200_HGEMM_ERR_CUDA;
        const int rc = entry(A_slabs[i], B_replicas[i], C_slabs[i], rows, N, K, nullptr, -1, mg->streams[i]);
        if (rc != B200_HGEMM_OK) return rc;
        if (!cuda_ok(cudaEventRecord(mg->stop[i], mg->streams[i]), "cudaEventRecord")) return B200_HGEMM_ERR_CUDA;
        mg->timed[i] = true;
    }
    return B200_HGEMM_OK;
}

int b200_mg_gather_c(b200_mg *mg, void *const *C_slabs, void *const *C_full, size_t M, size_t N) {
    if (!mg || !C_slabs || !C_full || M == 0 || N == 0) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceRestore restore;
    for (int src = 0; src < mg->n; ++src) {
        size_t row0 = 0, rows = 0;
        mg_slab(mg, M, src, &row0, &rows);
        if (rows == 0) continue;
        if (!C_slabs[src]) return B200_HGEMM_ERR_INVALID_ARG;
        if (!cuda_ok(cudaSetDevice(mg->devices[src]), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        for (int dst = 0; dst < mg->n; ++dst) {
            if (!C_full[dst]) continue;
            char *to = static_cast<char *>(C_full[dst]) + row0 * N * sizeof(__half);
            // on the owner's stream, so the copy follows the multiply that produced the slab
            if (!cuda_ok(cudaMemcpyPeerAsync(to, mg->devices[dst], C_slabs[src], mg->devices[src], rows * N * sizeof(__half),
                                             mg->streams[src]),
                         "cudaMemcpyPeerAsync")) {
                return B200_HGEMM_ERR_CUDA;
            }
        }
    }
    return B200_HGEMM_OK;
}

int b200_mg_synchronize(b200_mg *mg) {
    if (!mg) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceRestore restore;
    for (int i = 0; i < mg->n; ++i) {
        if (!cuda_ok(cudaSetDevice(mg->devices[i]), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        if (!cuda_ok(cudaStreamSynchronize(mg->streams[i]), "cudaStreamSynchronize")) return B200_HGEMM_ERR_CUDA;
    }
    // a bounded wait that expired on any of the devices ends the call with an error (the word is cleared)
    bool gave_up = false;
    for (int i = 0; i < mg->n; ++i) {
        if (!cuda_ok(cudaSetDevice(mg->devices[i]), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        DeviceState *st = nullptr;
        int rc = current_state(&st);
        if (rc != B200_HGEMM_OK) return rc;
        uint32_t word = 0;
        rc = read_error_word(st->error_word, mg->streams[i], &word);
        if (rc != B200_HGEMM_OK) return rc;
        gave_up = gave_up || word != 0;
    }
    return gave_up ? B200_HGEMM_ERR_DEVICE_WAIT : B200_HGEMM_OK;
}

int b200_mg_elapsed_ms_max(b200_mg *mg, float *ms) {
    if (!mg || !ms) return B200_HGEMM_ERR_INVALID_ARG;
    DeviceRestore restore;
    float worst = 0.f;
    for (int i = 0; i < mg->n; ++i) {
        if (!mg->timed[i]) continue;
        if (!cuda_ok(cudaSetDevice(mg->devices[i]), "cudaSetDevice")) return B200_HGEMM_ERR_CUDA;
        float t = 0.f;
        if (!cuda_ok(cudaEventElapsedTime(&t, mg->start[i], mg->stop[i]), "cudaEventElapsedTime")) return B200_HGEMM_ERR_CUDA;
        if (t > worst) worst = t;
    }
    *ms = worst;
    return B200_HGEMM_OK;
}

// ---- host-side helpers for tests --------------------------------------------------------
void b200_sched_tile_coord(uint32_t tile, uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m, uint32_t *m_blk,
                           uint32_t *n_blk) {
    TileCoord c = tile_coord(tile, m_blocks, n_blocks, group_m);
    *m_blk = c.m_blk;
    *n_blk = c.n_blk;
}

void b200_sched_tile_coord_fast(uint32_t tile, uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m, uint32_t *m_blk,
                                uint32_t *n_blk) {
    const Raster r = make_raster(m_blocks, n_blocks, group_m);
    TileCoord c = tile_coord_fast(tile, r);
    *m_blk = c.m_blk;
    *n_blk = c.n_blk;
}

void b200_debug_cluster_capacity(int clusters) {
    g_debug_cluster_capacity.store(clusters > 0 ? clusters : 0, std::memory_order_relaxed);
}

uint32_t b200_debug_fast_div(uint32_t n, uint32_t d) {
    return fast_div(n, make_fast_div(d));
}

uint32_t b200_sched_segments(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t *out,
                             uint32_t cap) {
    SegmentWalker w(part, parts, tiles, k_blocks);
    Segment s;
    uint32_t n = 0;
    while (w.next(s)) {
        if (n < cap) {
            out[3 * n + 0] = s.tile;
            out[3 * n + 1] = s.kb0;
            out[3 * n + 2] = s.kb1;
        }
        ++n;
    }
    return n;
}

void b200_sched_contributors(uint32_t tile, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t *first,
                             uint32_t *last) {
    const uint64_t total = static_cast<uint64_t>(tiles) * k_blocks;
    const uint64_t u0 = static_cast<uint64_t>(tile) * k_blocks;
    *first = part_of_unit(u0, parts, total);
    *last = part_of_unit(u0 + k_blocks - 1, parts, total);
}

uint32_t b200_sched_partial_slot(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t tile) {
    return partial_slot(part, parts, tiles, k_blocks, tile);
}

int b200_debug_wait_expiry(uint32_t limit_ms, b200_stream_t stream) {
    if (limit_ms == 0 || limit_ms > 1000) return B200_HGEMM_ERR_INVALID_ARG;  // a second at most
    DeviceState *st = nullptr;
    int rc = current_state(&st);
    if (rc != B200_HGEMM_OK) return rc;
    if (!st->sm100) return B200_HGEMM_ERR_NO_SM100;
    wait_expiry_probe_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(st->error_word,
                                                                                   static_cast<uint64_t>(limit_ms) * 1000000ull);
    if (!cuda_ok(cudaGetLastError(), "wait_expiry_probe_kernel")) return B200_HGEMM_ERR_CUDA;
    return B200_HGEMM_OK;
}

int b200_debug_wait_expiry_static(uint32_t limit_ms, b200_stream_t stream) {
    if (limit_ms == 0 || limit_ms > 1000) return B200_HGEMM_ERR_INVALID_ARG;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_HGEMM_ERR_CUDA;
    StaticDevice sd;
    const int rc = static_device(dev, &sd);
    if (rc != B200_HGEMM_OK) return rc;
    if (!sd.sm100) return B200_HGEMM_ERR_NO_SM100;
    wait_expiry_probe_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<uint32_t *>(sd.scratch),
                                                                                   static_cast<uint64_t>(limit_ms) * 1000000ull);
    if (!cuda_ok(cudaGetLastError(), "wait_expiry_probe_kernel")) return B200_HGEMM_ERR_CUDA;
    return B200_HGEMM_OK;
}

uint32_t b200_debug_idesc(uint32_t m, uint32_t n) {
    return umma_idesc_f16_f32(m, n);
}

uint64_t b200_debug_smem_desc(uint32_t smem_addr) {
    return umma_smem_desc_sw128(smem_addr);
}

}  // extern "C"
