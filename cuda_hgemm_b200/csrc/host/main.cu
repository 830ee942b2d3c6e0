// hgemm: the benchmark driver. Same flags, same flow and same log format as the reference's
// executable (src/main.cu:35-131): parse flags, pick the GPU, build a Tester, evaluate cuBLAS
// first (it defines the 100 % column), then the reference's own kernels when their library is
// given, then the sm_100a kernels of this repository.
#include <dlfcn.h>
#include <omp.h>

#include <functional>

#include "b200_hgemm.h"
#include "flags.h"
#include "tester.h"

#define HGEMM_FUNC(name) void name(half *A, half *B, half *C, size_t M, size_t N, size_t K)

HGEMM_FUNC(cublasTensorOp);
HGEMM_FUNC(cublasTensorOpFp32);

HGEMM_FUNC(b200Hgemm);
HGEMM_FUNC(b200HgemmCta1);
HGEMM_FUNC(b200HgemmCta2);
HGEMM_FUNC(b200HgemmSplitK);
HGEMM_FUNC(b200HgemmStreamK);
HGEMM_FUNC(b200HgemmSimt);

// the reference's flags, names and defaults unchanged (src/main.cu:35-45)
DEFINE_uint32(M, 512, "M");
DEFINE_uint32(N, 2048, "N");
DEFINE_uint32(K, 1024, "K");
DEFINE_bool(enable_wmma, true, "test the reference's WMMA API kernels (needs -ref_lib)");
DEFINE_bool(enable_mma, true, "test the reference's MMA PTX kernels (needs -ref_lib)");
DEFINE_uint32(warmup_iterations, 1, "warmup iteration numbers and average the result");
DEFINE_uint32(profiling_iterations, 10, "profiling iteration numbers and average the result");
DEFINE_uint32(sleep_duration, 100, "sleep_milliseconds between profiling");
DEFINE_bool(enable_check, false, "check the GPU result against an FP32-accumulate host GEMM");
DEFINE_uint32(cpu_procs, static_cast<uint32_t>(omp_get_num_procs()), "processor num used of CPU");
DEFINE_uint32(gpu_rank, 0, "the used GPU rank");
// additions
DEFINE_bool(enable_b200, true, "test the sm_100a tcgen05 kernels");
DEFINE_bool(enable_variants, true, "also test each fixed variant (1-CTA, 2-CTA, split-k, stream-k), not only auto dispatch");
DEFINE_bool(enable_naive, false, "also test the naive kernels (reference Simt/Wmma/Mma-Naive and the FP32 CUDA-core kernel)");
DEFINE_string(ref_lib, "", "shared library built from the reference's kernel sources; empty = skip them");
DEFINE_uint64(seed, 2023, "seed of the input matrices");
DEFINE_string(dist, "uniform", "input distribution: uniform ([-1,1)) or normal (A ~ N(0,1), B ~ N(0,1/K))");
DEFINE_uint32(check_rows, 512, "rows of C checked against the host GEMM when M is larger (0 = all rows)");
DEFINE_uint32(l2_rotate, 1, "distinct B buffers cycled through the timed loop so that B is not served from L2");
DEFINE_string(json, "", "append one JSON line per evaluated kernel to this file");
DEFINE_bool(enable_multicast, false, "let the auto dispatch use the kernels with multicast operand loads (this process owns one GPU)");

namespace {

typedef void (*HgemmFn)(half *, half *, half *, size_t, size_t, size_t);

// Itanium-mangled `void name(half*, half*, half*, size_t, size_t, size_t)`: the reference declares
// its kernels with C++ linkage.
std::string mangled_entry(const std::string &name) {
    return "_Z" + std::to_string(name.size()) + name + "P6__halfS0_S0_mmm";
}

struct RefKernel {
    const char *symbol;
    const char *log_name;
    bool wmma;
    bool naive;
    size_t m_align, n_align, k_align, k_min;  // shape limits of the kernel (it has no edge guards)
};

// evaluation order and log names of the reference driver (src/main.cu:100-123)
const RefKernel kRefKernels[] = {
    {"simtNaive", "Simt-Naive", false, true, 16, 16, 1, 1},
    {"wmmaNaive", "Wmma-Naive", true, true, 16, 16, 16, 16},
    {"wmmaPadding", "Wmma-Padding", true, false, 256, 128, 32, 32},
    {"wmmaAsync", "Wmma-Async", true, false, 256, 128, 32, 32},
    {"wmmaAsyncPg2s", "Wmma-Async-Pg2s", true, false, 256, 128, 32, 64},
    {"wmmaAsyncPg2sPs2r", "Wmma-Async-Pg2s-Ps2r", true, false, 256, 128, 32, 64},
    {"wmmaAsyncStage2", "Wmma-Async-Stage2", true, false, 256, 128, 32, 64},
    {"wmmaAsyncStage3", "Wmma-Async-Stage3", true, false, 256, 128, 32, 96},
    {"mmaNaive", "Mma-Naive", false, true, 16, 8, 16, 16},
    {"mmaPermuted", "Mma-Permuted", false, false, 256, 128, 32, 32},
    {"mmaAsync", "Mma-Async", false, false, 256, 128, 32, 32},
    {"mmaAsyncPg2s", "Mma-Async-Pg2s", false, false, 256, 128, 32, 64},
    {"mmaAsyncPg2sPs2r", "Mma-Async-Pg2s-Ps2r", false, false, 256, 128, 32, 64},
    {"mmaAsyncStage2", "Mma-Async-Stage2", false, false, 256, 128, 32, 64},
    {"mmaAsyncStage3", "Mma-Async-Stage3", false, false, 256, 128, 32, 96},
    {"mmaAsyncStage4", "Mma-Async-Stage4", false, false, 256, 128, 32, 128},
};

void log_device(const cudaDeviceProp &prop) {
    int driver = 0, runtime = 0;
    HGEMM_CHECK_CUDART_ERROR(cudaDriverGetVersion(&driver));
    HGEMM_CHECK_CUDART_ERROR(cudaRuntimeGetVersion(&runtime));
    HLOG("CUDA driver version / runtime version: %d.%d / %d.%d", driver / 1000, (driver % 100) / 10, runtime / 1000,
         (runtime % 100) / 10);
    HLOG("CUDA capability major/minor version number: %d.%d (%s)", prop.major, prop.minor,
         convert_SM_to_arch_name(prop.major, prop.minor));
    const int cores = convert_SM_to_cores(prop.major, prop.minor);
    HLOG("%d multiprocessors, %d CUDA cores/MP: %d CUDA cores", prop.multiProcessorCount, cores,
         cores * prop.multiProcessorCount);
    HLOG("Total amount of global memory: %.0f MBytes (%zu Bytes)", static_cast<double>(prop.totalGlobalMem) / 1048576,
         prop.totalGlobalMem);
    HLOG("Total shared memory per multiprocessor: %.0f KBytes (%zu Bytes)",
         static_cast<double>(prop.sharedMemPerMultiprocessor) / 1024, prop.sharedMemPerMultiprocessor);
    HLOG("L2 cache size: %.0f KBytes (%d Bytes)", static_cast<double>(prop.l2CacheSize) / 1024, prop.l2CacheSize);
    HLOG("Memory bus width: %d-bit", prop.memoryBusWidth);
}

}  // namespace

int main(int argc, char *argv[]) {
    GFLAGS_NAMESPACE::ParseCommandLineFlags(&argc, &argv, true);

    omp_set_num_threads(static_cast<int>(FLAGS_cpu_procs));
    HGEMM_CHECK_CUDART_ERROR(cudaSetDevice(static_cast<int>(FLAGS_gpu_rank)));

    cudaDeviceProp dev_prop;
    HGEMM_CHECK_CUDART_ERROR(cudaGetDeviceProperties(&dev_prop, static_cast<int>(FLAGS_gpu_rank)));
    HLOG("CUDA HGEMM start with %u CPU processes on the %u-th GPU: %s", FLAGS_cpu_procs, FLAGS_gpu_rank, dev_prop.name);
    log_device(dev_prop);
    HLOG("%s", b200_hgemm_version());

    HLOG("A (%u x %u) * B (%u x %u) = C (%u x %u)", FLAGS_M, FLAGS_K, FLAGS_K, FLAGS_N, FLAGS_M, FLAGS_N);
    HLOG("Profiling: enable wmma: %d, enable mma: %d, warmup iterations: %u, profiling iterations: %u, sleep duration: "
         "%u ms, enable check: %d",
         FLAGS_enable_wmma, FLAGS_enable_mma, FLAGS_warmup_iterations, FLAGS_profiling_iterations, FLAGS_sleep_duration,
         FLAGS_enable_check);
    HGEMM_CHECK(FLAGS_dist == "uniform" || FLAGS_dist == "normal");

    TesterOptions opt;
    opt.seed = FLAGS_seed;
    opt.normal_inputs = (FLAGS_dist == "normal");
    opt.check_rows = FLAGS_check_rows;
    opt.cpu_procs = static_cast<int>(FLAGS_cpu_procs);
    opt.json_path = FLAGS_json;
    opt.l2_rotate = FLAGS_l2_rotate;
    Tester tester(FLAGS_M, FLAGS_N, FLAGS_K, FLAGS_warmup_iterations, FLAGS_profiling_iterations, FLAGS_sleep_duration,
                  FLAGS_enable_check, opt);

    tester.evaluate(cublasTensorOp, "Cublas-Tensor-Op", false);
    tester.evaluate(cublasTensorOpFp32, "Cublas-Tensor-Op-Fp32", false);

    // the reference's kernels, compiled unmodified from its sources into a shared library
    if (!FLAGS_ref_lib.empty() && (FLAGS_enable_wmma || FLAGS_enable_mma)) {
        void *handle = dlopen(FLAGS_ref_lib.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!handle) {
            HLOG("cannot load reference kernels from %s: %s", FLAGS_ref_lib.c_str(), dlerror());
            return EXIT_FAILURE;
        }
        for (const RefKernel &k : kRefKernels) {
            const bool family_on = (k.symbol[0] == 's') ? true : (k.wmma ? FLAGS_enable_wmma : FLAGS_enable_mma);
            if (!family_on || (k.naive && !FLAGS_enable_naive)) continue;
            if (FLAGS_M % k.m_align || FLAGS_N % k.n_align || FLAGS_K % k.k_align || FLAGS_K < k.k_min) {
                HLOG("%s skipped: it has no edge handling and needs M %% %zu == N %% %zu == K %% %zu == 0, K >= %zu",
                     k.log_name, k.m_align, k.n_align, k.k_align, k.k_min);
                continue;
            }
            HgemmFn fn = reinterpret_cast<HgemmFn>(dlsym(handle, mangled_entry(k.symbol).c_str()));
            if (!fn) {
                HLOG("%s not found in %s", k.symbol, FLAGS_ref_lib.c_str());
                continue;
            }
            tester.evaluate(fn, k.log_name, false);
        }
    }

    if (FLAGS_enable_b200) {
        if (FLAGS_enable_multicast && b200_hgemm_enable_multicast(1) != B200_HGEMM_OK) {
            HLOG("multicast kernels not available (companion library absent, or this process is one rank of several)");
        }
        tester.evaluate(b200Hgemm, "B200-Tcgen05-Auto");
        if (FLAGS_enable_variants && FLAGS_K % 8 == 0) {
            tester.evaluate(b200HgemmCta1, "B200-Tcgen05-1Cta");
            tester.evaluate(b200HgemmCta2, "B200-Tcgen05-2Cta");
            tester.evaluate(b200HgemmSplitK, "B200-Tcgen05-SplitK");
            tester.evaluate(b200HgemmStreamK, "B200-Tcgen05-StreamK");
        }
        if (FLAGS_enable_naive) tester.evaluate(b200HgemmSimt, "B200-Simt-Fp32Acc-Naive");
        const int dev_err = b200_hgemm_last_device_error();
        if (dev_err != 0) {
            HLOG("device-side error word: %d", dev_err);
            return EXIT_FAILURE;
        }
    }

    GFLAGS_NAMESPACE::ShutDownCommandLineFlags();

    if (FLAGS_enable_check && !tester.allPassed()) {
        HLOG("Done: at least one checked kernel is outside tolerance");
        return 2;
    }
    HLOG("Done");
    return 0;
}
