// Check macros of the benchmark driver. Same names and same convention as the reference's
// (src/common/common.h:20-65): a failed check logs and ends the process. The library behind
// the C ABI never exits; only this driver does.
#pragma once

#include <stdint.h>
#include <stdlib.h>

#include <algorithm>
#include <string>

#include "cublas_v2.h"
#include "cuda_fp16.h"
#include "cuda_runtime.h"
#include "logging.h"
#include "util.h"

namespace hgemm_check {

[[noreturn]] inline void die() {
    exit(EXIT_FAILURE);
}

inline void cuda(cudaError_t status, const char *file, int line, const char *func) {
    if (status == cudaSuccess) return;
    int runtime = 0, driver = 0;
    cudaRuntimeGetVersion(&runtime);
    cudaDriverGetVersion(&driver);
    ::hgemm_log::emit(file, line, func, "CUDA Runtime API error = %04d \"%s\", runtime version: %d, driver version: %d",
                      static_cast<int>(status), cudaGetErrorName(status), runtime, driver);
    die();
}

inline void cublas(cublasStatus_t status, const char *file, int line, const char *func) {
    if (status == CUBLAS_STATUS_SUCCESS) return;
    ::hgemm_log::emit(file, line, func, "CUBLAS API error = %04d, runtime version: %zu", static_cast<int>(status),
                      cublasGetCudartVersion());
    die();
}

}  // namespace hgemm_check

#define HGEMM_LIKELY(x) __builtin_expect(!!(x), 1)
#define HGEMM_UNLIKELY(x) __builtin_expect(!!(x), 0)

#define HGEMM_CHECK(cond)                      \
    do {                                       \
        if (HGEMM_UNLIKELY(!(cond))) {         \
            HLOG("Check failed: %s", #cond);   \
            ::hgemm_check::die();              \
        }                                      \
    } while (0)

#define HGEMM_CHECK_EQ(a, b) HGEMM_CHECK((a) == (b))
#define HGEMM_CHECK_NE(a, b) HGEMM_CHECK((a) != (b))
#define HGEMM_CHECK_LE(a, b) HGEMM_CHECK((a) <= (b))
#define HGEMM_CHECK_LT(a, b) HGEMM_CHECK((a) < (b))
#define HGEMM_CHECK_GE(a, b) HGEMM_CHECK((a) >= (b))
#define HGEMM_CHECK_GT(a, b) HGEMM_CHECK((a) > (b))

#define HGEMM_DISALLOW_COPY_AND_ASSIGN(TypeName) \
    TypeName(const TypeName &) = delete;         \
    TypeName &operator=(const TypeName &) = delete

#define HGEMM_CHECK_CUDART_ERROR(expr) ::hgemm_check::cuda((expr), __FILE__, __LINE__, __FUNCTION__)
#define HGEMM_CHECK_CUBLAS_ERROR(expr) ::hgemm_check::cublas((expr), __FILE__, __LINE__, __FUNCTION__)
