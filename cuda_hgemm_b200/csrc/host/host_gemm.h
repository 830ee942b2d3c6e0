// Host-side FP32-accumulate GEMM of the benchmark driver: the checker behind -enable_check
// and the reported CPU baseline. The reference links OpenMP and has a -cpu_procs flag but no
// host GEMM (src/main.cu:44,50); its check compares against cuBLAS instead
// (src/common/tester.h:41-47). The GEMM library never calls this code: it has no CPU path.
//
//   ref[i][j] = sum_k float(A[i*K + k]) * float(B[j*K + k])     (layouts: src/simt_naive.cu:18-24)
#pragma once

#include <math.h>
#include <omp.h>

#include <vector>

#include "common.h"

namespace host_gemm {

// Rows [row0, row0 + rows) of the product into `out` (rows x N, FP32). Returns seconds spent
// in the multiply itself (FP16 -> FP32 conversion of the operands excluded).
inline double rows_f32(const half *A, const half *B, float *out, size_t N, size_t K, size_t row0, size_t rows,
                       int threads) {
    if (threads < 1) threads = 1;
    std::vector<float> af(rows * K), bf(N * K);
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long long i = 0; i < static_cast<long long>(rows * K); ++i) af[i] = __half2float(A[row0 * K + i]);
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long long i = 0; i < static_cast<long long>(N * K); ++i) bf[i] = __half2float(B[i]);

    const double t0 = omp_get_wtime();
    const long long row_blocks = static_cast<long long>(div_ceil(rows, 8));
    const long long col_blocks = static_cast<long long>(div_ceil(N, 64));
#pragma omp parallel for num_threads(threads) collapse(2) schedule(dynamic, 4)
    for (long long rb = 0; rb < row_blocks; ++rb) {
        for (long long cb = 0; cb < col_blocks; ++cb) {
            const size_t i_end = std::min(rows, static_cast<size_t>(rb + 1) * 8);
            const size_t j_end = std::min(N, static_cast<size_t>(cb + 1) * 64);
            for (size_t j = static_cast<size_t>(cb) * 64; j < j_end; ++j) {
                const float *b = &bf[j * K];
                for (size_t i = static_cast<size_t>(rb) * 8; i < i_end; ++i) {
                    const float *a = &af[i * K];
                    float acc = 0.f;
#pragma omp simd reduction(+ : acc)
                    for (size_t k = 0; k < K; ++k) acc += a[k] * b[k];
                    out[i * N + j] = acc;
                }
            }
        }
    }
    return omp_get_wtime() - t0;
}

struct Report {
    double max_abs = 0, avg_abs = 0, max_ref = 0, rms_ref = 0, max_rel = 0;
    size_t violations = 0, non_finite = 0, count = 0;
    bool pass(double rtol) const {
        return non_finite == 0 && violations == 0 && max_rel <= rtol;
    }
};

// Difference of FP16 results against the FP32 reference over `count` elements:
// max/mean absolute difference (the reference's two numbers, src/common/matrix.h:102-113),
// max-norm relative error, and the count of elements outside rtol*|ref| + rtol*rms(ref).
inline Report compare(const half *c, const float *ref, size_t count, double rtol, int threads) {
    Report r;
    r.count = count;
    double max_abs = 0, sum_abs = 0, max_ref = 0, sum_sq = 0;
    long long non_finite = 0;
#pragma omp parallel for num_threads(threads) schedule(static) reduction(max : max_abs, max_ref) \
    reduction(+ : sum_abs, sum_sq, non_finite)
    for (long long i = 0; i < static_cast<long long>(count); ++i) {
        const double v = __half2float(c[i]), t = ref[i];
        if (!std::isfinite(v)) {
            ++non_finite;
            continue;
        }
        const double d = fabs(v - t);
        max_abs = std::max(max_abs, d);
        max_ref = std::max(max_ref, fabs(t));
        sum_abs += d;
        sum_sq += t * t;
    }
    const double rms = sqrt(sum_sq / static_cast<double>(count ? count : 1));
    long long violations = 0;
#pragma omp parallel for num_threads(threads) schedule(static) reduction(+ : violations)
    for (long long i = 0; i < static_cast<long long>(count); ++i) {
        const double v = __half2float(c[i]), t = ref[i];
        if (std::isfinite(v) && fabs(v - t) > rtol * fabs(t) + rtol * rms) ++violations;
    }
    r.max_abs = max_abs;
    r.avg_abs = sum_abs / static_cast<double>(count ? count : 1);
    r.max_ref = max_ref;
    r.rms_ref = rms;
    r.max_rel = max_ref > 0 ? max_abs / max_ref : (max_abs > 0 ? INFINITY : 0);
    r.violations = static_cast<size_t>(violations);
    r.non_finite = static_cast<size_t>(non_finite);
    return r;
}

}  // namespace host_gemm
