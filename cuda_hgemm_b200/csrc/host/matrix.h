// Host + device FP16 buffer of the benchmark driver.
//
// Same public face as the reference's Matrix (src/common/matrix.h:13-132: rows/cols/element
// count, host and device pointers, tearUp, moveToHost/moveToDevice, memSetHost/memSetDevice,
// checkValue), with these differences:
//   * the fill is SEEDED and counter-based -- element i of stream s under seed S is a pure
//     function of (S, s, i) -- so runs are reproducible and the fill parallelises over host
//     threads with a result that does not depend on their number (the reference draws from an
//     unseeded std::random_device in one serial loop, matrix.h:28-33);
//   * uniform[min, max) as in the reference, or normal(0, sigma) for the decode/prefill shapes;
//   * poisonDevice() fills C with FP16 NaNs so that an element a kernel never wrote is caught
//     (the reference pre-fills C with whatever `base` holds, tester.h:56);
//   * checkAgainst() compares with an FP32 host reference and returns a verdict, where
//     checkValue() only logs two numbers (matrix.h:97-114).
#pragma once

#include <math.h>
#include <omp.h>
#include <string.h>

#include <string>

#include "common.h"
#include "host_gemm.h"

namespace hgemm_rng {

// splitmix64 finaliser: a bijective 64-bit mix.
inline uint64_t mix(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline uint64_t draw(uint64_t seed, uint64_t stream, uint64_t index) {
    return mix(mix(seed ^ (stream * 0xD1B54A32D192ED03ull)) + index);
}

// 24 random bits -> [0, 1)
inline float unit(uint64_t bits) {
    return static_cast<float>(bits >> 40) * (1.0f / 16777216.0f);
}

inline float uniform(uint64_t seed, uint64_t stream, uint64_t index, float lo, float hi) {
    return lo + (hi - lo) * unit(draw(seed, stream, index));
}

// Box-Muller on two independent draws.
inline float normal(uint64_t seed, uint64_t stream, uint64_t index, float sigma) {
    const uint64_t bits = draw(seed, stream, index);
    const float u1 = (static_cast<float>(bits >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0, 1)
    const float u2 = static_cast<float>((bits >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    return sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

}  // namespace hgemm_rng

enum class MatrixFill { kUniform, kNormal, kNone };

class Matrix {
public:
    // `stream` separates the random sequences of different matrices under one seed.
    Matrix(size_t row, size_t col, const std::string &name = "Matrix", float min = -1.0f, float max = 1.0f,
           uint64_t seed = 2023, uint64_t stream = 0, MatrixFill fill = MatrixFill::kUniform, float sigma = 1.0f)
        : m_row(row), m_col(col), m_name(name), m_min(min), m_max(max) {
        HGEMM_CHECK_GT(m_row, 0);
        HGEMM_CHECK_GT(m_col, 0);
        m_elem_num = m_row * m_col;
        HGEMM_CHECK_EQ(m_elem_num / m_row, m_col);

        HGEMM_CHECK_CUDART_ERROR(cudaMallocHost(reinterpret_cast<void **>(&m_host_ptr), m_elem_num * sizeof(half)));
        HGEMM_CHECK_CUDART_ERROR(cudaMalloc(reinterpret_cast<void **>(&m_dev_ptr), m_elem_num * sizeof(half)));

        half *dst = m_host_ptr;
        const long long n = static_cast<long long>(m_elem_num);
        if (fill == MatrixFill::kUniform) {
#pragma omp parallel for schedule(static)
            for (long long i = 0; i < n; ++i) dst[i] = __float2half_rn(hgemm_rng::uniform(seed, stream, i, min, max));
        } else if (fill == MatrixFill::kNormal) {
#pragma omp parallel for schedule(static)
            for (long long i = 0; i < n; ++i) dst[i] = __float2half_rn(hgemm_rng::normal(seed, stream, i, sigma));
        } else {
            memset(dst, 0, m_elem_num * sizeof(half));
        }
        moveToDevice();
        HLOG("%s: %zu * %zu, cpu: %p, gpu: %p", m_name.c_str(), m_row, m_col, static_cast<void *>(m_host_ptr),
             static_cast<void *>(m_dev_ptr));
    }

    ~Matrix() {
        if (m_host_ptr) cudaFreeHost(m_host_ptr);
        if (m_dev_ptr) cudaFree(m_dev_ptr);
    }

    size_t getRow() const { return m_row; }
    size_t getCol() const { return m_col; }
    size_t getElemNum() const { return m_elem_num; }
    half *getHostPtr() const { return m_host_ptr; }
    half *getDevPtr() const { return m_dev_ptr; }

    // Device copy of another matrix of the same shape into this one.
    void tearUp(Matrix *base) {
        HGEMM_CHECK(base);
        HGEMM_CHECK_EQ(m_row, base->getRow());
        HGEMM_CHECK_EQ(m_col, base->getCol());
        HGEMM_CHECK_CUDART_ERROR(cudaMemcpy(m_dev_ptr, base->getDevPtr(), bytes(), cudaMemcpyDeviceToDevice));
    }

    void moveToHost() { HGEMM_CHECK_CUDART_ERROR(cudaMemcpy(m_host_ptr, m_dev_ptr, bytes(), cudaMemcpyDeviceToHost)); }
    void moveToDevice() { HGEMM_CHECK_CUDART_ERROR(cudaMemcpy(m_dev_ptr, m_host_ptr, bytes(), cudaMemcpyHostToDevice)); }
    void memSetHost() { memset(m_host_ptr, 0, bytes()); }
    void memSetDevice() { HGEMM_CHECK_CUDART_ERROR(cudaMemset(m_dev_ptr, 0, bytes())); }

    // Every element becomes the FP16 NaN 0x7E7E.
    void poisonDevice() { HGEMM_CHECK_CUDART_ERROR(cudaMemset(m_dev_ptr, 0x7E, bytes())); }

    // The reference's check: log max and mean absolute difference against another matrix's host copy.
    void checkValue(Matrix *base) {
        HGEMM_CHECK(base);
        HGEMM_CHECK_EQ(m_row, base->getRow());
        HGEMM_CHECK_EQ(m_col, base->getCol());
        const half *mine = m_host_ptr, *theirs = base->getHostPtr();
        double max_diff = 0.0, sum_diff = 0.0;
        const long long n = static_cast<long long>(m_elem_num);
#pragma omp parallel for schedule(static) reduction(max : max_diff) reduction(+ : sum_diff)
        for (long long i = 0; i < n; ++i) {
            const double d = fabs(static_cast<double>(__half2float(mine[i])) - static_cast<double>(__half2float(theirs[i])));
            max_diff = std::max(max_diff, d);
            sum_diff += d;
        }
        m_max_diff = max_diff;
        m_avg_diff = sum_diff / static_cast<double>(m_elem_num);
        HLOG("Max diff: %f, avg diff: %f", m_max_diff, m_avg_diff);
    }

    // Host copy, rows [row0, row0 + rows), against an FP32 reference of those rows.
    host_gemm::Report checkAgainst(const float *ref, size_t row0, size_t rows, double rtol, int threads) const {
        HGEMM_CHECK_LE(row0 + rows, m_row);
        return host_gemm::compare(m_host_ptr + row0 * m_col, ref, rows * m_col, rtol, threads);
    }

    double maxDiff() const { return m_max_diff; }
    double avgDiff() const { return m_avg_diff; }

private:
    size_t bytes() const { return m_elem_num * sizeof(half); }

    const size_t m_row;
    const size_t m_col;
    const std::string m_name;
    const float m_min;
    const float m_max;

    size_t m_elem_num = 0;
    half *m_host_ptr = nullptr;
    half *m_dev_ptr = nullptr;
    double m_max_diff = 0.0;
    double m_avg_diff = 0.0;

    HGEMM_DISALLOW_COPY_AND_ASSIGN(Matrix);
};
