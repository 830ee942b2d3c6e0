// Event-pair timer on one stream (reference src/common/cuda_timer.h:11-52): start() records,
// end() records, waits for the second event and returns the milliseconds between the two.
#pragma once

#include "common.h"

class CudaTimer {
public:
    explicit CudaTimer(cudaStream_t stream = nullptr) : m_stream(stream) {
        HGEMM_CHECK_CUDART_ERROR(cudaEventCreate(&m_begin));
        HGEMM_CHECK_CUDART_ERROR(cudaEventCreate(&m_finish));
    }

    ~CudaTimer() {
        if (m_begin) cudaEventDestroy(m_begin);
        if (m_finish) cudaEventDestroy(m_finish);
    }

    void start() {
        HGEMM_CHECK_CUDART_ERROR(cudaEventRecord(m_begin, m_stream));
    }

    float end() {
        float ms = 0.f;
        HGEMM_CHECK_CUDART_ERROR(cudaEventRecord(m_finish, m_stream));
        HGEMM_CHECK_CUDART_ERROR(cudaEventSynchronize(m_finish));
        HGEMM_CHECK_CUDART_ERROR(cudaEventElapsedTime(&ms, m_begin, m_finish));
        return ms;
    }

private:
    cudaStream_t m_stream;
    cudaEvent_t m_begin = nullptr;
    cudaEvent_t m_finish = nullptr;

    HGEMM_DISALLOW_COPY_AND_ASSIGN(CudaTimer);
};
