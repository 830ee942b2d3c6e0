// cuBLAS comparison entries of the benchmark driver.
//
// cublasTensorOp issues exactly the call the reference makes (src/cublas_tensor_op.cu:17-25):
// C^T (N x M, column-major) = B^T * A with FP16 compute, so that row-major C falls out.
// cublasTensorOpFp32 is the same call with FP32 compute (alpha and beta then have to be
// float), which is the arithmetic the new kernels use; the ">= cuBLAS" target is judged
// against the faster of the two.
#include "common.h"

namespace {

cublasHandle_t tensor_op_handle() {
    static cublasHandle_t handle = [] {
        cublasHandle_t h = nullptr;
        HGEMM_CHECK_CUBLAS_ERROR(cublasCreate(&h));
        HGEMM_CHECK_CUBLAS_ERROR(cublasSetMathMode(h, CUBLAS_TENSOR_OP_MATH));
        return h;
    }();
    return handle;
}

cublasStatus_t gemm_fp16_compute(cudaStream_t stream, const half *A, const half *B, half *C, size_t M, size_t N, size_t K) {
    const half alpha = __float2half(1.0f), beta = __float2half(0.0f);
    cublasHandle_t h = tensor_op_handle();
    cublasStatus_t st = cublasSetStream(h, stream);
    if (st != CUBLAS_STATUS_SUCCESS) return st;
    return cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, static_cast<int>(N), static_cast<int>(M), static_cast<int>(K), &alpha,
                        B, CUDA_R_16F, static_cast<int>(K), A, CUDA_R_16F, static_cast<int>(K), &beta, C, CUDA_R_16F,
                        static_cast<int>(N), CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
}

cublasStatus_t gemm_fp32_compute(cudaStream_t stream, const half *A, const half *B, half *C, size_t M, size_t N, size_t K) {
    const float alpha = 1.0f, beta = 0.0f;
    cublasHandle_t h = tensor_op_handle();
    cublasStatus_t st = cublasSetStream(h, stream);
    if (st != CUBLAS_STATUS_SUCCESS) return st;
    return cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, static_cast<int>(N), static_cast<int>(M), static_cast<int>(K), &alpha,
                        B, CUDA_R_16F, static_cast<int>(K), A, CUDA_R_16F, static_cast<int>(K), &beta, C, CUDA_R_16F,
                        static_cast<int>(N), CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
}

}  // namespace

#ifdef HGEMM_COMPARE_C_ABI
// The same two calls behind a C ABI for the Python benchmark (0 on success, the cuBLAS status otherwise).
extern "C" int hgemm_compare_cublas_fp16(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                                         void *stream) {
    return static_cast<int>(gemm_fp16_compute(static_cast<cudaStream_t>(stream), static_cast<const half *>(A),
                                              static_cast<const half *>(B), static_cast<half *>(C), M, N, K));
}

extern "C" int hgemm_compare_cublas_fp32(const void *A, const void *B, void *C, size_t M, size_t N, size_t K,
                                         void *stream) {
    return static_cast<int>(gemm_fp32_compute(static_cast<cudaStream_t>(stream), static_cast<const half *>(A),
                                              static_cast<const half *>(B), static_cast<half *>(C), M, N, K));
}

// Times `iters` back-to-back calls of any GEMM entry point of the C-ABI shape after `warmup`
// calls, between two events on `stream`: the reference driver's protocol
// (src/common/tester.h:59-64,89-95) without an interpreter in the loop. Returns mean
// milliseconds per call, or a negative value when a call or a CUDA function failed.
typedef int (*hgemm_entry_fn)(const void *, const void *, void *, size_t, size_t, size_t, void *);

extern "C" double hgemm_compare_time_loop(hgemm_entry_fn fn, const void *A, const void *B, void *C, size_t M, size_t N,
                                          size_t K, int warmup, int iters, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1.0;
    double result = -1.0;
    bool ok = true;
    for (int i = 0; i < warmup && ok; ++i) ok = fn(A, B, C, M, N, K, stream) == 0;
    ok = ok && cudaEventRecord(e0, s) == cudaSuccess;
    for (int i = 0; i < iters && ok; ++i) ok = fn(A, B, C, M, N, K, stream) == 0;
    ok = ok && cudaEventRecord(e1, s) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
    float ms = 0.f;
    if (ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && iters > 0) result = static_cast<double>(ms) / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return result;
}

// The same with the B operand taken in turn from `n_b` buffers (call i uses Bs[i % n_b]): for shapes
// whose B would otherwise be served from L2 on every call after the first (the decode shapes: B is
// about as large as L2). `warmup` calls run first, untimed.
extern "C" double hgemm_compare_time_loop_rotate(hgemm_entry_fn fn, const void *A, const void *const *Bs, int n_b, void *C,
                                                 size_t M, size_t N, size_t K, int warmup, int iters, void *stream) {
    if (n_b < 1) return -1.0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1.0;
    double result = -1.0;
    bool ok = true;
    int turn = 0;
    for (int i = 0; i < warmup && ok; ++i, ++turn) ok = fn(A, Bs[turn % n_b], C, M, N, K, stream) == 0;
    ok = ok && cudaEventRecord(e0, s) == cudaSuccess;
    for (int i = 0; i < iters && ok; ++i, ++turn) ok = fn(A, Bs[turn % n_b], C, M, N, K, stream) == 0;
    ok = ok && cudaEventRecord(e1, s) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
    float ms = 0.f;
    if (ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && iters > 0) result = static_cast<double>(ms) / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return result;
}
#else
void cublasTensorOp(half *A, half *B, half *C, size_t M, size_t N, size_t K) {
    HGEMM_CHECK_CUBLAS_ERROR(gemm_fp16_compute(nullptr, A, B, C, M, N, K));
}

void cublasTensorOpFp32(half *A, half *B, half *C, size_t M, size_t N, size_t K) {
    HGEMM_CHECK_CUBLAS_ERROR(gemm_fp32_compute(nullptr, A, B, C, M, N, K));
}
#endif
