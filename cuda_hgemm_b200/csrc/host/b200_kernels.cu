// Entry points of the new kernels in the reference's calling convention
// `void name(half *A, half *B, half *C, size_t M, size_t N, size_t K)` (reference
// src/main.cu:11): thin wrappers over the C ABI on the default stream. The reference's
// kernels return void and end the process when their set-up fails
// (src/mma/mma_async_stage4.cu:619-635); these keep that convention by checking the status.
#include "b200_hgemm.h"
#include "common.h"

#define B200_WRAP(name, call)                                                                          \
    void name(half *A, half *B, half *C, size_t M, size_t N, size_t K) {                               \
        const int status = call(A, B, C, M, N, K, nullptr);                                            \
        if (HGEMM_UNLIKELY(status != B200_HGEMM_OK)) {                                                 \
            HLOG(#call " failed: %d (%s)", status, b200_hgemm_status_string(status));                  \
            exit(EXIT_FAILURE);                                                                        \
        }                                                                                              \
    }

B200_WRAP(b200Hgemm, b200_hgemm)
B200_WRAP(b200HgemmCta1, b200_hgemm_cta1)
B200_WRAP(b200HgemmCta2, b200_hgemm_cta2)
B200_WRAP(b200HgemmSplitK, b200_hgemm_splitk)
B200_WRAP(b200HgemmStreamK, b200_hgemm_streamk)
B200_WRAP(b200HgemmSimt, b200_hgemm_simt)
