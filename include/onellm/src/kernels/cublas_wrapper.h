// Drop-in for src/kernels/cublas_wrapper.h + cublas_wrapper.cc of oneLLM (:14-69; Gemm :45-90,
// stridedBatchedGemm :92-147).  Keeps the class the examples and layer constructors pass around, but
// no cuBLAS call is made: both methods run the library's own kernel through
// onellm_gemm_strided_batched with the BLAS convention (column-major, C = alpha*op(A)*op(B) + beta*C).
// The handles are stored and otherwise unused; <cublas_v2.h> is needed for their types only.
#pragma once
#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "src/utils/macro.h"

class cublasWrapper {
private:
    cublasHandle_t cublas_handle_;
    cublasLtHandle_t cublaslt_handle_;
    int dtype_ = ONELLM_F32;
    cudaStream_t stream_ = nullptr;

public:
    cublasWrapper(cublasHandle_t cublas_handle, cublasLtHandle_t cublaslt_handle)
        : cublas_handle_(cublas_handle), cublaslt_handle_(cublaslt_handle)
    {
    }
    ~cublasWrapper() {}

    void setFP32GemmConfig() { dtype_ = ONELLM_F32; }
    void setFP16GemmConfig() { dtype_ = ONELLM_F16; }
    void setStream(cudaStream_t stream) { stream_ = stream; }  // addition; default: legacy stream

    void Gemm(cublasOperation_t transa, cublasOperation_t transb, const int m, const int n, const int k, const void* A,
              const int lda, const void* B, const int ldb, void* C, const int ldc, float alpha = 1.0f, float beta = 0.0f)
    {
        stridedBatchedGemm(transa, transb, m, n, k, A, lda, 0, B, ldb, 0, C, ldc, 0, 1, alpha, beta);
    }

    void stridedBatchedGemm(cublasOperation_t transa, cublasOperation_t transb, const int m, const int n, const int k,
                            const void* A, const int lda, const int64_t strideA, const void* B, const int ldb,
                            const int64_t strideB, void* C, const int ldc, const int64_t strideC, const int batchCount,
                            float f_alpha = 1.0f, float f_beta = 0.0f)
    {
        ONELLM_B200_CALL(onellm_gemm_strided_batched(dtype_, transa != CUBLAS_OP_N, transb != CUBLAS_OP_N, m, n, k, A, lda,
                                                     (long)strideA, B, ldb, (long)strideB, C, ldc, (long)strideC, batchCount,
                                                     f_alpha, f_beta, stream_));
    }
};
