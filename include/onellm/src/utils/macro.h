// Drop-in for src/utils/macro.h of oneLLM: CHECK (:6-20), CHECK_CUBLAS (:63-72),
// DeviceSyncAndCheckCudaError (:74-84), ONELLM_CHECK / ONELLM_CHECK_WITH_INFO (:86-106), plus
// ONELLM_B200_CALL, which turns a status of the onellm_b200 C ABI into the std::runtime_error the
// reference's callers expect from a failed launch.
#pragma once
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "onellm_b200.h"

#ifndef CHECK
#define CHECK(call)                                                                                     \
    do {                                                                                                \
        const cudaError_t onellm_check_rc = (call);                                                     \
        if (onellm_check_rc != cudaSuccess) {                                                           \
            std::printf("CUDA Error:\n    File:       %s\n    Line:       %d\n    Error code: %d\n"      \
                        "    Error text: %s\n",                                                         \
                        __FILE__, __LINE__, (int)onellm_check_rc, cudaGetErrorString(onellm_check_rc)); \
            std::exit(1);                                                                               \
        }                                                                                               \
    } while (0)
#endif

inline const char* _cudaGetErrorEnum(cudaError_t e) { return cudaGetErrorString(e); }

inline const char* _cudaGetErrorEnum(cublasStatus_t e)
{
    static const struct { cublasStatus_t code; const char* name; } names[] = {
        {CUBLAS_STATUS_SUCCESS, "CUBLAS_STATUS_SUCCESS"},
        {CUBLAS_STATUS_NOT_INITIALIZED, "CUBLAS_STATUS_NOT_INITIALIZED"},
        {CUBLAS_STATUS_ALLOC_FAILED, "CUBLAS_STATUS_ALLOC_FAILED"},
        {CUBLAS_STATUS_INVALID_VALUE, "CUBLAS_STATUS_INVALID_VALUE"},
        {CUBLAS_STATUS_ARCH_MISMATCH, "CUBLAS_STATUS_ARCH_MISMATCH"},
        {CUBLAS_STATUS_MAPPING_ERROR, "CUBLAS_STATUS_MAPPING_ERROR"},
        {CUBLAS_STATUS_EXECUTION_FAILED, "CUBLAS_STATUS_EXECUTION_FAILED"},
        {CUBLAS_STATUS_INTERNAL_ERROR, "CUBLAS_STATUS_INTERNAL_ERROR"},
        {CUBLAS_STATUS_NOT_SUPPORTED, "CUBLAS_STATUS_NOT_SUPPORTED"},
        {CUBLAS_STATUS_LICENSE_ERROR, "CUBLAS_STATUS_LICENSE_ERROR"},
    };
    for (const auto& n : names)
        if (n.code == e) return n.name;
    return "<unknown>";
}

inline std::string onellm_where(const char* file, int line) { return std::string(file) + ":" + std::to_string(line) + " \n"; }

template <typename T>
void check(T result, char const* const /*func*/, const char* const file, int const line)
{
    if (result) throw std::runtime_error(std::string("[TM][ERROR] CUDA runtime error: ") + _cudaGetErrorEnum(result) + " " + onellm_where(file, line));
}
#define CHECK_CUBLAS(val) check((val), #val, __FILE__, __LINE__)

inline void syncAndCheck(const char* const file, int const line)
{
    const cudaError_t sync_rc = cudaDeviceSynchronize();
    const cudaError_t last_rc = cudaGetLastError();
    const cudaError_t rc = sync_rc != cudaSuccess ? sync_rc : last_rc;
    if (rc != cudaSuccess)
        throw std::runtime_error(std::string("[TM][ERROR] CUDA runtime error: ") + cudaGetErrorString(rc) + " " + onellm_where(file, line));
}
#define DeviceSyncAndCheckCudaError() syncAndCheck(__FILE__, __LINE__)

[[noreturn]] inline void throwRuntimeError(const char* const file, int const line, std::string const& info = "")
{
    throw std::runtime_error("[oneLLM][ERROR] " + info + " Assertion fail: " + onellm_where(file, line));
}

inline void onellmAssert(bool result, const char* const file, int const line, std::string const& info = "")
{
    if (!result) throwRuntimeError(file, line, info);
}

#define ONELLM_CHECK(val) onellmAssert((val), __FILE__, __LINE__)
#define ONELLM_CHECK_WITH_INFO(val, info)                             \
    do {                                                              \
        if (!(val)) onellmAssert(false, __FILE__, __LINE__, (info));  \
    } while (0)

// status of an onellm_b200 entry point -> exception carrying the library's message
inline void onellm_b200_call(int status, const char* what, const char* file, int line)
{
    if (status != ONELLM_OK)
        throw std::runtime_error(std::string("[oneLLM][ERROR] ") + what + ": " + onellm_last_error() + " " + onellm_where(file, line));
}
#define ONELLM_B200_CALL(expr) onellm_b200_call((expr), #expr, __FILE__, __LINE__)
