// Drop-in for src/utils/cuda_utils.h + cuda_utils.cu of oneLLM: GPUMalloc (:3-8), GPUFree (:12-19),
// cudaH2Dcpy (:23-27), loadWeightFromBin (:47-108).  Header-only templates, so fp16 and fp32
// instantiate alike.  Differences from the reference loader: a file whose size is not exactly
// sizeof(T_IN) * elements is an error (the reference skips it without a word), the status is
// returned (0 ok, -1 failed), and T_IN != T converts on the host (float files into half weights).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <iostream>
#include <string>
#include <vector>

#include "src/utils/macro.h"

template <typename T>
void GPUMalloc(T** ptr, size_t size)
{
    CHECK(cudaMalloc(reinterpret_cast<void**>(ptr), sizeof(T) * size));
}

template <typename T>
void GPUFree(T*& ptr)
{
    if (ptr != nullptr) {
        CHECK(cudaFree(ptr));
        ptr = nullptr;
    }
}

template <typename T>
void cudaH2Dcpy(T* tgt, const T* src, const size_t size)
{
    CHECK(cudaMemcpy(tgt, src, sizeof(T) * size, cudaMemcpyHostToDevice));
}

template <typename T, typename T_IN>
int loadWeightFromBin(T* ptr, std::vector<size_t> shape, std::string filename)
{
    if (shape.empty() || shape.size() > 2) {
        std::fprintf(stderr, "[oneLLM] %s: weights have one or two dimensions\n", filename.c_str());
        return -1;
    }
    size_t count = 1;
    for (size_t d : shape) count *= d;
    if (count == 0) return 0;
    std::FILE* f = std::fopen(filename.c_str(), "rb");
    if (!f) {
        std::fprintf(stderr, "[oneLLM] cannot open weight file %s\n", filename.c_str());
        return -1;
    }
    std::fseek(f, 0, SEEK_END);
    const long bytes = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (bytes < 0 || static_cast<size_t>(bytes) != count * sizeof(T_IN)) {
        std::fprintf(stderr, "[oneLLM] %s holds %ld bytes, expected %zu\n", filename.c_str(), bytes, count * sizeof(T_IN));
        std::fclose(f);
        return -1;
    }
    std::vector<T_IN> host(count);
    const size_t got = std::fread(host.data(), sizeof(T_IN), count, f);
    std::fclose(f);
    if (got != count) return -1;
    if (std::is_same<T, T_IN>::value) {
        cudaH2Dcpy(ptr, reinterpret_cast<const T*>(host.data()), count);
    } else {
        std::vector<T> conv(count);
        for (size_t i = 0; i < count; i++) conv[i] = static_cast<T>(static_cast<float>(host[i]));
        cudaH2Dcpy(ptr, conv.data(), count);
    }
    return 0;
}
