// Drop-in for src/weights/base_weights.h of oneLLM (:5-49): the precision tag of a weight and the
// {shape, data, type, bias} record every projection is described by.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>
#include <vector>

enum class WeightType { FP32_W, FP16_W, INT8_W, UNSUPPORTED_W };

inline int getBitNum(WeightType type)
{
    return type == WeightType::FP32_W ? 32 : type == WeightType::FP16_W ? 16 : type == WeightType::INT8_W ? 8 : 0;
}

template <typename T>
inline WeightType getWeightType()
{
    using U = typename std::remove_cv<T>::type;
    return std::is_same<U, float>::value    ? WeightType::FP32_W
           : std::is_same<U, half>::value   ? WeightType::FP16_W
           : std::is_same<U, int8_t>::value ? WeightType::INT8_W
                                            : WeightType::UNSUPPORTED_W;
}

// data: [shape[0] = K_in, shape[1] = N_out] row-major on the device; bias: [N_out] or null
struct BaseWeight {
    std::vector<int> shape;
    void* data = nullptr;
    WeightType type = WeightType::FP32_W;
    void* bias = nullptr;
};
