// Drop-in for src/kernels/activation_kernel.h of oneLLM (:2-3, activation_kernel.cu:23-32):
// out[t, i] = silu(input[t, 0, i]) * input[t, 1, i], input [batch_size, 2, intermedia_size].
#pragma once
#include <cuda_fp16.h>

#include "src/utils/macro.h"

template <typename T>
void launchAct(const T* input, T* out, const int batch_size, const int intermedia_size)
{
    static_assert(sizeof(T) == 4 || sizeof(T) == 2, "float or half");
    ONELLM_B200_CALL(onellm_swiglu(sizeof(T) == 2 ? ONELLM_F16 : ONELLM_F32, input, out, batch_size, intermedia_size, nullptr));
}
