// Drop-in for src/kernels/build_casual_mask.h of oneLLM (:4-9, build_casual_mask.cu:27-60):
// mask [batch, max_q_len, max_k_len] of 1/0 with the shipped predicate (:40-43).
#pragma once
#include <cuda_fp16.h>

#include "src/utils/macro.h"

template <typename T>
void launchBuildCausalMasks(T* mask, const int* q_lens, const int* k_lens, int max_q_len, int max_k_len, int batch_size)
{
    static_assert(sizeof(T) == 4 || sizeof(T) == 2, "float or half");
    ONELLM_B200_CALL(onellm_build_causal_mask(sizeof(T) == 2 ? ONELLM_F16 : ONELLM_F32, mask, q_lens, k_lens, max_q_len, max_k_len,
                                              batch_size, /*attend_history=*/0, nullptr));
}
