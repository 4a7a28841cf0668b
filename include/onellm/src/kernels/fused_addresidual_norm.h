// Drop-in for src/kernels/fused_addresidual_norm.h of oneLLM (:4-12, fused_addresidual_norm.cu:109-141):
// residual <- decoder_out + residual + bias; decoder_out <- scale * residual * rsqrt(mean(residual^2) + eps).
// bias may be null.
#pragma once
#include <cuda_fp16.h>

#include "src/utils/macro.h"

template <typename T>
void launchFusedAddBiasResidualRMSNorm(T* residual, T* decoder_out, const T* bias, const T* scale, float eps, int num_tokens,
                                       int hidden_units)
{
    static_assert(sizeof(T) == 4 || sizeof(T) == 2, "float or half");
    ONELLM_B200_CALL(onellm_add_residual_rmsnorm(sizeof(T) == 2 ? ONELLM_F16 : ONELLM_F32, residual, decoder_out, bias, scale, eps,
                                                 num_tokens, hidden_units, nullptr));
}
