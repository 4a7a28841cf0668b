// Drop-in for src/kernels/rmsnorm_kernel.h of oneLLM (:6-9, rmsnorm_kernel.cu:85-103): in-place
// RMSNorm of decoder_out [tokens, hidden] with gamma [hidden].  Any hidden size (the reference
// launches hidden/4 threads and stops working above 4096).
#pragma once
#include "src/utils/tensor.h"
#include "src/weights/llama/norm_weights.h"

inline void launchRMSNorm(Tensor* decoder_out, LayerNormWeight& attn_norm_weight, float eps)
{
    ONELLM_CHECK_WITH_INFO(decoder_out->shape.size() >= 2, "launchRMSNorm: [tokens, hidden] expected");
    const int hidden = decoder_out->shape.back();
    ONELLM_B200_CALL(onellm_rmsnorm(onellmDtype(decoder_out->dtype), decoder_out->data, attn_norm_weight.gamma, eps,
                                    decoder_out->size() / hidden, hidden, nullptr));
}
