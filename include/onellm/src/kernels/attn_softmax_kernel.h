// Drop-in for src/kernels/attn_softmax_kernel.h of oneLLM (:5-8, attn_softmax_kernel.cu:121-176):
// attn_score = softmax(scale * qk) over the columns the mask keeps; qk [B, H, q_len, k_len],
// mask [B, q_len, k_len] in the dtype of qk.  May run in place.
#pragma once
#include "src/utils/tensor.h"

inline void launchScaleMaskAndSoftmax(Tensor* qk, Tensor* mask, Tensor* attn_score, float scale)
{
    ONELLM_CHECK_WITH_INFO(qk->shape.size() == 4, "launchScaleMaskAndSoftmax: qk [B, H, q_len, k_len] expected");
    ONELLM_B200_CALL(onellm_scale_mask_softmax(onellmDtype(qk->dtype), attn_score->data, qk->data, mask->data, qk->shape[0],
                                               qk->shape[1], qk->shape[2], qk->shape[3], scale, nullptr));
}
