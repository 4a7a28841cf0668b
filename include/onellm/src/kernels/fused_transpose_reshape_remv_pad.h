// Drop-in for src/kernels/fused_transpose_reshape_remv_pad.h of oneLLM (:5-6,
// fused_transpose_reshape_remv_pad.cu:29-51): [B, H, S, D] -> [num_tokens, H*D] without the pad rows.
#pragma once
#include "src/utils/tensor.h"

inline void launchTransposeOutRemovePadding(Tensor* qkv_buf_w_pad, Tensor* padding_offset, Tensor* qkv_buf_wo_pad_1)
{
    const std::vector<int>& s = qkv_buf_w_pad->shape;
    ONELLM_CHECK_WITH_INFO(s.size() == 4, "launchTransposeOutRemovePadding: [B, H, S, D] expected");
    ONELLM_B200_CALL(onellm_transpose_remove_padding(onellmDtype(qkv_buf_w_pad->dtype), qkv_buf_wo_pad_1->data, qkv_buf_w_pad->data,
                                                     static_cast<const int*>(padding_offset->data), qkv_buf_wo_pad_1->shape[0], s[0],
                                                     s[2], s[1], s[3], nullptr));
}
