// Drop-in for src/kernels/qkv_bias_and_RoPE.h of oneLLM (:6-14, qkv_bias_and_RoPE.cu:167-207):
// context-phase bias + RoPE (position = history_length[b] + index inside the prompt) + re-padding:
// QKV {num_tokens, H + 2*Hkv, D} -> q_buf {B, H, S, D}, k_buf / v_buf {B, Hkv, S, D}.
#pragma once
#include "src/models/llama/llama_params.h"
#include "src/utils/tensor.h"
#include "src/weights/base_weights.h"

inline void launchAddFusedQKVBiasTransposeAndRoPE(Tensor* q_buf, Tensor* k_buf, Tensor* v_buf, Tensor* QKV, BaseWeight& qkv,
                                                  Tensor* padding_offset, Tensor* history_length, Tensor* /*input_length*/,
                                                  LLaMAAttentionStaticParams& params)
{
    ONELLM_CHECK_WITH_INFO(QKV->shape.size() == 3 && q_buf->shape.size() == 4, "launchAddFusedQKVBiasTransposeAndRoPE: bad shapes");
    const int T = QKV->shape[0], QH = QKV->shape[1], D = QKV->shape[2];
    const int B = q_buf->shape[0], H = q_buf->shape[1], S = q_buf->shape[2];
    ONELLM_B200_CALL(onellm_qkv_bias_rope_transpose(onellmDtype(QKV->dtype), q_buf->data, k_buf->data, v_buf->data, QKV->data, qkv.bias,
                                                    static_cast<const int*>(padding_offset->data),
                                                    static_cast<const int*>(history_length->data), B, S, T, H, (QH - H) / 2, D,
                                                    params.rotary_embedding_dim, params.rotary_embedding_base, nullptr));
}
