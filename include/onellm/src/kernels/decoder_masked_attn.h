// Drop-in for src/kernels/decoder_masked_attn.h of oneLLM (:7-14, decoder_masked_attn.cu:280-327):
// decode-step attention for one new token per sequence: bias + RoPE on q and k, k/v appended to the
// cache at row step-1, softmax(q.K^T / sqrt(D)).V over rows [0, step).
//   qkv_buf {B, H + 2*Hkv, D}; qkv.bias [(H + 2*Hkv)*D] or null; step: one int on the host;
//   k_cache / v_cache: ONE layer's cache, either {L, B, Hkv, S, D} (the layers' tensors; the caller
//   points data at the layer) or {S, B, Hkv, D} (the order the reference kernel indexes, :163,205);
//   mha_output {B, H*D}.  `finished` is accepted and unused, as in the reference.
// The rotation uses position `step`, as the reference kernel does (:186).
#pragma once
#include <cmath>

#include "src/models/llama/llama_params.h"
#include "src/utils/tensor.h"
#include "src/weights/base_weights.h"

inline void launchDecoderMaskedMHA(Tensor* qkv_buf, BaseWeight& qkv, Tensor* k_cache, Tensor* v_cache, Tensor* /*finished*/,
                                   Tensor* step, Tensor* mha_output, LLaMAAttentionStaticParams& static_params)
{
    ONELLM_CHECK_WITH_INFO(qkv_buf->shape.size() == 3, "launchDecoderMaskedMHA: qkv_buf {B, H+2Hkv, D} expected");
    const int B = qkv_buf->shape[0], QH = qkv_buf->shape[1], D = qkv_buf->shape[2];
    const std::vector<int>& cs = k_cache->shape;
    ONELLM_CHECK_WITH_INFO(cs.size() == 5 || cs.size() == 4, "launchDecoderMaskedMHA: 4-D or 5-D cache expected");
    const int Hkv = cs[2];
    const int H = QH - 2 * Hkv;
    long stride_b, stride_h, stride_s;
    int S;
    if (cs.size() == 5) {  // {L, B, Hkv, S, D}
        S = cs[3];
        stride_b = (long)Hkv * S * D; stride_h = (long)S * D; stride_s = D;
    } else {               // {S, B, Hkv, D}
        S = cs[0];
        stride_b = (long)Hkv * D; stride_h = D; stride_s = (long)cs[1] * Hkv * D;
    }
    const int cur = readScalarInt(step);
    ONELLM_CHECK_WITH_INFO(cur >= 1 && cur <= S, "launchDecoderMaskedMHA: step outside the cache");
    const int dt = onellmDtype(qkv_buf->dtype);
    const size_t esz = getTypeSize(qkv_buf->dtype);
    const char* base = static_cast<const char*>(qkv_buf->data);
    const char* bias = static_cast<const char*>(qkv.bias);
    static thread_local void* ws = nullptr;
    static thread_local size_t ws_bytes = 0;
    const size_t need = onellm_decode_attn_workspace_bytes(B, H, D, cur);
    if (need > ws_bytes) {
        if (ws) CHECK(cudaFree(ws));
        CHECK(cudaMalloc(&ws, need));
        ws_bytes = need;
    }
    ONELLM_B200_CALL(onellm_decode_attn(dt, base, base + (size_t)H * D * esz, base + (size_t)(H + Hkv) * D * esz, (long)QH * D,
                                        (long)QH * D, (long)QH * D, bias, bias ? bias + (size_t)H * D * esz : nullptr,
                                        bias ? bias + (size_t)(H + Hkv) * D * esz : nullptr, k_cache->data, v_cache->data, stride_b,
                                        stride_h, stride_s, B, H, Hkv, D, cur, nullptr, /*rope_pos=*/cur,
                                        static_params.rotary_embedding_dim, static_params.rotary_embedding_base,
                                        1.0f / std::sqrt((float)D), mha_output->data, (long)H * D, ws, ws_bytes, nullptr));
}
