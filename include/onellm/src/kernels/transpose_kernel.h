// Drop-in for src/kernels/transpose_kernel.h of oneLLM (:5-11, transpose_kernel.cu:45-88): copies
// rows [0, context_length[b]) of one layer's K and V cache into {B, H, max_k_len, D} buffers,
// repeating every KV head H/Hkv times.  The source is {B, Hkv, S, D} or the whole {L, B, Hkv, S, D}
// cache with layer_id selecting the layer (the reference reads Hkv and S from shape[1] and shape[2]).
#pragma once
#include "src/utils/tensor.h"

inline void launchTransposeKVCache(Tensor* k_cache_src, Tensor* v_cache_src, Tensor* context_length, Tensor* layer_id,
                                   Tensor* k_cache_dst, Tensor* v_cache_dst)
{
    const size_t rank = k_cache_src->shape.size();
    ONELLM_CHECK_WITH_INFO((rank == 4 || rank == 5) && k_cache_dst->shape.size() == 4, "launchTransposeKVCache: bad shapes");
    const int B = k_cache_dst->shape[0], H = k_cache_dst->shape[1], max_k = k_cache_dst->shape[2], D = k_cache_dst->shape[3];
    const int Hkv = k_cache_src->shape[rank - 3], S = k_cache_src->shape[rank - 2];
    size_t layer_bytes = 0;
    if (rank == 5) layer_bytes = (size_t)readScalarInt(layer_id) * B * Hkv * S * D * getTypeSize(k_cache_src->dtype);
    const int dt = onellmDtype(k_cache_src->dtype);
    const int* ctx = static_cast<const int*>(context_length->data);
    ONELLM_B200_CALL(onellm_repeat_kv(dt, k_cache_dst->data, static_cast<const char*>(k_cache_src->data) + layer_bytes, ctx, B, H, Hkv,
                                      max_k, S, D, nullptr));
    ONELLM_B200_CALL(onellm_repeat_kv(dt, v_cache_dst->data, static_cast<const char*>(v_cache_src->data) + layer_bytes, ctx, B, H, Hkv,
                                      max_k, S, D, nullptr));
}
