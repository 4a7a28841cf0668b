// Drop-in for src/kernels/append_to_kvcache.h of oneLLM (:20-26, append_to_kvcache.cu:73-114):
// k_src / v_src {B, Hkv, max_q_len, D} -> rows history_length[b] + [0, cur_query_length[b]) of the
// cache.  k_dst / v_dst are {B, Hkv, S, D} or the whole {L, B, Hkv, S, D} cache, in which case layer_id
// selects the layer (the reference reads S from shape[2] and always writes layer 0).
// Argument order: the declaration is (k_src, v_src, layer_id, cur_query_length, history_length, ...),
// but the context-attention layer calls it as (k_src, v_src, input_length, history_length, layer_id, ...)
// (src/layers/attention/context_attention.cpp:126-127).  All three are Tensor*, so both compile; the
// one whose data is a host pointer is taken as layer_id and the other two keep their relative order,
// which gives the intended meaning for both call sites.
#pragma once
#include "src/utils/tensor.h"

inline void launchAppendKVCache(Tensor* k_src, Tensor* v_src, Tensor* arg3, Tensor* arg4, Tensor* arg5, Tensor* k_dst, Tensor* v_dst)
{
    Tensor *layer_id = arg3, *cur_query_length = arg4, *history_length = arg5;
    if (!isHostPointer(arg3->data) && isHostPointer(arg5->data)) {
        cur_query_length = arg3;
        history_length = arg4;
        layer_id = arg5;
    }
    ONELLM_CHECK_WITH_INFO(k_src->shape.size() == 4, "launchAppendKVCache: k_src {B, Hkv, max_q_len, D} expected");
    const int B = k_src->shape[0], Hkv = k_src->shape[1], max_q = k_src->shape[2], D = k_src->shape[3];
    const size_t rank = k_dst->shape.size();
    ONELLM_CHECK_WITH_INFO(rank == 4 || rank == 5, "launchAppendKVCache: 4-D or 5-D cache expected");
    const int S = k_dst->shape[rank - 2];
    size_t layer_bytes = 0;
    if (rank == 5) layer_bytes = (size_t)readScalarInt(layer_id) * B * Hkv * S * D * getTypeSize(k_dst->dtype);
    const int dt = onellmDtype(k_src->dtype);
    const int* cur = static_cast<const int*>(cur_query_length->data);
    const int* hist = static_cast<const int*>(history_length->data);
    ONELLM_B200_CALL(onellm_append_kv_cache(dt, static_cast<char*>(k_dst->data) + layer_bytes, k_src->data, cur, hist, B, Hkv, max_q, S, D,
                                            nullptr, nullptr));
    ONELLM_B200_CALL(onellm_append_kv_cache(dt, static_cast<char*>(v_dst->data) + layer_bytes, v_src->data, cur, hist, B, Hkv, max_q, S, D,
                                            nullptr, nullptr));
}
