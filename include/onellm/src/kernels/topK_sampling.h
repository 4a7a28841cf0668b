// Drop-in for src/kernels/topK_sampling.h of oneLLM (:9-14, topK_sampling.cu:43-70): one token per
// row from its top-K candidates.  topk_id / topk_val {B, K} (ids may be row*vocab + column);
// params: "vocab_size", "step" (seeds the generator: curand_init(step, row, 0)), "end_id".
// seqlen[b] += !finished[b]; is_finished[b] = (token == end_id).  The walk over the candidates is the
// corrected one; params["literal_walk"] = 1 (an addition) reproduces the shipped arithmetic (:31-33).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "src/utils/params.h"
#include "src/utils/tensor.h"

inline void launchSampling(Tensor* topk_id, Tensor* topk_val, Tensor* seqlen, Tensor* is_finished, Tensor* output_id, IntDict& params)
{
    const auto literal = params.find("literal_walk");
    ONELLM_B200_CALL(onellm_topk_sample(static_cast<const int*>(topk_id->data), static_cast<const float*>(topk_val->data),
                                        topk_id->shape[0], topk_id->shape[1], /*temperature=*/1.0f, params.at("step"), nullptr,
                                        params.at("vocab_size"), params.at("end_id"),
                                        literal != params.end() && literal->second != 0, static_cast<int*>(output_id->data),
                                        static_cast<int*>(seqlen->data), static_cast<unsigned char*>(is_finished->data), nullptr,
                                        nullptr));
}
