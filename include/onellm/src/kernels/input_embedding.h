// Drop-in for src/kernels/input_embedding.h of oneLLM (:5-7, input_embedding.cu:23-40):
// output[b, s, :] = embed_table[input_ids[b, s], :].
#pragma once
#include "src/utils/tensor.h"

inline void launchInputEmbedding(Tensor* input_ids, Tensor* output, Tensor* embed_table)
{
    const int hidden = output->shape.back();
    ONELLM_B200_CALL(onellm_embedding(onellmDtype(output->dtype), static_cast<const int*>(input_ids->data), output->data,
                                      embed_table->data, output->size() / hidden, hidden, embed_table->shape[0], nullptr, nullptr));
}
