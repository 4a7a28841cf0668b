// Drop-in for src/weights/llama/norm_weights.h of oneLLM (:2-4).  gamma keeps the reference's float*
// type; an fp16 model stores half data behind it and passes dtype FP16 in the tensors it normalises.
#pragma once
struct LayerNormWeight {
    float* gamma = nullptr;
};
