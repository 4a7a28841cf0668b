// Drop-in for src/weights/llama/attention_weights.h of oneLLM (:4-10).
#pragma once
#include "src/weights/base_weights.h"

struct LLaMAattentionWeights {
    BaseWeight q, k, v;  // unfused projections (unused by the layers)
    BaseWeight qkv;      // [hidden, (H + 2*Hkv) * D], bias [(H + 2*Hkv) * D]
    BaseWeight output;   // [H*D, hidden]
};
