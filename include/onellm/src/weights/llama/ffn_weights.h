// Drop-in for src/weights/llama/ffn_weights.h of oneLLM (:4-8).
#pragma once
#include "src/weights/base_weights.h"

struct LLaMAFFNWeights {
    BaseWeight gate;  // [hidden, inter]
    BaseWeight up;    // [hidden, inter]
    BaseWeight down;  // [inter, hidden]
};
