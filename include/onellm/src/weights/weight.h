// Drop-in for src/weights/weight.h of oneLLM (:2-4): anything that can fill itself from a path prefix.
#pragma once
#include <string>

struct Weight {
    virtual void loadWeights(std::string weight_path) = 0;
    virtual ~Weight() = default;
};
