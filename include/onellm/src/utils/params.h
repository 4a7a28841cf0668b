// Drop-in for src/utils/params.h of oneLLM (:4-5): name -> value dictionaries handed to launchSampling.
#pragma once
#include <string>
#include <unordered_map>

using IntDict = std::unordered_map<std::string, int>;
using floatDict = std::unordered_map<std::string, float>;
