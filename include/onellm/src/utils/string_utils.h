// Drop-in for src/utils/string_utils.h of oneLLM (fmtstr :7-22, vec2str :24-38, arr2str :40-53):
// printf-style formatting into std::string and "(a, b, c)" rendering of sequences.
#pragma once
#include <cstdio>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

template <typename... Args>
inline std::string fmtstr(const std::string& format, Args... args)
{
    const int n = std::snprintf(nullptr, 0, format.c_str(), args...);
    if (n < 0) throw std::runtime_error("fmtstr: invalid format string");
    std::string out(static_cast<size_t>(n) + 1, '\0');
    std::snprintf(&out[0], out.size(), format.c_str(), args...);
    out.resize(static_cast<size_t>(n));
    return out;
}

template <typename T>
inline std::string arr2str(T* arr, size_t size)
{
    std::ostringstream os;
    os << "(";
    for (size_t i = 0; i < size; ++i) os << (i ? ", " : "") << arr[i];
    os << ")";
    return os.str();
}

template <typename T>
inline std::string vec2str(std::vector<T> vec)
{
    return arr2str(vec.data(), vec.size());
}
