// Helpers shared by the drop-in test programs: the seeded generator tests/test_dropin_gpu.py mirrors, uploads, and
// raw float dumps into the output directory.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "src/utils/macro.h"

static uint32_t g_state = 12345u;
static float next_uniform()  // the generator tests/test_dropin_gpu.py mirrors
{
    g_state = g_state * 1664525u + 1013904223u;
    return (float)(g_state >> 8) / 16777216.0f - 0.5f;
}
static std::vector<float> randv(size_t n, float scale)
{
    std::vector<float> v(n);
    for (auto& x : v) x = next_uniform() * scale;
    return v;
}
template <typename T>
static T* to_dev(const std::vector<T>& h)
{
    T* d = nullptr;
    CHECK(cudaMalloc((void**)&d, h.size() * sizeof(T)));
    CHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}
static std::string g_dir;
static void dump(const char* name, const void* dev, size_t n_floats)
{
    std::vector<float> h(n_floats);
    CHECK(cudaMemcpy(h.data(), dev, n_floats * sizeof(float), cudaMemcpyDeviceToHost));
    std::FILE* f = std::fopen((g_dir + "/" + name + ".f32").c_str(), "wb");
    if (!f || std::fwrite(h.data(), sizeof(float), n_floats, f) != n_floats) {
        std::fprintf(stderr, "cannot write %s\n", name);
        std::exit(2);
    }
    std::fclose(f);
}

