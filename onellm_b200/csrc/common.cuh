// Shared helpers for the sm_100a kernels and their C-ABI entry points.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "onellm_b200.h"

namespace onellm {

// Thread-local text of the last failure, returned by onellm_last_error().
void set_error(const char* fmt, ...);

#define ONELLM_REQUIRE(cond, code, ...)          \
    do {                                         \
        if (!(cond)) {                           \
            ::onellm::set_error(__VA_ARGS__);    \
            return (code);                       \
        }                                        \
    } while (0)

#define ONELLM_CUDA(call)                                                                    \
    do {                                                                                     \
        cudaError_t e__ = (call);                                                            \
        if (e__ != cudaSuccess) {                                                            \
            ::onellm::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),     \
                                __FILE__, __LINE__);                                         \
            return ONELLM_ERR_CUDA;                                                          \
        }                                                                                    \
    } while (0)

// Launch errors (bad configuration, missing kernel image) show up here; execution errors
// surface at the caller's next synchronisation, as in the reference.
#define ONELLM_CHECK_LAUNCH()                                                                \
    do {                                                                                     \
        cudaError_t e__ = cudaPeekAtLastError();                                             \
        if (e__ != cudaSuccess) {                                                            \
            (void)cudaGetLastError();                                                        \
            ::onellm::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), \
                                __FILE__, __LINE__);                                         \
            return ONELLM_ERR_CUDA;                                                          \
        }                                                                                    \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int num_sms()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// 16-byte vector of T <-> float registers.
template <typename T>
struct Vec16;

template <>
struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float (&f)[4])
    {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ static __forceinline__ void unpack(const uint4& r, float (&f)[4])
    {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
        f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[4])
    {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
};

template <>
struct Vec16<__half> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void unpack(const uint4& r, float (&f)[8])
    {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ void load(const __half* p, float (&f)[8])
    {
        unpack(*reinterpret_cast<const uint4*>(p), f);
    }
};

__device__ __forceinline__ uint4 ld_nc_16(const void* p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

inline size_t dtype_size(int dtype) { return dtype == ONELLM_F16 ? 2 : (dtype == ONELLM_F32 ? 4 : 0); }

}  // namespace onellm
