// Shared helpers for the sm_100a kernels and their C-ABI entry points.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "onellm_b200.h"

namespace onellm {

// Thread-local text of the last failure, returned by onellm_last_error().
void set_error(const char* fmt, ...);
// Every kernel launch of the library is counted per host thread (launch_pdl does it itself).
void note_launch(int n = 1);
long launches_noted();

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

// Function attributes (cudaFuncSetAttribute), occupancy figures and the SM count belong to a device, not to
// the process: whatever caches them is indexed by the device the calling thread has current.
constexpr int kMaxDevices = 64;
inline int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}

// Runs `f` (returning cudaError_t) the first time it is reached on each device; later calls on that device
// return cudaSuccess without running it.  One object per call site (a function-local static).
class DeviceOnce {
    std::mutex mu_;
    bool done_[kMaxDevices] = {};

  public:
    template <typename F>
    cudaError_t run(F f)
    {
        const int dev = current_device();
        std::lock_guard<std::mutex> lock(mu_);
        if (done_[dev]) return cudaSuccess;
        const cudaError_t e = f();
        if (e == cudaSuccess) done_[dev] = true;
        return e;
    }
};

// Every kernel of a decode step asks for the same L1 / shared-memory split (the largest shared memory).  An SM
// changes its split only while it is idle: a kernel that follows one with a different split finds the old split
// on every SM that still holds a block, fits fewer of its own blocks there, and a launch planned for one wave runs
// in two (measured on B200: the 33 MB o_proj behind the decode attention took 20 us instead of 10).
// Call before launching `kernel`; the attribute is set once per (kernel, device).
cudaError_t prefer_max_shared(const void* kernel);

inline int num_sms()
{
    static int n[kMaxDevices] = {};
    const int dev = current_device();
    if (n[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
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

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
constexpr int kMaxStages = 26;
// wait_group takes an immediate; the ring depth is chosen per launch, hence the switch
__device__ __forceinline__ void cp_async_wait_dyn(int pending)
{
    switch (pending) {
#define ONELLM_W(n) case n: cp_async_wait<n>(); break;
        ONELLM_W(0) ONELLM_W(1) ONELLM_W(2) ONELLM_W(3) ONELLM_W(4) ONELLM_W(5) ONELLM_W(6) ONELLM_W(7) ONELLM_W(8)
        ONELLM_W(9) ONELLM_W(10) ONELLM_W(11) ONELLM_W(12) ONELLM_W(13) ONELLM_W(14) ONELLM_W(15) ONELLM_W(16)
        ONELLM_W(17) ONELLM_W(18) ONELLM_W(19) ONELLM_W(20) ONELLM_W(21) ONELLM_W(22) ONELLM_W(23)
#undef ONELLM_W
        default: cp_async_wait<24>(); break;
    }
}
// Programmatic dependent launch.  A kernel launched with launch_pdl() may start while the
// kernel before it in the stream is still running; pdl_wait() blocks until that kernel has
// completed and its writes are visible, so everything that reads (or overwrites) data the
// previous kernel touches must come after it.  EVERY kernel of a chain calls pdl_wait() once,
// also when it has nothing to wait for: completion is only transitive through the waits.
// pdl_launch_dependents() lets the next kernel begin its own independent prologue early.
// Both are no-ops in a kernel that was launched normally.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    note_launch();
    (void)prefer_max_shared(reinterpret_cast<const void*>(kernel));  // one L1 / shared-memory split for every kernel of a step
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// warp-level tensor-core helpers (mma.sync path)
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi)
{
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
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

// Tensor-parallel epilogue of a projection (p2p_allreduce.cu owns the buffers): the block that has
// finished an output element pushes it, as one 8-byte word {two fp16 values, sequence number}, into this
// rank's slot on every peer, then waits for the peers' words of the same element in its own memory and
// adds them in rank order.  world <= 1: not in use.
// two_shot (large messages on many ranks): token row t belongs to rank t % world.  Every rank sends its partial
// of a row to the row's owner only; the owner adds the partials in rank order, the residual and the bias, stores
// the result and sends it, again as {two fp16 values, sequence number}, to every peer's `final` buffer; the
// others store what they receive.  Same arithmetic, same bits as the one-shot form, 2 (world-1)/world of a
// message per rank on the wire instead of (world-1) messages, at the price of a second hop.
constexpr int kTpMaxBlocks = 1024;  // sequence counters available to one launch
struct TpEpilogue {
    uint2* push[8];        // this rank's slot in the receive buffer of rank r (entry of the own rank unused)
    const uint2* mine;     // this rank's receive buffer of this call: [world][slot_words]
    uint2* final_push[8];  // two_shot: the final-value buffer of rank r for this call
    const uint2* final_mine;
    int two_shot;
    size_t slot_words;
    int* counters;         // one sequence counter per thread block of the launch
    int* error;            // set when a bounded wait gave up
    int rank, world;
};

inline size_t dtype_size(int dtype) { return dtype == ONELLM_F16 ? 2 : (dtype == ONELLM_F32 ? 4 : 0); }

}  // namespace onellm
