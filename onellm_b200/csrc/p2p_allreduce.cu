// One-shot all-reduce over peer memory, fused with the residual add, for the tensor-parallel decode step.
//
// In the tensor-parallel decoder the partial outputs of o_proj and down_proj ([tokens, hidden] fp16,
// 64 KB at batch 8) are summed over the ranks and added to the residual stream
// (src/layers/decoder/self_decoder.cpp:50-73 of the reference run under tensor parallelism).  A
// library all-reduce costs ten to twenty microseconds of latency for such a message, twice per layer.
// Here every rank keeps its partial in a buffer the other ranks can map (CUDA IPC over NVLink /
// NVSwitch), tells them with one flag store per peer that it is complete, and then reads all the
// partials itself with plain peer loads, adds them in rank order (every rank gets bit-identical sums)
// together with the residual and the bias, and writes only its own copy of the residual stream:
//
//     residual <- residual + bias + sum_r partial_r
//
// Synchronisation is per thread block and needs no cross-block state: block b of rank r owns a
// sequence counter, stores it into slot [b][r] of every peer's flag array and waits until its own
// slots [b][0..world) have reached it.  Two send buffers are used in turn (o_proj, down_proj); a rank
// can only overwrite a buffer two calls later, after every peer has announced the call in between,
// which it does only once its reads of the earlier call are over.  Every wait is bounded: when it
// runs out the block sets the error word of its rank and carries on with whatever the peers' buffers
// hold, so the kernel always ends.
//
// No multicast, no multimem: plain loads and stores on mapped peer memory.
#include <string.h>

#include <vector>

#include "common.cuh"

namespace onellm {

constexpr int kP2pMaxWorld = 8;
constexpr int kP2pMaxBlocks = 64;
constexpr int kP2pThreads = 256;
constexpr int kP2pVecPerThread = 4;                       // 16-byte vectors per thread
constexpr long long kP2pWaitCycles = 2000LL * 1000 * 1000;  // a wait for a peer gives up after about a second of SM clocks

// Layout of the block every rank allocates and exports:
//   [0]            control: flags[kP2pMaxBlocks][kP2pMaxWorld] (written by peers), counters[kP2pMaxBlocks], error
//   [kCtlBytes]    send buffer 0, send buffer 1 (max_elems halfs each)
struct P2pControl {
    int flags[kP2pMaxBlocks][kP2pMaxWorld];
    int counters[kP2pMaxBlocks];
    int error;
    int pad[63];
};
constexpr size_t kCtlBytes = (sizeof(P2pControl) + 255) / 256 * 256;

struct P2pPeers {
    const __half* data[kP2pMaxWorld];  // send buffer of this call on every rank (own included)
    P2pControl* ctl[kP2pMaxWorld];     // control block of every rank (own included)
};

__device__ __forceinline__ void st_relaxed_sys(int* p, int v) { asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_relaxed_sys(const int* p)
{
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acquire_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// peer data is read once per call, after the acquire on the peer's flag: a system-scope load that
// bypasses the non-coherent path
__device__ __forceinline__ uint4 ld_relaxed_sys_16(const void* p)
{
    uint4 r;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

__global__ void __launch_bounds__(kP2pThreads)
p2p_allreduce_add_kernel(const P2pPeers peers, int rank, int world, __half* __restrict__ resid, const __half* __restrict__ bias,
                         int n_elems, int row_len)
{
    __shared__ int s_seq;
    pdl_launch_dependents();
    pdl_wait();  // the projection that wrote this rank's partial has completed and its stores are visible
    P2pControl* mine = peers.ctl[rank];
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        const int seq = mine->counters[b] + 1;
        mine->counters[b] = seq;
        s_seq = seq;
    }
    __syncthreads();
    const int seq = s_seq;
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        // "partial number seq of rank `rank` is complete".  No release fence is needed in front of the store:
        // the partial was written by the kernel before this one, whose completion (griddepcontrol.wait above)
        // has already made it visible at system scope.
        st_relaxed_sys(&peers.ctl[p]->flags[b][rank], seq);
        const long long t0 = clock64();  // the SM's own cycle counter: reading it costs nothing next to the poll
        while (ld_relaxed_sys(&mine->flags[b][p]) < seq) {
            if (clock64() - t0 > kP2pWaitCycles) {
                atomicExch(&mine->error, 1);
                break;
            }
        }
        fence_acquire_sys();  // the peer's partial is read only after its flag has been seen
    }
    __syncthreads();
    const int n_vec = n_elems / 8;
    const int v0 = (b * kP2pThreads + threadIdx.x) * kP2pVecPerThread;
    uint4 part[kP2pMaxWorld][kP2pVecPerThread];
#pragma unroll
    for (int r = 0; r < kP2pMaxWorld; r++)
        if (r < world) {
#pragma unroll
            for (int j = 0; j < kP2pVecPerThread; j++)
                if (v0 + j < n_vec) part[r][j] = ld_relaxed_sys_16(peers.data[r] + (size_t)(v0 + j) * 8);
        }
#pragma unroll
    for (int j = 0; j < kP2pVecPerThread; j++) {
        const int v = v0 + j;
        if (v >= n_vec) break;
        float acc[8] = {}, f[8];
#pragma unroll
        for (int r = 0; r < kP2pMaxWorld; r++)
            if (r < world) {
                Vec16<__half>::unpack(part[r][j], f);
#pragma unroll
                for (int e = 0; e < 8; e++) acc[e] += f[e];
            }
        Vec16<__half>::load(resid + (size_t)v * 8, f);
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += f[e];
        if (bias) {
            Vec16<__half>::load(bias + ((size_t)v * 8) % row_len, f);
#pragma unroll
            for (int e = 0; e < 8; e++) acc[e] += f[e];
        }
        *reinterpret_cast<uint4*>(resid + (size_t)v * 8) = Vec16<__half>::pack(acc);
    }
}

struct P2pComm {
    int rank = 0, world = 1, device = 0;
    size_t max_elems = 0, block_bytes = 0;
    void* local = nullptr;                    // this rank's block
    void* mapped[kP2pMaxWorld] = {};          // every rank's block in this process's address space
    bool connected = false;
};

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_p2p_create(int rank, int world, size_t max_elems, onellm_p2p** out)
{
    ONELLM_REQUIRE(out, ONELLM_ERR_ARG, "p2p_create: null pointer");
    ONELLM_REQUIRE(world >= 2 && world <= kP2pMaxWorld && rank >= 0 && rank < world, ONELLM_ERR_ARG, "p2p_create: rank %d of %d (2..%d ranks)",
                   rank, world, kP2pMaxWorld);
    ONELLM_REQUIRE(max_elems >= 8 && max_elems % 8 == 0 &&
                       max_elems <= (size_t)kP2pMaxBlocks * kP2pThreads * kP2pVecPerThread * 8,
                   ONELLM_ERR_ARG, "p2p_create: max_elems must be a multiple of 8, at most %d",
                   kP2pMaxBlocks * kP2pThreads * kP2pVecPerThread * 8);
    P2pComm* c = new P2pComm();
    c->rank = rank;
    c->world = world;
    c->max_elems = max_elems;
    c->block_bytes = kCtlBytes + 2 * ((max_elems * sizeof(__half) + 255) / 256 * 256);
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(&c->local, c->block_bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->block_bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("p2p_create: %s", cudaGetErrorString(e));
        if (c->local) cudaFree(c->local);
        delete c;
        return ONELLM_ERR_CUDA;
    }
    c->mapped[rank] = c->local;
    *out = reinterpret_cast<onellm_p2p*>(c);
    return ONELLM_OK;
}

extern "C" int onellm_p2p_handle(onellm_p2p* h, void* handle64)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    ONELLM_REQUIRE(c && handle64, ONELLM_ERR_ARG, "p2p_handle: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == ONELLM_P2P_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t hd;
    ONELLM_CUDA(cudaIpcGetMemHandle(&hd, c->local));
    memcpy(handle64, &hd, sizeof(hd));
    return ONELLM_OK;
}

extern "C" int onellm_p2p_connect(onellm_p2p* h, const void* handles)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    ONELLM_REQUIRE(c && handles, ONELLM_ERR_ARG, "p2p_connect: null pointer");
    ONELLM_REQUIRE(!c->connected, ONELLM_ERR_STATE, "p2p_connect: already connected");
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t hd;
        memcpy(&hd, static_cast<const char*>(handles) + (size_t)r * sizeof(hd), sizeof(hd));
        const cudaError_t e = cudaIpcOpenMemHandle(&c->mapped[r], hd, cudaIpcMemLazyEnablePeerAccess);
        ONELLM_REQUIRE(e == cudaSuccess, ONELLM_ERR_COMM, "p2p_connect: cannot map the buffer of rank %d: %s", r, cudaGetErrorString(e));
    }
    c->connected = true;
    return ONELLM_OK;
}

extern "C" void* onellm_p2p_send_buffer(onellm_p2p* h, int which)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    if (!c || which < 0 || which > 1) return nullptr;
    const size_t buf_bytes = (c->max_elems * sizeof(__half) + 255) / 256 * 256;
    return static_cast<char*>(c->local) + kCtlBytes + (size_t)which * buf_bytes;
}

extern "C" int onellm_p2p_allreduce_add(onellm_p2p* h, int dtype, int which, void* resid, const void* bias, int n_elems, int row_len,
                                        void* stream)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    ONELLM_REQUIRE(c && resid, ONELLM_ERR_ARG, "p2p_allreduce_add: null pointer");
    ONELLM_REQUIRE(c->connected, ONELLM_ERR_STATE, "p2p_allreduce_add: call onellm_p2p_connect first");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "p2p_allreduce_add: only F16 is implemented");
    ONELLM_REQUIRE(which == 0 || which == 1, ONELLM_ERR_ARG, "p2p_allreduce_add: send buffer 0 or 1");
    ONELLM_REQUIRE(n_elems > 0 && n_elems % 8 == 0 && (size_t)n_elems <= c->max_elems && row_len > 0 && row_len % 8 == 0 &&
                       n_elems % row_len == 0,
                   ONELLM_ERR_ARG, "p2p_allreduce_add: %d elements in rows of %d do not fit (multiples of 8, at most %zu)", n_elems,
                   row_len, c->max_elems);
    ONELLM_REQUIRE(aligned16(resid) && (!bias || aligned16(bias)), ONELLM_ERR_ARG, "p2p_allreduce_add: pointers must be 16-byte aligned");
    P2pPeers peers = {};
    const size_t buf_bytes = (c->max_elems * sizeof(__half) + 255) / 256 * 256;
    for (int r = 0; r < c->world; r++) {
        peers.ctl[r] = static_cast<P2pControl*>(c->mapped[r]);
        peers.data[r] = reinterpret_cast<const __half*>(static_cast<const char*>(c->mapped[r]) + kCtlBytes + (size_t)which * buf_bytes);
    }
    const int per_block = kP2pThreads * kP2pVecPerThread * 8;
    const int blocks = (n_elems + per_block - 1) / per_block;  // the same on every rank: blocks pair up by index
    ONELLM_CUDA(launch_pdl(p2p_allreduce_add_kernel, dim3(blocks), dim3(kP2pThreads), 0, reinterpret_cast<cudaStream_t>(stream), peers,
                           c->rank, c->world, (__half*)resid, (const __half*)bias, n_elems, row_len));
    return ONELLM_OK;
}

extern "C" int onellm_p2p_error(onellm_p2p* h)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    if (!c || !c->local) return -1;
    int v = 0;
    if (cudaMemcpy(&v, &static_cast<P2pControl*>(c->local)->error, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return v;
}

extern "C" void onellm_p2p_destroy(onellm_p2p* h)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    if (!c) return;
    for (int r = 0; r < c->world; r++)
        if (r != c->rank && c->mapped[r]) cudaIpcCloseMemHandle(c->mapped[r]);
    if (c->local) cudaFree(c->local);
    delete c;
}
