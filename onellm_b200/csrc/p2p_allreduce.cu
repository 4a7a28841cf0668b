// One-shot all-reduce over peer memory, fused with the residual add, for the tensor-parallel decode step.
//
// In the tensor-parallel decoder the partial outputs of o_proj and down_proj ([tokens, hidden] fp16,
// 64 KB at batch 8) are summed over the ranks and added to the residual stream
// (src/layers/decoder/self_decoder.cpp:50-73 of the reference run under tensor parallelism).  A
// library all-reduce costs ten to twenty microseconds of latency for such a message, twice per layer.
// Here every rank owns receive buffers the other ranks can map (CUDA IPC over NVLink / NVSwitch).
// One kernel per call: each rank PUSHES its partial into its slot of every peer's receive buffer with
// plain peer stores, then waits for the peers' partials to arrive in its own memory, adds them in rank
// order (every rank gets bit-identical sums) together with the residual and the bias, and writes only
// its own copy of the residual stream:
//
//     residual <- residual + bias + sum_r partial_r
//
// There are no flags and no fences: every 8-byte word that crosses the link is {two fp16 values, the
// call's sequence number}, written with one store, so a word is valid exactly when its sequence number
// is the one the receiver expects (the receiver polls the data itself; the cost of a call is one
// one-way store latency instead of a flag round plus a load round trip).  Sequence numbers are per
// thread block (block b of every rank pairs with block b of the others), so there is no cross-block
// state.  Two receive buffers are used in turn (o_proj, down_proj): a rank can only overwrite a slot two
// calls later, after the owner has pushed the call in between, which it does only once its reads of the
// earlier call are over.  Every wait is bounded: when it runs out the block sets the error word of its
// rank and carries on with whatever the buffers hold, so the kernel always ends.
//
// No multicast, no multimem: plain loads and stores on mapped peer memory.
#include <string.h>

#include <vector>

#include "common.cuh"

namespace onellm {

constexpr int kP2pMaxWorld = 8;
constexpr int kP2pMaxBlocks = 128;
constexpr int kP2pThreads = 256;
constexpr int kP2pVecPerThread = 2;                       // 16-byte vectors per thread
constexpr long long kP2pWaitCycles = 2000LL * 1000 * 1000;  // a wait for a peer gives up after about a second of SM clocks

// Layout of the block every rank allocates and exports:
//   [0]            control: counters[kP2pMaxBlocks] (sequence number per thread block), error, the same
//                  counters again for the projections that push from their own epilogue
//   [kCtlBytes]    send buffer 0, send buffer 1 (max_elems halfs each; written by this rank's projections)
//   [..]           receive buffers [2][world][max_elems / 2] of 8-byte words {half2 data, sequence number},
//                  slot [which][r] written by rank r
//   [..]           final-value buffers [2][max_elems / 2] of the same words (two-shot form of the projections'
//                  exchange: element e written by the rank that owns its token row)
struct P2pControl {
    int counters[kP2pMaxBlocks];
    int error;
    int pad[63];
    int gemm_counters[kTpMaxBlocks];  // sequence numbers of the projections that reduce in their own epilogue
};
constexpr size_t kCtlBytes = (sizeof(P2pControl) + 255) / 256 * 256;

struct P2pPeers {
    uint2* recv[kP2pMaxWorld];  // this rank's slot [which][rank] in the receive buffer of every rank (own entry unused)
};

__device__ __forceinline__ void st_relaxed_sys_16(void* p, uint4 v)
{
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_16(const void* p)
{
    uint4 r;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

// send: this rank's partial (local); my_recv: this rank's receive buffer of this call, [world][slot_words] words.
__global__ void __launch_bounds__(kP2pThreads)
p2p_allreduce_add_kernel(const P2pPeers peers, P2pControl* __restrict__ ctl, const __half* __restrict__ send,
                         const uint2* __restrict__ my_recv, size_t slot_words, int rank, int world, __half* __restrict__ resid,
                         const __half* __restrict__ bias, int n_elems, int row_len)
{
    __shared__ int s_seq;
    pdl_launch_dependents();
    pdl_wait();  // the projection that wrote this rank's partial has completed
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        const int seq = ctl->counters[b] + 1;
        ctl->counters[b] = seq;
        s_seq = seq;
    }
    __syncthreads();
    const uint32_t seq = (uint32_t)s_seq;
    const int n_vec = n_elems / 8;           // 16 bytes of fp16 = 4 words on the wire
    const int v0 = (b * kP2pThreads + threadIdx.x) * kP2pVecPerThread;

    // 1. push: {d0, seq, d1, seq} {d2, seq, d3, seq} per 16 bytes of the partial, to every peer
    uint4 own[kP2pVecPerThread];
#pragma unroll
    for (int j = 0; j < kP2pVecPerThread; j++) {
        own[j] = make_uint4(0u, 0u, 0u, 0u);
        if (v0 + j < n_vec) own[j] = *reinterpret_cast<const uint4*>(send + (size_t)(v0 + j) * 8);
    }
#pragma unroll
    for (int r = 0; r < kP2pMaxWorld; r++)
        if (r < world && r != rank) {
#pragma unroll
            for (int j = 0; j < kP2pVecPerThread; j++)
                if (v0 + j < n_vec) {
                    uint2* dst = peers.recv[r] + (size_t)(v0 + j) * 4;
                    st_relaxed_sys_16(dst, make_uint4(own[j].x, seq, own[j].y, seq));
                    st_relaxed_sys_16(dst + 2, make_uint4(own[j].z, seq, own[j].w, seq));
                }
        }

    // 2. collect: a word of a peer is there when it carries this call's sequence number
    uint4 part[kP2pMaxWorld][kP2pVecPerThread];
    const long long t0 = clock64();  // the SM's own cycle counter bounds the wait
    bool gave_up = false;
#pragma unroll
    for (int r = 0; r < kP2pMaxWorld; r++)
        if (r < world) {
#pragma unroll
            for (int j = 0; j < kP2pVecPerThread; j++) {
                part[r][j] = own[j];
                if (r == rank || v0 + j >= n_vec) continue;
                const uint2* src = my_recv + (size_t)r * slot_words + (size_t)(v0 + j) * 4;
                uint4 lo, hi;
                for (;;) {
                    lo = ld_relaxed_sys_16(src);
                    hi = ld_relaxed_sys_16(src + 2);
                    if ((lo.y == seq && lo.w == seq && hi.y == seq && hi.w == seq) || gave_up) break;
                    if (clock64() - t0 > kP2pWaitCycles) {
                        atomicExch(&ctl->error, 1);
                        gave_up = true;
                    }
                }
                part[r][j] = make_uint4(lo.x, lo.z, hi.x, hi.z);
            }
        }

    // 3. sum in rank order, add residual and bias, store
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
    size_t send_bytes() const { return (max_elems * sizeof(__half) + 255) / 256 * 256; }
    size_t slot_words() const { return max_elems / 2; }
    // receive slot [which][src] inside the block that starts at `base`
    uint2* recv_slot(void* base, int which, int src) const
    {
        return reinterpret_cast<uint2*>(static_cast<char*>(base) + kCtlBytes + 2 * send_bytes()) +
               ((size_t)which * world + src) * slot_words();
    }
    // final-value buffer [which] (two-shot exchange) inside the block that starts at `base`
    uint2* final_slot(void* base, int which) const { return recv_slot(base, 2, 0) + (size_t)which * slot_words(); }
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
    c->block_bytes = kCtlBytes + 2 * c->send_bytes() + (size_t)2 * (world + 1) * c->slot_words() * sizeof(uint2);
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
    return static_cast<char*>(c->local) + kCtlBytes + (size_t)which * c->send_bytes();
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
    for (int r = 0; r < c->world; r++) peers.recv[r] = c->recv_slot(c->mapped[r], which, c->rank);  // my slot on rank r
    const int per_block = kP2pThreads * kP2pVecPerThread * 8;
    const int blocks = (n_elems + per_block - 1) / per_block;  // the same on every rank: blocks pair up by index
    ONELLM_CUDA(launch_pdl(p2p_allreduce_add_kernel, dim3(blocks), dim3(kP2pThreads), 0, reinterpret_cast<cudaStream_t>(stream), peers,
                           static_cast<P2pControl*>(c->local), static_cast<const __half*>(onellm_p2p_send_buffer(h, which)),
                           (const uint2*)c->recv_slot(c->local, which, 0), c->slot_words(), c->rank, c->world, (__half*)resid,
                           (const __half*)bias, n_elems, row_len));
    return ONELLM_OK;
}

namespace onellm {
// bytes a rank would put on the wire in the one-shot form from which the projections' exchange goes two-shot
static long long g_two_shot_bytes = 3ll << 20;
// skinny_gemm_staged.cu
cudaError_t skinny_kn_staged_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K, bool dual,
                                      cudaStream_t st, const __half* resid, const __half* bias, float rms_eps, const TpEpilogue* tp);
}

// The projection and the all-reduce in ONE kernel: resid <- resid + bias + sum over ranks of (x . W), W this
// rank's [K, N] slice.  A block that has finished two output elements pushes them to every peer at once and
// gathers the peers' values of the same elements, so the link latency overlaps the rest of the projection.
extern "C" int onellm_p2p_gemm_allreduce_add(onellm_p2p* h, int dtype, int which, const void* x, const void* W, void* resid,
                                             const void* bias, int M, int N, int K, void* stream)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    ONELLM_REQUIRE(c && x && W && resid, ONELLM_ERR_ARG, "p2p_gemm_allreduce_add: null pointer");
    ONELLM_REQUIRE(c->connected, ONELLM_ERR_STATE, "p2p_gemm_allreduce_add: call onellm_p2p_connect first");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "p2p_gemm_allreduce_add: only F16 is implemented");
    ONELLM_REQUIRE(which == 0 || which == 1, ONELLM_ERR_ARG, "p2p_gemm_allreduce_add: receive buffer 0 or 1");
    ONELLM_REQUIRE(M >= 1 && M <= 64 && N > 0 && K > 0 && K % 16 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED,
                   "p2p_gemm_allreduce_add: 1..64 tokens, K %% 16 == 0, N %% 8 == 0");
    ONELLM_REQUIRE((size_t)M * N <= c->max_elems, ONELLM_ERR_ARG, "p2p_gemm_allreduce_add: %d x %d elements exceed the %zu the communicator holds",
                   M, N, c->max_elems);
    ONELLM_REQUIRE(aligned16(x) && aligned16(W) && aligned16(resid) && (!bias || aligned16(bias)) && x != resid, ONELLM_ERR_ARG,
                   "p2p_gemm_allreduce_add: pointers must be 16-byte aligned and x must not be the residual");
    TpEpilogue tp = {};
    for (int r = 0; r < c->world; r++) tp.push[r] = c->recv_slot(c->mapped[r], which, c->rank);
    tp.mine = c->recv_slot(c->local, which, 0);
    for (int r = 0; r < c->world; r++) tp.final_push[r] = c->final_slot(c->mapped[r], which);
    tp.final_mine = c->final_slot(c->local, which);
    // one-shot moves (world - 1) tagged copies of the message per rank, two-shot 2 (world - 1) / world of one over
    // two hops: worth it for the 64-token messages of the 13B shape on 4 ranks (7.94 -> 7.58 ms per step) and more,
    // not for a batch of 8, and never on 2 ranks (the same bytes over two hops)
    tp.two_shot = (c->world > 2 || g_two_shot_bytes == 0) && (long long)(c->world - 1) * M * N * 4 >= g_two_shot_bytes ? 1 : 0;
    tp.slot_words = c->slot_words();
    P2pControl* ctl = static_cast<P2pControl*>(c->local);
    tp.counters = ctl->gemm_counters;
    tp.error = &ctl->error;
    tp.rank = c->rank;
    tp.world = c->world;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const cudaError_t e = skinny_kn_staged_dispatch((const __half*)x, (const __half*)W, nullptr, (__half*)resid, M, N, K, false, st,
                                                    (const __half*)resid, (const __half*)bias, -1.f, &tp);
    if (e == cudaErrorInvalidConfiguration) {
        // The exchange inside the projection needs every block of the launch resident at once (a block waits for the
        // block of the same index on its peers).  A shape whose plan does not fit one wave is refused by the launcher
        // before anything runs; the same sum is then taken in two kernels: the plain projection into this rank's send
        // buffer, and the stand-alone exchange.  The plan depends on the shape and the GPU model only, so every rank
        // takes the same branch.
        (void)cudaGetLastError();
        __half* send = static_cast<__half*>(onellm_p2p_send_buffer(h, which));
        ONELLM_CUDA(skinny_kn_staged_dispatch((const __half*)x, (const __half*)W, nullptr, send, M, N, K, false, st, nullptr, nullptr, -1.f,
                                              nullptr));
        return onellm_p2p_allreduce_add(h, dtype, which, resid, bias, M * N, N, stream);
    }
    ONELLM_CUDA(e);
    return ONELLM_OK;
}

extern "C" long long onellm_p2p_two_shot_bytes(long long bytes)
{
    const long long before = g_two_shot_bytes;
    if (bytes >= 0) g_two_shot_bytes = bytes;
    return before;
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

namespace onellm {
// device address of the communicator's error word, for callers that read it with their own copy
const int* p2p_error_word(onellm_p2p* h)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    return (c && c->local) ? &static_cast<P2pControl*>(c->local)->error : nullptr;
}
}  // namespace onellm

extern "C" void onellm_p2p_destroy(onellm_p2p* h)
{
    P2pComm* c = reinterpret_cast<P2pComm*>(h);
    if (!c) return;
    for (int r = 0; r < c->world; r++)
        if (r != c->rank && c->mapped[r]) cudaIpcCloseMemHandle(c->mapped[r]);
    if (c->local) cudaFree(c->local);
    delete c;
}
