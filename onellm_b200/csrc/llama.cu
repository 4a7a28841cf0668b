// LLaMA model class and generation loop on top of the kernel ABI (host side, C++).
//
// The reference leaves this part unwritten: src/models/llama/llama.h is empty and
// src/models/llama/llama.cpp:1-50 is a comment outline (embedding -> RMSNorm -> fused QKV ->
// RoPE + attention -> o_proj -> add-residual RMSNorm -> SwiGLU MLP -> ... -> LM head -> top-K
// sampling).  This file implements that outline for decode, sequencing the kernels in the
// order LlamaSelfDecoder::forward does (src/layers/decoder/self_decoder.cpp:15-78): one
// RMSNorm before layer 0, then per layer QKV projection, fused masked attention, output
// projection, fused add-residual RMSNorm, gate/up + SwiGLU, down projection, fused
// add-residual RMSNorm with the next layer's (or the final) gamma.
//
// Differences from that loop, on purpose:
//   - the residual stream is kept separate from the normalised activations (the reference
//     normalises decoder_input in place and then adds it back as "residual");
//   - the KV cache is addressed per layer, [L, B, Hkv, S, D] as the layers allocate it
//     (src/layers/attention/masked_self_attention.cpp:62-70 passes layer_id but the kernels
//     use offset 0);
//   - RoPE positions are 0-based in both phases (the decode kernel of the reference uses
//     `step` while the new row lands in slot step-1);
//   - `tok_embeddings` feeds the input embedding and `output` the LM head (the reference's
//     loader swaps them, src/weights/llama/llama_weights.cc:40-41).
//
// Weights use the reference's on-disk format: one headerless little-endian array per
// tensor, names as in src/weights/llama/llama_weights.cc:39-45 and
// src/weights/llama/layer_weights.cc:44-54.  Files may hold fp32 (the reference's type) or
// fp16; a missing or wrongly sized file is an error here, not a silent skip.
//
// Tensor parallelism: query/KV heads and FFN columns are sliced at load time; the partial
// o_proj and down_proj outputs are summed with ncclAllReduce on the model's stream.  NCCL is
// bound at run time with dlopen, so a single-GPU process needs no NCCL at all.
//
// A decode step is captured once per (row-bucket, mode) as a CUDA graph and replayed: the
// attention and sampling kernels read the step counter from device memory.
#include <dlfcn.h>
#include <math.h>
#include <nccl.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace onellm {

// ---- NCCL, bound lazily ---------------------------------------------------------------------
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok() const { return handle && CommInitRank && AllReduce && CommDestroy && GetUniqueId; }
};

static NcclApi& nccl_api()
{
    static NcclApi api;
    if (!api.handle) {
        // a library already loaded under this name (e.g. by torch) is reused by the loader
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) {
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
            api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
        }
    }
    return api;
}

// ---- small kernels of the model driver -------------------------------------------------------
// First kernel of every step, launched with a full stream dependency: everything after it sees
// the new step.
__global__ void advance_step_kernel(int* step) { *step += 1; }

// ids[b] = prompt[b * prompt_len + (*step - 1)]; launched with a full stream dependency
__global__ void gather_prompt_ids_kernel(const int* __restrict__ prompt, int prompt_len, const int* __restrict__ step,
                                         int* __restrict__ ids, int B)
{
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) ids[b] = prompt[(size_t)b * prompt_len + (*step - 1)];
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// w[i] = mean + std * N(0,1), counter-based (seed, tensor tag, index) so that any slice of a
// tensor can be generated independently: `row_stride`/`col0` describe the slice of a
// [rows, full_cols] tensor this buffer holds.
__global__ void init_normal_kernel(__half* __restrict__ w, size_t rows, size_t cols, size_t full_cols, size_t row0,
                                   size_t col0, uint64_t seed, uint64_t tag, float mean, float std)
{
    const size_t n = rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i % cols;
        const uint64_t gi = (row0 + r) * full_cols + col0 + c;
        const uint64_t h = splitmix64(seed * 0x100000001B3ull + tag * 0x9E3779B1ull + gi);
        const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0,1]
        const float u2 = (float)(uint32_t)((h >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        w[i] = __float2half_rn(mean + std * z);
    }
}

// W[k, :] *= gamma[k]: the RMSNorm in front of a projection, moved into the projection's weights
// (RMSNorm(x) . W = rsqrt(mean(x^2) + eps) * (x . diag(gamma) W)), product rounded once to fp16.
__global__ void fold_gamma_kernel(__half* __restrict__ w, const __half* __restrict__ gamma, size_t rows, size_t cols)
{
    const size_t n = rows * cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = __float2half_rn(__half2float(w[i]) * __half2float(gamma[i / cols]));
}

// dst [cols, rows] = src [rows, cols]^T, 32 x 32 tiles through shared memory
__global__ void transpose_half_kernel(__half* __restrict__ dst, const __half* __restrict__ src, int rows, int cols)
{
    __shared__ __half tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[i][threadIdx.x] = src[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][i];
    }
}

__global__ void fill_half_kernel(__half* w, size_t n, float v)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = __float2half_rn(v);
}

__global__ void half_to_float_kernel(const __half* in, float* out, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __half2float(in[i]);
}

// ---- the model ---------------------------------------------------------------------------------
struct LayerW {
    __half *attn_norm, *ffn_norm, *w_qkv, *wo, *w1, *w3, *w2, *b_qkv, *b_o;
};

enum StepMode { MODE_GATHER = 1, MODE_HEAD = 2 };

struct Llama {
    onellm_llama_config c;
    int Hl, Hkvl, Il, qkv_cols;  // per-rank slices
    char* arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<LayerW> layers;
    __half *tok_emb = nullptr, *out_w = nullptr, *out_norm = nullptr;
    __half *k_cache = nullptr, *v_cache = nullptr;
    size_t cache_layer_elems = 0;
    // activations
    int *d_ids = nullptr, *d_prompt = nullptr, *d_step = nullptr, *d_out_ids = nullptr, *d_seqlen = nullptr,
        *d_topk_id = nullptr, *d_bad_id = nullptr;
    // per sequence: cached length minus cur_len (<= 0; all zero unless the prompts had different lengths)
    int* d_step_off = nullptr;
    std::vector<int> seq_off;  // host copy
    unsigned char* d_finished = nullptr;
    float *d_topk_val = nullptr, *d_u = nullptr;
    uint32_t* d_skip = nullptr;  // the sampler's per-row skip-ahead table (sampling.cu)
    int skip_ok = 0;             // 1 once the table is built and has matched the direct draws
    __half *res = nullptr, *y = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr,
           *logits = nullptr;
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    onellm_p2p* p2p = nullptr;  // peer-memory all-reduce of the decode step (tensor parallel)
    bool p2p_connected = false;
    bool use_p2p = true;        // false: keep ncclAllReduce in the decode step although peer memory is connected
    int* h_comm_err = nullptr;  // pinned: the communicator's error word, copied out at every point the host waits anyway
    // state
    int batch = 0, cur_len = 0, prompt_cap = 0, graph_prompt_len = 0;
    int top_k = 1, literal_walk = 0;
    float temperature = 1.0f;
    bool weights_ready = false, use_graphs = true;
    int head_layout = ONELLM_W_NK;  // ONELLM_W_KN once finalize_weights has transposed the LM head
    cudaStream_t stream = nullptr;
    std::map<long, cudaGraphExec_t> graphs;
    ncclComm_t comm = nullptr;
    long launches = 0;  // kernels enqueued by this model (graph replays count their nodes)
    std::map<long, int> graph_nodes;
    std::map<long, int> warmed;  // keys whose first step already ran outside a capture
    // context-phase scratch for T prompt tokens, grown on demand (separate from the arena)
    char* pf_buf = nullptr;
    size_t pf_tokens = 0;
    bool prefill_by_decode = false;  // true: run the context phase one position at a time (reference path for tests)
    bool prefill_norm_kernels = false;  // true: keep the norm kernels in the context phase on one GPU too (comparison)
};

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// sampling.cu: the sampler's per-row skip-ahead table
size_t skip_table_words(int rows);
int build_skip_table(uint32_t* table, int rows, int* usable, cudaStream_t st);

struct Carver {
    char* base;
    size_t off = 0;
    template <typename T>
    T* take(size_t n)
    {
        off = align_up(off, 256);
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += n * sizeof(T);
        return p;
    }
};

// One pass computes the size (base == nullptr), the second hands out pointers.
static void carve(Llama& m, Carver& cv)
{
    const auto& c = m.c;
    const size_t h = c.hidden, D = c.head_size, B = c.max_batch, V = c.vocab_size;
    m.layers.resize(c.num_layers);
    for (auto& L : m.layers) {
        L.attn_norm = cv.take<__half>(h);
        L.ffn_norm = cv.take<__half>(h);
        L.w_qkv = cv.take<__half>(h * m.qkv_cols);
        L.wo = cv.take<__half>((size_t)m.Hl * D * h);
        L.w1 = cv.take<__half>(h * m.Il);
        L.w3 = cv.take<__half>(h * m.Il);
        L.w2 = cv.take<__half>((size_t)m.Il * h);
        L.b_qkv = c.attn_bias ? cv.take<__half>(m.qkv_cols) : nullptr;
        L.b_o = c.attn_bias ? cv.take<__half>(h) : nullptr;
    }
    m.tok_emb = cv.take<__half>(V * h);
    m.out_w = cv.take<__half>(V * h);
    m.out_norm = cv.take<__half>(h);
    m.cache_layer_elems = B * m.Hkvl * (size_t)c.max_seq_len * D;
    m.k_cache = cv.take<__half>(m.cache_layer_elems * c.num_layers);
    m.v_cache = cv.take<__half>(m.cache_layer_elems * c.num_layers);
    m.d_ids = cv.take<int>(B);
    m.prompt_cap = c.max_seq_len;
    m.d_prompt = cv.take<int>(B * (size_t)c.max_seq_len);
    m.d_step = cv.take<int>(4);
    m.d_step_off = cv.take<int>(B);
    m.d_out_ids = cv.take<int>(B);
    m.d_seqlen = cv.take<int>(B);
    m.d_topk_id = cv.take<int>(B * 64);
    m.d_bad_id = cv.take<int>(4);
    m.d_finished = cv.take<unsigned char>(B);
    m.d_topk_val = cv.take<float>(B * 64);
    m.d_u = cv.take<float>(B);
    m.d_skip = cv.take<uint32_t>(skip_table_words((int)B));
    m.res = cv.take<__half>(B * h);
    m.y = cv.take<__half>(B * h);
    m.qkv = cv.take<__half>(B * m.qkv_cols);
    m.attn = cv.take<__half>(B * (size_t)m.Hl * D);
    m.act = cv.take<__half>(B * (size_t)m.Il);
    m.logits = cv.take<__half>(B * V);
    m.attn_ws_bytes = onellm_decode_attn_workspace_bytes((int)B, m.Hl, (int)D, c.max_seq_len);
    m.attn_ws = cv.take<char>(m.attn_ws_bytes);
}

static int blocks_for(size_t n) { return (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096); }

const int* p2p_error_word(onellm_p2p* h);  // p2p_allreduce.cu
int embedding_launch(int dtype, const int* ids, void* out, void* out2, const void* table, int n_tokens, int hidden,
                     int vocab, int* bad_id_flag, bool pdl, cudaStream_t st);
// sampling.cu
int topk_sample_launch(const int* topk_id, const float* topk_val, int B, int K, float temperature, int rng_step,
                       const int* rng_step_dev, int vocab_size, int end_id, int literal_walk, int* output_id,
                       int* seqlen, unsigned char* finished, float* u_out, int* output_id2, bool early_seed,
                       const uint32_t* skip_table, cudaStream_t st);

#define RC(call)              \
    do {                      \
        int rc__ = (call);    \
        if (rc__) return rc__; \
    } while (0)

static int tp_allreduce(Llama& m, __half* buf, size_t n)
{
    if (m.c.tp_size <= 1) return ONELLM_OK;
    ONELLM_REQUIRE(m.comm, ONELLM_ERR_STATE, "llama: tp_size %d but no communicator (call onellm_llama_init_comm)",
                   m.c.tp_size);
    const ncclResult_t r = nccl_api().AllReduce(buf, buf, n, ncclHalf, ncclSum, m.comm, m.stream);
    ONELLM_REQUIRE(r == ncclSuccess, ONELLM_ERR_COMM, "ncclAllReduce: %s",
                   nccl_api().GetErrorString ? nccl_api().GetErrorString(r) : "error");
    note_launch();
    return ONELLM_OK;
}

// Tensor parallel over peer memory: a rank whose wait for a peer ran out (about a second of SM clocks) has set
// its communicator's error word and gone on with whatever its receive slot held, so its residual stream, and
// from there its sampled tokens and cache rows, may differ from the other ranks'.  The engine copies the word
// out wherever it waits for the stream anyway (queue_comm_check before the wait, comm_check after it) and
// turns a set word into ONELLM_ERR_COMM.
static int queue_comm_check(Llama& m)
{
    if (!m.p2p_connected || !m.h_comm_err) return ONELLM_OK;
    ONELLM_CUDA(cudaMemcpyAsync(m.h_comm_err, p2p_error_word(m.p2p), sizeof(int), cudaMemcpyDeviceToHost, m.stream));
    return ONELLM_OK;
}
static int comm_check(Llama& m, const char* where)
{
    if (!m.p2p_connected || !m.h_comm_err) return ONELLM_OK;
    ONELLM_REQUIRE(*m.h_comm_err == 0, ONELLM_ERR_COMM,
                   "%s: a wait for a tensor-parallel peer ran out (rank %d of %d); the ranks' results may have diverged since",
                   where, m.c.tp_rank, m.c.tp_size);
    return ONELLM_OK;
}

// Enqueues one decode step for m.batch sequences on m.stream.  `step_bound` sizes the
// attention grid; the real step is read from d_step on the device.
static int enqueue_step(Llama& m, int mode, int step_bound, int prompt_len)
{
    const auto& c = m.c;
    const int B = m.batch, h = c.hidden, D = c.head_size;
    cudaStream_t st = m.stream;
    void* sp = (void*)st;
    // The step counter advances first.  This kernel, the id gather and the embedding are
    // launched with full stream dependencies; every later kernel of the step may overlap its
    // predecessor's tail (programmatic dependent launch) and therefore starts after these.
    note_launch();
    (void)prefer_max_shared((const void*)advance_step_kernel);  // same L1 / shared-memory split as every kernel behind it
    (void)prefer_max_shared((const void*)gather_prompt_ids_kernel);
    advance_step_kernel<<<1, 1, 0, st>>>(m.d_step);
    if (mode & MODE_GATHER) {
        note_launch();
        gather_prompt_ids_kernel<<<(B + 127) / 128, 128, 0, st>>>(m.d_prompt, prompt_len, m.d_step, m.d_ids, B);
    }
    const long cs_b = (long)m.Hkvl * c.max_seq_len * D, cs_h = (long)c.max_seq_len * D, cs_s = D;
    const float scale = 1.0f / sqrtf((float)D);
    auto attention = [&](int l) -> int {
        const LayerW& L = m.layers[l];
        const __half* q = m.qkv;
        const __half* k = m.qkv + (size_t)m.Hl * D;
        const __half* v = m.qkv + (size_t)(m.Hl + m.Hkvl) * D;
        const __half* bq = L.b_qkv;
        const __half* bk = L.b_qkv ? L.b_qkv + (size_t)m.Hl * D : nullptr;
        const __half* bv = L.b_qkv ? L.b_qkv + (size_t)(m.Hl + m.Hkvl) * D : nullptr;
        return onellm_decode_attn_ragged(ONELLM_F16, q, k, v, m.qkv_cols, m.qkv_cols, m.qkv_cols, bq, bk, bv,
                                         m.k_cache + (size_t)l * m.cache_layer_elems, m.v_cache + (size_t)l * m.cache_layer_elems,
                                         cs_b, cs_h, cs_s, B, m.Hl, m.Hkvl, D, step_bound, m.d_step, m.d_step_off,
                                         step_bound - 1, c.rot_dim, c.rope_base, scale, m.attn, (long)m.Hl * D, m.attn_ws,
                                         m.attn_ws_bytes, sp);
    };
    const __half* head_in = m.y;
    if (c.tp_size == 1) {
        // Five kernels per layer, no norm kernels: the residual stream lives in m.res, each projection
        // that follows a norm reads it raw and scales by rsqrt(mean(x^2) + eps) on the way out (the
        // norm's gamma is already inside its weights), o_proj and down_proj add their result to it.
        RC(embedding_launch(ONELLM_F16, m.d_ids, m.res, nullptr, m.tok_emb, B, h, c.vocab_size, m.d_bad_id, false, st));
        for (int l = 0; l < c.num_layers; l++) {
            const LayerW& L = m.layers[l];
            RC(onellm_gemm_fused(ONELLM_F16, m.res, L.w_qkv, nullptr, m.qkv, B, m.qkv_cols, h, c.rms_eps, nullptr, nullptr, sp));
            RC(attention(l));
            RC(onellm_gemm_fused(ONELLM_F16, m.attn, L.wo, nullptr, m.res, B, h, m.Hl * D, -1.f, m.res, L.b_o, sp));
            RC(onellm_gemm_fused(ONELLM_F16, m.res, L.w1, L.w3, m.act, B, m.Il, h, c.rms_eps, nullptr, nullptr, sp));
            RC(onellm_gemm_fused(ONELLM_F16, m.act, L.w2, nullptr, m.res, B, h, m.Il, -1.f, m.res, nullptr, sp));
        }
        if (mode & MODE_HEAD) {
            RC(onellm_rmsnorm(ONELLM_F16, m.res, m.out_norm, c.rms_eps, B, h, sp));  // in place: the stream ends here
        }
        head_in = m.res;
    } else if (m.p2p_connected && m.use_p2p) {
        // tensor parallel over peer memory: o_proj and down_proj reduce over the ranks in their own epilogue
        // (every finished pair of elements is pushed to the peers and the peers' values gathered) and add
        // the sum, and the bias, into this rank's copy of the residual stream.  Five kernels per layer as on
        // one GPU: no all-reduce kernel, no norm kernels, no NCCL.
        RC(embedding_launch(ONELLM_F16, m.d_ids, m.res, nullptr, m.tok_emb, B, h, c.vocab_size, m.d_bad_id, false, st));
        for (int l = 0; l < c.num_layers; l++) {
            const LayerW& L = m.layers[l];
            RC(onellm_gemm_fused(ONELLM_F16, m.res, L.w_qkv, nullptr, m.qkv, B, m.qkv_cols, h, c.rms_eps, nullptr, nullptr, sp));
            RC(attention(l));
            RC(onellm_p2p_gemm_allreduce_add(m.p2p, ONELLM_F16, 0, m.attn, L.wo, m.res, L.b_o, B, h, m.Hl * D, sp));
            RC(onellm_gemm_fused(ONELLM_F16, m.res, L.w1, L.w3, m.act, B, m.Il, h, c.rms_eps, nullptr, nullptr, sp));
            RC(onellm_p2p_gemm_allreduce_add(m.p2p, ONELLM_F16, 1, m.act, L.w2, m.res, nullptr, B, h, m.Il, sp));
        }
        if (mode & MODE_HEAD) {
            RC(onellm_rmsnorm(ONELLM_F16, m.res, m.out_norm, c.rms_eps, B, h, sp));
        }
        head_in = m.res;
    } else {
        // tensor parallel over NCCL: partial sums of o_proj and down_proj are all-reduced before the residual
        // add, so the norm kernels stay (their per-layer gamma is all ones after finalize_weights)
        RC(embedding_launch(ONELLM_F16, m.d_ids, m.y, m.res, m.tok_emb, B, h, c.vocab_size, m.d_bad_id, false, st));
        RC(onellm_rmsnorm(ONELLM_F16, m.y, m.layers[0].attn_norm, c.rms_eps, B, h, sp));
        for (int l = 0; l < c.num_layers; l++) {
            const LayerW& L = m.layers[l];
            RC(onellm_gemm(ONELLM_F16, m.y, L.w_qkv, m.qkv, B, m.qkv_cols, h, ONELLM_W_KN, sp));
            RC(attention(l));
            RC(onellm_gemm(ONELLM_F16, m.attn, L.wo, m.y, B, h, m.Hl * D, ONELLM_W_KN, sp));
            RC(tp_allreduce(m, m.y, (size_t)B * h));
            RC(onellm_add_residual_rmsnorm(ONELLM_F16, m.res, m.y, L.b_o, L.ffn_norm, c.rms_eps, B, h, sp));
            RC(onellm_gemm_swiglu(ONELLM_F16, m.y, L.w1, L.w3, m.act, B, m.Il, h, sp));
            RC(onellm_gemm(ONELLM_F16, m.act, L.w2, m.y, B, h, m.Il, ONELLM_W_KN, sp));
            RC(tp_allreduce(m, m.y, (size_t)B * h));
            const __half* next_gamma = (l + 1 < c.num_layers) ? m.layers[l + 1].attn_norm : m.out_norm;
            RC(onellm_add_residual_rmsnorm(ONELLM_F16, m.res, m.y, nullptr, next_gamma, c.rms_eps, B, h, sp));
        }
    }
    if (mode & MODE_HEAD) {
        RC(onellm_gemm(ONELLM_F16, head_in, m.out_w, m.logits, B, c.vocab_size, h, m.head_layout, sp));
        RC(onellm_topk(ONELLM_F16, m.logits, B, c.vocab_size, m.top_k, m.d_topk_val, m.d_topk_id, 0, sp));
        RC(topk_sample_launch(m.d_topk_id, m.d_topk_val, B, m.top_k, m.temperature, 0, m.d_step, c.vocab_size,
                              c.eos_id, m.literal_walk, m.d_out_ids, m.d_seqlen, m.d_finished, m.d_u, m.d_ids, /*early_seed=*/true,
                              m.skip_ok ? m.d_skip : nullptr, st));
    }
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

static void drop_graphs(Llama& m)
{
    for (auto& kv : m.graphs) cudaGraphExecDestroy(kv.second);
    m.graphs.clear();
    m.graph_nodes.clear();
    m.warmed.clear();
}

// Runs one step (attending cur_len + 1 rows) and advances cur_len.
static int run_step(Llama& m, int mode, int prompt_len)
{
    const int step = m.cur_len + 1;
    ONELLM_REQUIRE(step <= m.c.max_seq_len, ONELLM_ERR_STATE, "llama: sequence length %d exceeds max_seq_len %d", step,
                   m.c.max_seq_len);
    int bound = (step + 255) / 256 * 256;
    if (bound > m.c.max_seq_len) bound = m.c.max_seq_len;
    if (!m.use_graphs) {
        const long before = launches_noted();
        RC(enqueue_step(m, mode, bound, prompt_len));
        m.launches += launches_noted() - before;
        m.cur_len++;
        return ONELLM_OK;
    }
    const long key = ((long)bound << 20) | ((long)m.batch << 8) | ((long)mode << 4) | (m.top_k > 1 ? 1 : 0);
    // prompt_len, top_k, temperature are baked into the captured nodes: changing them drops the cache
    auto it = m.graphs.find(key);
    if (it == m.graphs.end() && !m.warmed.count(key)) {
        // first step of this shape runs eagerly: the launch planners query occupancy and set
        // function attributes once per kernel, which must not happen inside a stream capture
        m.warmed[key] = 1;
        const long before = launches_noted();
        RC(enqueue_step(m, mode, bound, prompt_len));
        m.launches += launches_noted() - before;
        m.cur_len++;
        return ONELLM_OK;
    }
    if (it == m.graphs.end()) {
        const long before = launches_noted();  // what the capture records = the nodes of one replay
        cudaGraph_t g = nullptr;
        ONELLM_CUDA(cudaStreamBeginCapture(m.stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_step(m, mode, bound, prompt_len);
        const cudaError_t e = cudaStreamEndCapture(m.stream, &g);
        if (rc) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        ONELLM_REQUIRE(e == cudaSuccess && g, ONELLM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t ge = nullptr;
        const cudaError_t e2 = cudaGraphInstantiate(&ge, g, 0);
        cudaGraphDestroy(g);
        ONELLM_REQUIRE(e2 == cudaSuccess, ONELLM_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e2));
        m.graph_nodes[key] = (int)(launches_noted() - before);
        it = m.graphs.emplace(key, ge).first;
    }
    ONELLM_CUDA(cudaGraphLaunch(it->second, m.stream));
    m.launches += m.graph_nodes[key];
    m.cur_len++;
    return ONELLM_OK;
}

// row cu[b + 1] - 1 of the packed [T, h] activations -> row b of dst
__global__ void gather_last_rows_kernel(const __half* __restrict__ src, const int* __restrict__ cu, __half* __restrict__ dst, int h)
{
    const __half* s = src + (size_t)(cu[blockIdx.x + 1] - 1) * h;
    __half* d = dst + (size_t)blockIdx.x * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) d[i] = s[i];
}

// ---- context phase ------------------------------------------------------------------------------
// All prompt tokens of the batch at once: tensor-core projections (M = batch * prompt_len), the
// fused QKV bias + RoPE + cache write, causal attention over the cache, then the LM head on the
// last token of every sequence.  Same arithmetic as running the positions one by one through the
// decode kernels (which `prefill_by_decode` still does, for cross-checking).
// lens[b] new tokens of sequence b (packed in d_prompt in sequence order) behind the cur_len + seq_off[b] positions it
// has cached.
static int prefill_context(Llama& m, int B, const int* lens)
{
    const auto& c = m.c;
    const int h = c.hidden, D = c.head_size;
    size_t T = 0;
    int P = 0;
    for (int b = 0; b < B; b++) {
        T += (size_t)lens[b];
        P = lens[b] > P ? lens[b] : P;
    }
    cudaStream_t st = m.stream;
    void* sp = (void*)st;
    // scratch layout for T tokens
    const int ss_parts = onellm_gemm_rows_parts(h, 0);  // partial row sums written by the projections that end in the stream
    const size_t per_tok = ((size_t)2 * h + m.qkv_cols + (size_t)m.Hl * D + (size_t)m.Il) * sizeof(__half) +
                           ((size_t)2 * ss_parts + 1) * sizeof(float);
    if (T > m.pf_tokens) {
        ONELLM_CUDA(cudaStreamSynchronize(st));
        if (m.pf_buf) cudaFree(m.pf_buf);
        m.pf_buf = nullptr;
        m.pf_tokens = 0;
        const cudaError_t e = cudaMalloc(&m.pf_buf, T * per_tok + 10 * 256 + (size_t)(2 * c.max_batch + 2) * sizeof(int));
        ONELLM_REQUIRE(e == cudaSuccess, ONELLM_ERR_CUDA, "llama_prefill: cannot allocate context scratch for %zu tokens: %s", T,
                       cudaGetErrorString(e));
        m.pf_tokens = T;
    }
    Carver cv{m.pf_buf};
    __half* y = cv.take<__half>(T * h);
    __half* res = cv.take<__half>(T * h);
    __half* qkv = cv.take<__half>(T * m.qkv_cols);
    __half* attn = cv.take<__half>(T * (size_t)m.Hl * D);
    __half* act = cv.take<__half>(T * (size_t)m.Il);
    float* ss0 = cv.take<float>(T);
    float* ss_a = cv.take<float>(T * ss_parts);
    float* ss_b = cv.take<float>(T * ss_parts);
    int* d_cu = cv.take<int>(c.max_batch + 1);
    int* d_hist = cv.take<int>(c.max_batch);
    std::vector<int> cu(B + 1, 0), hist(B), off(B);
    m.seq_off.resize(c.max_batch, 0);
    for (int b = 0; b < B; b++) hist[b] = m.cur_len + m.seq_off[b];
    int new_max = 0;
    for (int b = 0; b < B; b++) {
        cu[b + 1] = cu[b] + lens[b];
        new_max = hist[b] + lens[b] > new_max ? hist[b] + lens[b] : new_max;
    }
    for (int b = 0; b < B; b++) off[b] = hist[b] + lens[b] - new_max;
    ONELLM_CUDA(cudaMemcpyAsync(m.d_step_off, off.data(), B * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(d_cu, cu.data(), (B + 1) * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(d_hist, hist.data(), B * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaStreamSynchronize(st));  // cu / hist / off live on this stack frame

    const long launches_before = launches_noted();
    const long cs_b = (long)m.Hkvl * c.max_seq_len * D, cs_h = (long)c.max_seq_len * D, cs_s = D;
    const float scale = 1.0f / sqrtf((float)D);
    const bool norm_free = c.tp_size == 1 && !m.prefill_norm_kernels;
    if (norm_free) {
        // One GPU: no norm kernels, as in the decode step.  The residual stream lives in `res`; a projection behind a
        // norm reads it raw and scales its rows by rsqrt(mean(x^2) + eps) on the way out (the gammas are inside the
        // weights), o_proj and down_proj add their result to the stream in their epilogue and leave, per column tile,
        // the sum of squares of what they stored: the row statistics of the next projection.
        RC(embedding_launch(ONELLM_F16, m.d_prompt, res, nullptr, m.tok_emb, (int)T, h, c.vocab_size, m.d_bad_id, false, st));
        RC(onellm_row_sumsq(ONELLM_F16, res, (int)T, h, ss0, sp));
        for (int l = 0; l < c.num_layers; l++) {
            const LayerW& L = m.layers[l];
            __half* kc = m.k_cache + (size_t)l * m.cache_layer_elems;
            __half* vc = m.v_cache + (size_t)l * m.cache_layer_elems;
            RC(onellm_gemm_rows(ONELLM_F16, res, L.w_qkv, nullptr, qkv, (int)T, m.qkv_cols, h, l == 0 ? ss0 : ss_a, l == 0 ? 1 : ss_parts,
                                c.rms_eps, nullptr, nullptr, nullptr, sp));
            RC(onellm_qkv_bias_rope_kvcache(ONELLM_F16, qkv, L.b_qkv, d_cu, d_hist, kc, vc, cs_b, cs_h, cs_s, (int)T, B, m.Hl, m.Hkvl,
                                            D, c.rot_dim, c.rope_base, c.max_seq_len, m.d_bad_id + 1, sp));
            RC(onellm_context_attn(ONELLM_F16, qkv, m.qkv_cols, kc, vc, cs_b, cs_h, cs_s, d_cu, d_hist, B, P, m.Hl, m.Hkvl, D, scale,
                                   attn, sp));
            RC(onellm_gemm_rows(ONELLM_F16, attn, L.wo, nullptr, res, (int)T, h, m.Hl * D, nullptr, 0, c.rms_eps, res, L.b_o, ss_b, sp));
            RC(onellm_gemm_rows(ONELLM_F16, res, L.w1, L.w3, act, (int)T, m.Il, h, ss_b, ss_parts, c.rms_eps, nullptr, nullptr, nullptr, sp));
            RC(onellm_gemm_rows(ONELLM_F16, act, L.w2, nullptr, res, (int)T, h, m.Il, nullptr, 0, c.rms_eps, res, nullptr, ss_a, sp));
        }
        // last position of every sequence: the final norm (not folded), LM head, top-K, sampling
        note_launch();
        gather_last_rows_kernel<<<B, 256, 0, st>>>(res, d_cu, m.y, h);
        RC(onellm_rmsnorm(ONELLM_F16, m.y, m.out_norm, c.rms_eps, B, h, sp));
    } else {
    // d_prompt holds the new tokens packed in sequence order
    RC(embedding_launch(ONELLM_F16, m.d_prompt, y, res, m.tok_emb, (int)T, h, c.vocab_size, m.d_bad_id, false, st));
    RC(onellm_rmsnorm(ONELLM_F16, y, m.layers[0].attn_norm, c.rms_eps, (int)T, h, sp));
    for (int l = 0; l < c.num_layers; l++) {
        const LayerW& L = m.layers[l];
        __half* kc = m.k_cache + (size_t)l * m.cache_layer_elems;
        __half* vc = m.v_cache + (size_t)l * m.cache_layer_elems;
        RC(onellm_gemm(ONELLM_F16, y, L.w_qkv, qkv, (int)T, m.qkv_cols, h, ONELLM_W_KN, sp));
        RC(onellm_qkv_bias_rope_kvcache(ONELLM_F16, qkv, L.b_qkv, d_cu, d_hist, kc, vc, cs_b, cs_h, cs_s, (int)T, B, m.Hl, m.Hkvl,
                                        D, c.rot_dim, c.rope_base, c.max_seq_len, m.d_bad_id + 1, sp));
        RC(onellm_context_attn(ONELLM_F16, qkv, m.qkv_cols, kc, vc, cs_b, cs_h, cs_s, d_cu, d_hist, B, P, m.Hl, m.Hkvl, D, scale,
                               attn, sp));
        RC(onellm_gemm(ONELLM_F16, attn, L.wo, y, (int)T, h, m.Hl * D, ONELLM_W_KN, sp));
        RC(tp_allreduce(m, y, T * h));
        RC(onellm_add_residual_rmsnorm(ONELLM_F16, res, y, L.b_o, L.ffn_norm, c.rms_eps, (int)T, h, sp));
        RC(onellm_gemm_swiglu(ONELLM_F16, y, L.w1, L.w3, act, (int)T, m.Il, h, sp));  // SwiGLU in the epilogue at every M
        RC(onellm_gemm(ONELLM_F16, act, L.w2, y, (int)T, h, m.Il, ONELLM_W_KN, sp));
        RC(tp_allreduce(m, y, T * h));
        const __half* next_gamma = (l + 1 < c.num_layers) ? m.layers[l + 1].attn_norm : m.out_norm;
        RC(onellm_add_residual_rmsnorm(ONELLM_F16, res, y, nullptr, next_gamma, c.rms_eps, (int)T, h, sp));
    }
    // last position of every sequence -> LM head, top-K, sampling (seeded with the step counter, as the
    // position-by-position path does)
    note_launch();
    gather_last_rows_kernel<<<B, 256, 0, st>>>(y, d_cu, m.y, h);
    }
    RC(onellm_gemm(ONELLM_F16, m.y, m.out_w, m.logits, B, c.vocab_size, h, m.head_layout, sp));
    RC(onellm_topk(ONELLM_F16, m.logits, B, c.vocab_size, m.top_k, m.d_topk_val, m.d_topk_id, 0, sp));
    RC(topk_sample_launch(m.d_topk_id, m.d_topk_val, B, m.top_k, m.temperature, 0, m.d_step, c.vocab_size, c.eos_id,
                          m.literal_walk, m.d_out_ids, m.d_seqlen, m.d_finished, m.d_u, m.d_ids, /*early_seed=*/true,
                          m.skip_ok ? m.d_skip : nullptr, st));
    m.launches += launches_noted() - launches_before;
    for (int b = 0; b < B; b++) m.seq_off[b] = off[b];
    m.cur_len = new_max;
    return ONELLM_OK;
}

// ---- weight files ------------------------------------------------------------------------------
// Reads a [rows, cols] tensor (fp32 or fp16 on disk, told apart by the file size), keeps the
// slice rows [r0, r0+nr) x cols [c0, c0+nc), converts to fp16 and uploads it.
static int load_slice(const std::string& file, size_t rows, size_t cols, size_t r0, size_t nr, size_t c0, size_t nc,
                      __half* dst)
{
    FILE* f = fopen(file.c_str(), "rb");
    ONELLM_REQUIRE(f, ONELLM_ERR_IO, "cannot open weight file %s", file.c_str());
    fseek(f, 0, SEEK_END);
    const size_t bytes = (size_t)ftell(f);
    fseek(f, 0, SEEK_SET);
    const size_t n = rows * cols;
    if (bytes != n * 4 && bytes != n * 2) {
        fclose(f);
        set_error("weight file %s has %zu bytes, expected %zu (fp32) or %zu (fp16)", file.c_str(), bytes, n * 4, n * 2);
        return ONELLM_ERR_IO;
    }
    const bool f32 = bytes == n * 4;
    std::vector<char> raw(bytes);
    const size_t got = fread(raw.data(), 1, bytes, f);
    fclose(f);
    ONELLM_REQUIRE(got == bytes, ONELLM_ERR_IO, "short read on %s", file.c_str());
    std::vector<__half> out(nr * nc);
    for (size_t r = 0; r < nr; r++)
        for (size_t cc = 0; cc < nc; cc++) {
            const size_t i = (r0 + r) * cols + c0 + cc;
            out[r * nc + cc] =
                f32 ? __float2half_rn(reinterpret_cast<const float*>(raw.data())[i]) : reinterpret_cast<const __half*>(raw.data())[i];
        }
    ONELLM_CUDA(cudaMemcpy(dst, out.data(), out.size() * sizeof(__half), cudaMemcpyHostToDevice));
    return ONELLM_OK;
}

// The fused QKV weight [h, (H+2Hkv)D] is sliced per head group: this rank keeps its query
// heads, its key heads and its value heads, packed as [h, (Hl+2Hkvl)D].
static int load_qkv(Llama& m, const std::string& file, size_t rows, __half* dst)
{
    const auto& c = m.c;
    const size_t D = c.head_size, full = (size_t)(c.head_num + 2 * c.kv_head_num) * D;
    std::vector<__half> tmp;
    __half* stage = nullptr;
    ONELLM_CUDA(cudaMalloc(&stage, rows * full * sizeof(__half)));
    int rc = load_slice(file, rows, full, 0, rows, 0, full, stage);
    if (rc == ONELLM_OK) {
        const size_t qc = (size_t)m.Hl * D, kc = (size_t)m.Hkvl * D;
        const size_t src_col[3] = {(size_t)c.tp_rank * qc, (size_t)c.head_num * D + c.tp_rank * kc,
                                   (size_t)(c.head_num + c.kv_head_num) * D + c.tp_rank * kc};
        const size_t width[3] = {qc, kc, kc};
        size_t dcol = 0;
        for (int part = 0; part < 3 && rc == ONELLM_OK; part++) {
            const cudaError_t e = cudaMemcpy2D(dst + dcol, (size_t)m.qkv_cols * sizeof(__half), stage + src_col[part],
                                               full * sizeof(__half), width[part] * sizeof(__half), rows,
                                               cudaMemcpyDeviceToDevice);
            if (e != cudaSuccess) {
                set_error("cudaMemcpy2D: %s", cudaGetErrorString(e));
                rc = ONELLM_ERR_CUDA;
            }
            dcol += width[part];
        }
    }
    cudaFree(stage);
    return rc;
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_llama_create(const onellm_llama_config* cfg, onellm_llama** out)
{
    ONELLM_REQUIRE(cfg && out, ONELLM_ERR_ARG, "llama_create: null pointer");
    const auto& c = *cfg;
    ONELLM_REQUIRE(c.num_layers > 0 && c.hidden > 0 && c.head_num > 0 && c.kv_head_num > 0 && c.head_size > 0 &&
                       c.inter_size > 0 && c.vocab_size > 0 && c.max_seq_len > 0 && c.max_batch > 0,
                   ONELLM_ERR_ARG, "llama_create: non-positive dimension");
    ONELLM_REQUIRE(c.hidden == c.head_num * c.head_size, ONELLM_ERR_ARG, "llama_create: hidden != head_num*head_size");
    ONELLM_REQUIRE(c.head_num % c.kv_head_num == 0, ONELLM_ERR_ARG, "llama_create: head_num %% kv_head_num != 0");
    ONELLM_REQUIRE(c.tp_size >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_size, ONELLM_ERR_ARG, "llama_create: bad tp rank/size");
    ONELLM_REQUIRE(c.head_num % c.tp_size == 0 && c.kv_head_num % c.tp_size == 0 && c.inter_size % c.tp_size == 0,
                   ONELLM_ERR_UNSUPPORTED, "llama_create: heads / inter_size do not divide by tp_size %d", c.tp_size);
    ONELLM_REQUIRE((c.inter_size / c.tp_size) % 16 == 0 && c.hidden % 32 == 0, ONELLM_ERR_UNSUPPORTED,
                   "llama_create: hidden must be a multiple of 32 and the per-rank inter_size of 16");
    ONELLM_REQUIRE(c.head_size * 2 == 64 || c.head_size * 2 == 128 || c.head_size * 2 == 256 || c.head_size * 2 == 512,
                   ONELLM_ERR_UNSUPPORTED, "llama_create: head_size %d", c.head_size);
    ONELLM_REQUIRE(c.max_batch <= 64, ONELLM_ERR_UNSUPPORTED, "llama_create: max_batch %d > 64", c.max_batch);
    Llama* m = new Llama();
    m->c = c;
    if (m->c.rot_dim <= 0) m->c.rot_dim = c.head_size;
    if (m->c.rope_base <= 0.f) m->c.rope_base = 10000.f;
    if (m->c.rms_eps <= 0.f) m->c.rms_eps = 1e-5f;
    m->Hl = c.head_num / c.tp_size;
    m->Hkvl = c.kv_head_num / c.tp_size;
    m->Il = c.inter_size / c.tp_size;
    m->qkv_cols = (m->Hl + 2 * m->Hkvl) * c.head_size;
    Carver sizing{nullptr};
    carve(*m, sizing);
    m->arena_bytes = align_up(sizing.off, 256);
    cudaError_t e = cudaMalloc(&m->arena, m->arena_bytes);
    if (e != cudaSuccess) {
        set_error("llama_create: cudaMalloc of %zu bytes failed: %s", m->arena_bytes, cudaGetErrorString(e));
        delete m;
        return ONELLM_ERR_CUDA;
    }
    Carver real{m->arena};
    carve(*m, real);
    e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMemsetAsync(m->d_step, 0, 4 * sizeof(int), m->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(m->d_bad_id, 0, 4 * sizeof(int), m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (e == cudaSuccess && build_skip_table(m->d_skip, m->c.max_batch, &m->skip_ok, m->stream) != ONELLM_OK)
        e = cudaErrorUnknown;  // the text is already in the error slot
    if (e != cudaSuccess) {
        if (e != cudaErrorUnknown) set_error("llama_create: %s", cudaGetErrorString(e));
        if (m->stream) cudaStreamDestroy(m->stream);
        cudaFree(m->arena);
        delete m;
        return ONELLM_ERR_CUDA;
    }
    *out = reinterpret_cast<onellm_llama*>(m);
    return ONELLM_OK;
}

extern "C" int onellm_llama_last_draws(onellm_llama* h, float* host_u, int* host_step, int* table_in_use)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_u, ONELLM_ERR_ARG, "llama_last_draws: null pointer");
    ONELLM_CUDA(cudaMemcpyAsync(host_u, m->d_u, (size_t)m->c.max_batch * sizeof(float), cudaMemcpyDeviceToHost,
                                m->stream));
    int step = 0;
    ONELLM_CUDA(cudaMemcpyAsync(&step, m->d_step, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    ONELLM_CUDA(cudaStreamSynchronize(m->stream));
    if (host_step) *host_step = step;
    if (table_in_use) *table_in_use = m->skip_ok;
    return ONELLM_OK;
}

extern "C" void onellm_llama_destroy(onellm_llama* h)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    if (!m) return;
    cudaStreamSynchronize(m->stream);
    drop_graphs(*m);
    if (m->comm && nccl_api().CommDestroy) nccl_api().CommDestroy(m->comm);
    if (m->p2p) onellm_p2p_destroy(m->p2p);
    if (m->stream) cudaStreamDestroy(m->stream);
    cudaFree(m->arena);
    if (m->pf_buf) cudaFree(m->pf_buf);
    if (m->h_comm_err) cudaFreeHost(m->h_comm_err);
    delete m;
}

extern "C" int onellm_llama_set_prefill_by_decode(onellm_llama* h, int enabled)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_set_prefill_by_decode: null handle");
    m->prefill_by_decode = enabled == 1;
    m->prefill_norm_kernels = enabled == 2;
    return ONELLM_OK;
}

extern "C" size_t onellm_llama_device_bytes(const onellm_llama* h)
{
    return h ? reinterpret_cast<const Llama*>(h)->arena_bytes : 0;
}

extern "C" void* onellm_llama_stream(onellm_llama* h) { return h ? (void*)reinterpret_cast<Llama*>(h)->stream : nullptr; }

extern "C" int onellm_nccl_unique_id(void* id128)
{
    ONELLM_REQUIRE(id128, ONELLM_ERR_ARG, "nccl_unique_id: null pointer");
    ONELLM_REQUIRE(nccl_api().ok(), ONELLM_ERR_COMM, "NCCL library not found (libnccl.so.2)");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    const ncclResult_t r = nccl_api().GetUniqueId(&id);
    ONELLM_REQUIRE(r == ncclSuccess, ONELLM_ERR_COMM, "ncclGetUniqueId failed");
    memcpy(id128, &id, 128);
    return ONELLM_OK;
}

extern "C" int onellm_llama_init_comm(onellm_llama* h, const void* id128)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && id128, ONELLM_ERR_ARG, "llama_init_comm: null pointer");
    if (m->c.tp_size == 1) return ONELLM_OK;
    ONELLM_REQUIRE(nccl_api().ok(), ONELLM_ERR_COMM, "NCCL library not found (libnccl.so.2)");
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    const ncclResult_t r = nccl_api().CommInitRank(&m->comm, m->c.tp_size, id, m->c.tp_rank);
    ONELLM_REQUIRE(r == ncclSuccess, ONELLM_ERR_COMM, "ncclCommInitRank: %s",
                   nccl_api().GetErrorString ? nccl_api().GetErrorString(r) : "error");
    return ONELLM_OK;
}

// After the weights are in place: every layer's two norm vectors are multiplied into the rows of the
// projections that follow them (QKV; gate and up) and replaced by ones.  The decode step then needs no
// norm kernel between projections (onellm_gemm_fused scales by the row statistics on the way out), and
// the paths that still run the norm kernels (context phase, tensor parallel) compute x / rms(x) with the
// all-ones vectors in front of the same folded weights.  The final norm in front of the LM head stays.
static int finalize_weights(Llama& m)
{
    const auto& c = m.c;
    cudaStream_t st = m.stream;
    const size_t hd = c.hidden;
    for (auto& L : m.layers) {
        fold_gamma_kernel<<<blocks_for(hd * m.qkv_cols), 256, 0, st>>>(L.w_qkv, L.attn_norm, hd, (size_t)m.qkv_cols);
        fold_gamma_kernel<<<blocks_for(hd * m.Il), 256, 0, st>>>(L.w1, L.ffn_norm, hd, (size_t)m.Il);
        fold_gamma_kernel<<<blocks_for(hd * m.Il), 256, 0, st>>>(L.w3, L.ffn_norm, hd, (size_t)m.Il);
        fill_half_kernel<<<blocks_for(hd), 256, 0, st>>>(L.attn_norm, hd, 1.0f);
        fill_half_kernel<<<blocks_for(hd), 256, 0, st>>>(L.ffn_norm, hd, 1.0f);
    }
    // The LM head arrives as output.weight [vocab, hidden]; it is kept as [hidden, vocab], the orientation of every
    // other projection, so that the decode step streams it with the same staged kernel (5.5 TB/s against the
    // 3.7 TB/s of the register-fed kernel for [N, K] weights) and the context phase uses the MN-major tile path.
    m.head_layout = ONELLM_W_NK;
    if (c.vocab_size % 8 == 0) {  // the [K, N] kernels need 16-byte rows
        const size_t V = c.vocab_size;
        __half* tmp = nullptr;
        ONELLM_CUDA(cudaMalloc(&tmp, V * hd * sizeof(__half)));
        const dim3 grid((unsigned)((hd + 31) / 32), (unsigned)((V + 31) / 32));
        transpose_half_kernel<<<grid, dim3(32, 8), 0, st>>>(tmp, m.out_w, (int)V, (int)hd);
        const cudaError_t e1 = cudaMemcpyAsync(m.out_w, tmp, V * hd * sizeof(__half), cudaMemcpyDeviceToDevice, st);
        const cudaError_t e2 = cudaStreamSynchronize(st);
        cudaFree(tmp);
        ONELLM_CUDA(e1);
        ONELLM_CUDA(e2);
        m.head_layout = ONELLM_W_KN;
    }
    ONELLM_CHECK_LAUNCH();
    ONELLM_CUDA(cudaStreamSynchronize(st));
    m.weights_ready = true;
    return ONELLM_OK;
}

extern "C" int onellm_llama_init_random(onellm_llama* h, uint64_t seed, float std)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_init_random: null handle");
    const auto& c = m->c;
    const size_t hd = c.hidden, D = c.head_size, V = c.vocab_size;
    cudaStream_t st = m->stream;
    auto normal = [&](__half* w, size_t rows, size_t cols, size_t full_cols, size_t row0, size_t col0, uint64_t tag) {
        init_normal_kernel<<<blocks_for(rows * cols), 256, 0, st>>>(w, rows, cols, full_cols, row0, col0, seed, tag, 0.f, std);
    };
    auto ones = [&](__half* w, size_t n) { fill_half_kernel<<<blocks_for(n), 256, 0, st>>>(w, n, 1.0f); };
    const size_t full_qkv = (size_t)(c.head_num + 2 * c.kv_head_num) * D;
    const size_t qc = (size_t)m->Hl * D, kc = (size_t)m->Hkvl * D;
    for (int l = 0; l < c.num_layers; l++) {
        LayerW& L = m->layers[l];
        const uint64_t t0 = (uint64_t)l * 16;
        ones(L.attn_norm, hd);
        ones(L.ffn_norm, hd);
        // the three head groups of the fused QKV weight, each generated at its place in the
        // full tensor so that every TP degree sees the same model
        {
            // rows are [h]; columns of the packed local tensor map to three ranges of the full one
            const size_t src_col[3] = {(size_t)c.tp_rank * qc, (size_t)c.head_num * D + c.tp_rank * kc,
                                       (size_t)(c.head_num + c.kv_head_num) * D + c.tp_rank * kc};
            const size_t width[3] = {qc, kc, kc};
            // generate into a dense staging view per part, then place with a 2D copy
            __half* stage = nullptr;
            ONELLM_CUDA(cudaMallocAsync(&stage, hd * qc * sizeof(__half), st));
            size_t dcol = 0;
            for (int part = 0; part < 3; part++) {
                normal(stage, hd, width[part], full_qkv, 0, src_col[part], t0 + 0);
                ONELLM_CUDA(cudaMemcpy2DAsync(L.w_qkv + dcol, (size_t)m->qkv_cols * sizeof(__half), stage,
                                              width[part] * sizeof(__half), width[part] * sizeof(__half), hd,
                                              cudaMemcpyDeviceToDevice, st));
                dcol += width[part];
            }
            ONELLM_CUDA(cudaFreeAsync(stage, st));
        }
        normal(L.wo, qc, hd, hd, (size_t)c.tp_rank * qc, 0, t0 + 1);
        normal(L.w1, hd, m->Il, c.inter_size, 0, (size_t)c.tp_rank * m->Il, t0 + 2);
        normal(L.w3, hd, m->Il, c.inter_size, 0, (size_t)c.tp_rank * m->Il, t0 + 3);
        normal(L.w2, m->Il, hd, hd, (size_t)c.tp_rank * m->Il, 0, t0 + 4);
        if (L.b_qkv) ONELLM_CUDA(cudaMemsetAsync(L.b_qkv, 0, (size_t)m->qkv_cols * sizeof(__half), st));
        if (L.b_o) ONELLM_CUDA(cudaMemsetAsync(L.b_o, 0, hd * sizeof(__half), st));
    }
    normal(m->tok_emb, V, hd, hd, 0, 0, 1000001);
    normal(m->out_w, V, hd, hd, 0, 0, 1000002);
    ones(m->out_norm, hd);
    ONELLM_CHECK_LAUNCH();
    return finalize_weights(*m);
}

extern "C" int onellm_llama_load_weights(onellm_llama* h, const char* weight_path)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && weight_path, ONELLM_ERR_ARG, "llama_load_weights: null pointer");
    const auto& c = m->c;
    const std::string p(weight_path);
    const size_t hd = c.hidden, D = c.head_size, V = c.vocab_size, I = c.inter_size;
    const size_t qc = (size_t)m->Hl * D;
    RC(load_slice(p + ".norm.weight", 1, hd, 0, 1, 0, hd, m->out_norm));
    RC(load_slice(p + ".tok_embeddings.weight", V, hd, 0, V, 0, hd, m->tok_emb));
    RC(load_slice(p + ".output.weight", V, hd, 0, V, 0, hd, m->out_w));
    for (int l = 0; l < c.num_layers; l++) {
        LayerW& L = m->layers[l];
        const std::string lp = p + "layers." + std::to_string(l);
        RC(load_slice(lp + ".attention_norm.weight", 1, hd, 0, 1, 0, hd, L.attn_norm));
        RC(load_slice(lp + ".ffn_norm.weight", 1, hd, 0, 1, 0, hd, L.ffn_norm));
        RC(load_qkv(*m, lp + ".attention.w_qkv.weight", hd, L.w_qkv));
        RC(load_slice(lp + ".attention.wo.weight", hd, hd, (size_t)c.tp_rank * qc, qc, 0, hd, L.wo));
        RC(load_slice(lp + ".feed_forward.w1.weight", hd, I, 0, hd, (size_t)c.tp_rank * m->Il, m->Il, L.w1));
        RC(load_slice(lp + ".feed_forward.w3.weight", hd, I, 0, hd, (size_t)c.tp_rank * m->Il, m->Il, L.w3));
        RC(load_slice(lp + ".feed_forward.w2.weight", I, hd, (size_t)c.tp_rank * m->Il, m->Il, 0, hd, L.w2));
        if (c.attn_bias) {
            RC(load_qkv(*m, lp + ".attention.w_qkv.bias", 1, L.b_qkv));
            RC(load_slice(lp + ".attention.wo.bias", 1, hd, 0, 1, 0, hd, L.b_o));
        }
    }
    return finalize_weights(*m);
}

extern "C" int onellm_llama_set_sampling(onellm_llama* h, int top_k, float temperature, int literal_walk)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_set_sampling: null handle");
    ONELLM_REQUIRE(top_k >= 1 && top_k <= 64 && temperature > 0.f, ONELLM_ERR_ARG, "llama_set_sampling: top_k in [1,64], temperature > 0");
    if (top_k != m->top_k || temperature != m->temperature || literal_walk != m->literal_walk) {
        cudaStreamSynchronize(m->stream);
        drop_graphs(*m);
    }
    m->top_k = top_k;
    m->temperature = temperature;
    m->literal_walk = literal_walk;
    return ONELLM_OK;
}

extern "C" int onellm_llama_p2p_handle(onellm_llama* h, void* handle64)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && handle64, ONELLM_ERR_ARG, "llama_p2p_handle: null pointer");
    ONELLM_REQUIRE(m->c.tp_size > 1, ONELLM_ERR_STATE, "llama_p2p_handle: tp_size is 1");
    if (!m->p2p) {
        const size_t elems = ((size_t)m->c.max_batch * m->c.hidden + 7) / 8 * 8;
        RC(onellm_p2p_create(m->c.tp_rank, m->c.tp_size, elems, &m->p2p));
    }
    return onellm_p2p_handle(m->p2p, handle64);
}

extern "C" int onellm_llama_p2p_connect(onellm_llama* h, const void* handles)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && handles, ONELLM_ERR_ARG, "llama_p2p_connect: null pointer");
    ONELLM_REQUIRE(m->p2p, ONELLM_ERR_STATE, "llama_p2p_connect: call onellm_llama_p2p_handle first");
    RC(onellm_p2p_connect(m->p2p, handles));
    if (!m->h_comm_err) {
        ONELLM_CUDA(cudaMallocHost(&m->h_comm_err, sizeof(int)));
        *m->h_comm_err = 0;
    }
    ONELLM_CUDA(cudaStreamSynchronize(m->stream));
    drop_graphs(*m);
    m->p2p_connected = true;
    return ONELLM_OK;
}

extern "C" int onellm_llama_p2p_error(onellm_llama* h)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    return (m && m->p2p) ? onellm_p2p_error(m->p2p) : 0;
}

extern "C" int onellm_llama_set_tp_exchange(onellm_llama* h, int peer_memory)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_set_tp_exchange: null handle");
    ONELLM_REQUIRE(!peer_memory || m->c.tp_size == 1 || m->p2p_connected, ONELLM_ERR_STATE,
                   "llama_set_tp_exchange: peer memory is not connected (call onellm_llama_p2p_connect first)");
    if ((peer_memory != 0) != m->use_p2p) {
        ONELLM_CUDA(cudaStreamSynchronize(m->stream));
        drop_graphs(*m);  // the exchange is part of the captured step
    }
    m->use_p2p = peer_memory != 0;
    return ONELLM_OK;
}

extern "C" int onellm_llama_set_graphs(onellm_llama* h, int enabled)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_set_graphs: null handle");
    m->use_graphs = enabled != 0;
    return ONELLM_OK;
}

extern "C" int onellm_llama_prefill(onellm_llama* h, const int* host_ids, int batch, int prompt_len, int* host_first_ids)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_ids, ONELLM_ERR_ARG, "llama_prefill: null pointer");
    ONELLM_REQUIRE(m->weights_ready, ONELLM_ERR_STATE, "llama_prefill: weights not loaded");
    ONELLM_REQUIRE(batch >= 1 && batch <= m->c.max_batch, ONELLM_ERR_ARG, "llama_prefill: batch %d outside [1,%d]", batch, m->c.max_batch);
    ONELLM_REQUIRE(prompt_len >= 1 && prompt_len <= m->c.max_seq_len, ONELLM_ERR_ARG, "llama_prefill: prompt_len %d outside [1,%d]", prompt_len, m->c.max_seq_len);
    cudaStream_t st = m->stream;
    if (batch != m->batch || prompt_len != m->graph_prompt_len) {
        // batch and prompt length are baked into the captured launches
        ONELLM_CUDA(cudaStreamSynchronize(st));
        drop_graphs(*m);
    }
    m->batch = batch;
    m->graph_prompt_len = prompt_len;
    m->cur_len = 0;
    m->seq_off.assign(m->c.max_batch, 0);
    ONELLM_CUDA(cudaMemsetAsync(m->d_step_off, 0, (size_t)m->c.max_batch * sizeof(int), st));
    const int first_step = m->prefill_by_decode ? 0 : prompt_len;  // the step kernels increment before use
    ONELLM_CUDA(cudaMemcpyAsync(m->d_prompt, host_ids, (size_t)batch * prompt_len * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(m->d_step, &first_step, sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_seqlen, 0, (size_t)batch * sizeof(int), st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_finished, 0, (size_t)batch, st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_bad_id, 0, 4 * sizeof(int), st));
    ONELLM_CUDA(cudaStreamSynchronize(st));  // `first_step` lives on this stack frame
    if (m->prefill_by_decode) {
        // one position at a time through the decode kernels; only the last position needs the LM head
        for (int p = 0; p < prompt_len; p++)
            RC(run_step(*m, MODE_GATHER | (p == prompt_len - 1 ? MODE_HEAD : 0), prompt_len));
    } else {
        const std::vector<int> lens(batch, prompt_len);
        RC(prefill_context(*m, batch, lens.data()));
    }
    if (host_first_ids) ONELLM_CUDA(cudaMemcpyAsync(host_first_ids, m->d_out_ids, (size_t)batch * sizeof(int), cudaMemcpyDeviceToHost, st));
    RC(queue_comm_check(*m));
    ONELLM_CUDA(cudaStreamSynchronize(st));
    RC(comm_check(*m, "llama_prefill"));
    int bad[2] = {0, 0};
    ONELLM_CUDA(cudaMemcpy(bad, m->d_bad_id, 2 * sizeof(int), cudaMemcpyDeviceToHost));
    ONELLM_REQUIRE(bad[0] == 0, ONELLM_ERR_ARG, "llama_prefill: token id outside [0, vocab_size)");
    ONELLM_REQUIRE(bad[1] == 0, ONELLM_ERR_STATE, "llama_prefill: a position beyond max_seq_len was refused by the cache");
    ONELLM_REQUIRE(onellm_gemm_timeout_flag() <= 0, ONELLM_ERR_CUDA, "llama_prefill: a tensor-core GEMM block timed out");
    return ONELLM_OK;
}

// Prompts of different lengths: host_ids holds them packed one after the other, lens[b] tokens each.  Sequence b is
// cached in rows 0 .. lens[b]-1 of its cache; the step counter follows the longest sequence and the decode attention
// gives every other sequence its own, shorter, row count and position.
extern "C" int onellm_llama_prefill_ragged(onellm_llama* h, const int* host_ids, const int* lens, int batch, int* host_first_ids)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_ids && lens, ONELLM_ERR_ARG, "llama_prefill_ragged: null pointer");
    ONELLM_REQUIRE(m->weights_ready, ONELLM_ERR_STATE, "llama_prefill_ragged: weights not loaded");
    ONELLM_REQUIRE(batch >= 1 && batch <= m->c.max_batch, ONELLM_ERR_ARG, "llama_prefill_ragged: batch %d outside [1,%d]", batch, m->c.max_batch);
    size_t total = 0;
    int longest = 0;
    for (int b = 0; b < batch; b++) {
        ONELLM_REQUIRE(lens[b] >= 1 && lens[b] <= m->c.max_seq_len, ONELLM_ERR_ARG, "llama_prefill_ragged: lens[%d] = %d outside [1,%d]", b,
                       lens[b], m->c.max_seq_len);
        total += (size_t)lens[b];
        longest = lens[b] > longest ? lens[b] : longest;
    }
    cudaStream_t st = m->stream;
    ONELLM_CUDA(cudaStreamSynchronize(st));
    if (batch != m->batch) drop_graphs(*m);
    m->batch = batch;
    m->cur_len = 0;
    m->seq_off.assign(m->c.max_batch, 0);
    ONELLM_CUDA(cudaMemcpyAsync(m->d_prompt, host_ids, total * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(m->d_step, &longest, sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_seqlen, 0, (size_t)batch * sizeof(int), st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_finished, 0, (size_t)batch, st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_bad_id, 0, 4 * sizeof(int), st));
    ONELLM_CUDA(cudaStreamSynchronize(st));  // `longest` lives on this stack frame
    RC(prefill_context(*m, batch, lens));
    if (host_first_ids) ONELLM_CUDA(cudaMemcpyAsync(host_first_ids, m->d_out_ids, (size_t)batch * sizeof(int), cudaMemcpyDeviceToHost, st));
    RC(queue_comm_check(*m));
    ONELLM_CUDA(cudaStreamSynchronize(st));
    RC(comm_check(*m, "llama_prefill_ragged"));
    int bad[2] = {0, 0};
    ONELLM_CUDA(cudaMemcpy(bad, m->d_bad_id, 2 * sizeof(int), cudaMemcpyDeviceToHost));
    ONELLM_REQUIRE(bad[0] == 0, ONELLM_ERR_ARG, "llama_prefill_ragged: token id outside [0, vocab_size)");
    ONELLM_REQUIRE(bad[1] == 0, ONELLM_ERR_STATE, "llama_prefill_ragged: a position beyond max_seq_len was refused by the cache");
    ONELLM_REQUIRE(onellm_gemm_timeout_flag() <= 0, ONELLM_ERR_CUDA, "llama_prefill_ragged: a tensor-core GEMM block timed out");
    return ONELLM_OK;
}

// A further turn: n_new more tokens per sequence behind the cur_len positions already cached (history),
// through the context-phase kernels; the sampler is seeded with the new length, as after a prefill.
extern "C" int onellm_llama_extend(onellm_llama* h, const int* host_ids, int n_new, int* host_first_ids)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_ids, ONELLM_ERR_ARG, "llama_extend: null pointer");
    ONELLM_REQUIRE(m->batch > 0 && m->cur_len > 0, ONELLM_ERR_STATE, "llama_extend: call prefill first");
    ONELLM_REQUIRE(n_new >= 1 && m->cur_len + n_new <= m->c.max_seq_len, ONELLM_ERR_ARG,
                   "llama_extend: %d cached + %d new positions exceed max_seq_len %d", m->cur_len, n_new, m->c.max_seq_len);
    cudaStream_t st = m->stream;
    const int batch = m->batch, new_len = m->cur_len + n_new;
    ONELLM_CUDA(cudaMemcpyAsync(m->d_prompt, host_ids, (size_t)batch * n_new * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(m->d_step, &new_len, sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaStreamSynchronize(st));  // `new_len` lives on this stack frame
    const std::vector<int> lens(batch, n_new);
    RC(prefill_context(*m, batch, lens.data()));
    if (host_first_ids) ONELLM_CUDA(cudaMemcpyAsync(host_first_ids, m->d_out_ids, (size_t)batch * sizeof(int), cudaMemcpyDeviceToHost, st));
    RC(queue_comm_check(*m));
    ONELLM_CUDA(cudaStreamSynchronize(st));
    RC(comm_check(*m, "llama_extend"));
    int bad[2] = {0, 0};
    ONELLM_CUDA(cudaMemcpy(bad, m->d_bad_id, 2 * sizeof(int), cudaMemcpyDeviceToHost));
    ONELLM_REQUIRE(bad[0] == 0, ONELLM_ERR_ARG, "llama_extend: token id outside [0, vocab_size)");
    ONELLM_REQUIRE(bad[1] == 0, ONELLM_ERR_STATE, "llama_extend: a position beyond max_seq_len was refused by the cache");
    ONELLM_REQUIRE(onellm_gemm_timeout_flag() <= 0, ONELLM_ERR_CUDA, "llama_extend: a tensor-core GEMM block timed out");
    return ONELLM_OK;
}

// Declares `cur_len` positions of `batch` sequences as already cached (whatever the cache holds)
// and `host_ids` as the next input tokens: resumes decoding on a cache filled elsewhere, and lets
// profiling runs skip the context phase.
extern "C" int onellm_llama_seek(onellm_llama* h, int batch, int cur_len, const int* host_ids)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_ids, ONELLM_ERR_ARG, "llama_seek: null pointer");
    ONELLM_REQUIRE(m->weights_ready, ONELLM_ERR_STATE, "llama_seek: weights not loaded");
    ONELLM_REQUIRE(batch >= 1 && batch <= m->c.max_batch && cur_len >= 1 && cur_len < m->c.max_seq_len, ONELLM_ERR_ARG,
                   "llama_seek: batch or position out of range");
    cudaStream_t st = m->stream;
    ONELLM_CUDA(cudaStreamSynchronize(st));
    if (batch != m->batch) drop_graphs(*m);
    m->batch = batch;
    m->cur_len = cur_len;
    m->seq_off.assign(m->c.max_batch, 0);
    ONELLM_CUDA(cudaMemsetAsync(m->d_step_off, 0, (size_t)m->c.max_batch * sizeof(int), st));
    ONELLM_CUDA(cudaMemcpyAsync(m->d_step, &cur_len, sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemcpyAsync(m->d_ids, host_ids, (size_t)batch * sizeof(int), cudaMemcpyHostToDevice, st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_seqlen, 0, (size_t)batch * sizeof(int), st));
    ONELLM_CUDA(cudaMemsetAsync(m->d_finished, 0, (size_t)batch, st));
    ONELLM_CUDA(cudaStreamSynchronize(st));
    return ONELLM_OK;
}

extern "C" int onellm_llama_decode_step(onellm_llama* h, const int* host_in_ids, int* host_out_ids)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_decode_step: null handle");
    ONELLM_REQUIRE(m->batch > 0 && m->cur_len > 0, ONELLM_ERR_STATE, "llama_decode_step: call prefill first");
    cudaStream_t st = m->stream;
    if (host_in_ids)
        ONELLM_CUDA(cudaMemcpyAsync(m->d_ids, host_in_ids, (size_t)m->batch * sizeof(int), cudaMemcpyHostToDevice, st));
    RC(run_step(*m, MODE_HEAD, 0));
    if (host_out_ids) {
        ONELLM_CUDA(cudaMemcpyAsync(host_out_ids, m->d_out_ids, (size_t)m->batch * sizeof(int), cudaMemcpyDeviceToHost, st));
        RC(queue_comm_check(*m));
        ONELLM_CUDA(cudaStreamSynchronize(st));
        RC(comm_check(*m, "llama_decode_step"));
    }
    return ONELLM_OK;
}

extern "C" int onellm_llama_sync(onellm_llama* h)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_sync: null handle");
    RC(queue_comm_check(*m));
    ONELLM_CUDA(cudaStreamSynchronize(m->stream));
    return comm_check(*m, "llama_sync");
}

extern "C" int onellm_llama_generate(onellm_llama* h, const int* host_prompt, int batch, int prompt_len, int n_new, int* host_out)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_prompt && host_out && n_new >= 1, ONELLM_ERR_ARG, "llama_generate: bad argument");
    std::vector<int> ids(batch);
    RC(onellm_llama_prefill(h, host_prompt, batch, prompt_len, ids.data()));
    for (int b = 0; b < batch; b++) host_out[(size_t)b * n_new] = ids[b];
    for (int t = 1; t < n_new; t++) {
        RC(onellm_llama_decode_step(h, nullptr, ids.data()));
        for (int b = 0; b < batch; b++) host_out[(size_t)b * n_new + t] = ids[b];
    }
    return ONELLM_OK;
}

extern "C" int onellm_llama_get_logits(onellm_llama* h, float* host_logits)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && host_logits, ONELLM_ERR_ARG, "llama_get_logits: null pointer");
    ONELLM_REQUIRE(m->batch > 0, ONELLM_ERR_STATE, "llama_get_logits: nothing computed yet");
    const size_t n = (size_t)m->batch * m->c.vocab_size;
    float* tmp = nullptr;
    ONELLM_CUDA(cudaMalloc(&tmp, n * sizeof(float)));
    half_to_float_kernel<<<blocks_for(n), 256, 0, m->stream>>>(m->logits, tmp, n);
    cudaError_t e = cudaMemcpyAsync(host_logits, tmp, n * sizeof(float), cudaMemcpyDeviceToHost, m->stream);
    const int qrc = queue_comm_check(*m);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    cudaFree(tmp);
    ONELLM_REQUIRE(e == cudaSuccess, ONELLM_ERR_CUDA, "llama_get_logits: %s", cudaGetErrorString(e));
    RC(qrc);
    return comm_check(*m, "llama_get_logits");
}

extern "C" int onellm_llama_get_state(onellm_llama* h, int* cur_len, long* kernel_launches, int* host_seqlen, unsigned char* host_finished)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m, ONELLM_ERR_ARG, "llama_get_state: null handle");
    if (cur_len) *cur_len = m->cur_len;
    if (kernel_launches) *kernel_launches = m->launches;
    if (host_seqlen && m->batch) ONELLM_CUDA(cudaMemcpy(host_seqlen, m->d_seqlen, (size_t)m->batch * sizeof(int), cudaMemcpyDeviceToHost));
    if (host_finished && m->batch) ONELLM_CUDA(cudaMemcpy(host_finished, m->d_finished, (size_t)m->batch, cudaMemcpyDeviceToHost));
    return ONELLM_OK;
}

// Device pointers of one layer's cache and of the weights, for tests and tools.
extern "C" int onellm_llama_kv_cache(onellm_llama* h, int layer, void** k_cache, void** v_cache)
{
    Llama* m = reinterpret_cast<Llama*>(h);
    ONELLM_REQUIRE(m && layer >= 0 && layer < m->c.num_layers, ONELLM_ERR_ARG, "llama_kv_cache: bad argument");
    if (k_cache) *k_cache = m->k_cache + (size_t)layer * m->cache_layer_elems;
    if (v_cache) *v_cache = m->v_cache + (size_t)layer * m->cache_layer_elems;
    return ONELLM_OK;
}
