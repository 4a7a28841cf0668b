// Top-K selection and top-K sampling for sm_100a.
//
// Top-K generalises the reference's two-round block top-K with K fixed at 2
// (src/kernels/beamsearch_topK.cu:20-119, struct topK in src/kernels/beamsearch_topK.h:3-33)
// to 1 <= K <= 64 with a defined order for ties (lower column first).  Sampling restates
// SamplingKernel (src/kernels/topK_sampling.cu:6-41) with the same cuRAND call sequence.
//
// Top-K is a radix select, one thread block per row: four 8-bit histogram passes over an
// order-preserving integer image of the logits find the K-th largest key, then everything
// above it plus the lowest-indexed ties are gathered and rank-sorted.  The row (128 KB at
// vocab 32000) stays in L2 between passes.
#include <curand_kernel.h>
#include <math.h>

#include "common.cuh"

namespace onellm {

constexpr int kTopkThreads = 1024;
constexpr int kMaxK = 64;

__device__ __forceinline__ uint32_t float_key(float f)
{
    if (f != f) return 0u;  // NaN sorts below everything
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_float(uint32_t k)
{
    const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__half>(const __half* p, int i) { return __half2float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
topk_kernel(const T* __restrict__ logits, int vocab, int K, float* __restrict__ out_val, int* __restrict__ out_id,
            int global_ids)
{
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const T* x = logits + (size_t)row * vocab;
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;            // how many still to take among keys matching the prefix
    __shared__ int s_count;           // gather cursor
    __shared__ int warp_tot[kTopkThreads / 32];
    __shared__ uint32_t cand_key[kMaxK];
    __shared__ int cand_id[kMaxK];

    if (threadIdx.x == 0) {
        s_prefix = 0u;
        s_need = K;
        s_count = 0;
    }
    __syncthreads();

    // 1. K-th largest key, 8 bits at a time from the top
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = threadIdx.x; i < 256; i += kTopkThreads) hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int i = threadIdx.x; i < vocab; i += kTopkThreads) {
            const uint32_t k = float_key(load_logit<T>(x, i));
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int need = s_need, b = 255;
            for (; b > 0; b--) {
                if (hist[b] >= need) break;
                need -= hist[b];
            }
            s_prefix = prefix | ((uint32_t)b << shift);
            s_need = need;  // ties still to take once all 32 bits are fixed
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;
    const int need_ties = s_need;

    // 2. gather: everything above the K-th key (any order), then the lowest-indexed ties
    for (int i = threadIdx.x; i < vocab; i += kTopkThreads) {
        const uint32_t k = float_key(load_logit<T>(x, i));
        if (k > kth) {
            const int pos = atomicAdd(&s_count, 1);
            cand_key[pos] = k;
            cand_id[pos] = i;
        }
    }
    __syncthreads();
    const int n_above = s_count;  // == K - need_ties
    {
        // contiguous slices per thread so that an exclusive scan gives ranks in column order
        const int per = (vocab + kTopkThreads - 1) / kTopkThreads;
        const int c0 = threadIdx.x * per, c1 = min(c0 + per, vocab);
        int mine = 0;
        for (int i = c0; i < c1; i++) mine += (float_key(load_logit<T>(x, i)) == kth);
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((threadIdx.x & 31) >= o) incl += v;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            int v = threadIdx.x < kTopkThreads / 32 ? warp_tot[threadIdx.x] : 0;
            int inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, inc, o);
                if (threadIdx.x >= o) inc += u;
            }
            if (threadIdx.x < kTopkThreads / 32) warp_tot[threadIdx.x] = inc - v;  // exclusive
        }
        __syncthreads();
        int rank = warp_tot[threadIdx.x >> 5] + incl - mine;
        for (int i = c0; i < c1 && rank < need_ties; i++) {
            if (float_key(load_logit<T>(x, i)) == kth) {
                cand_key[n_above + rank] = kth;
                cand_id[n_above + rank] = i;
                rank++;
            }
        }
    }
    __syncthreads();

    // 3. rank sort: larger key first, lower column first among equals
    if (threadIdx.x < K) {
        const uint32_t k = cand_key[threadIdx.x];
        const int id = cand_id[threadIdx.x];
        int r = 0;
        for (int j = 0; j < K; j++) r += (cand_key[j] > k) || (cand_key[j] == k && cand_id[j] < id);
        const float v = key_float(k);
        out_val[(size_t)row * K + r] = (k == 0u) ? -INFINITY : v;
        out_id[(size_t)row * K + r] = global_ids ? row * vocab + id : id;
    }
}

__global__ void sample_kernel(const int* __restrict__ topk_id, const float* __restrict__ topk_val, int K,
                              float temperature, int rng_step, const int* __restrict__ rng_step_dev,
                              int vocab_size, int end_id, int literal_walk, int* __restrict__ output_id, int* __restrict__ seqlen,
                              unsigned char* __restrict__ finished, float* __restrict__ u_out,
                              int* __restrict__ output_id2)
{
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (threadIdx.x != 0) return;
    const float* v = topk_val + (size_t)b * K;
    const float v0 = v[0];
    float sum = 0.f;
    for (int i = 0; i < K; i++) sum += expf((v[i] - v0) / temperature);
    curandState_t state;
    const int seed = rng_step_dev ? *rng_step_dev : rng_step;
    curand_init((unsigned long long)seed, (unsigned long long)b, 0ULL, &state);
    const float u = curand_uniform(&state);
    if (u_out) u_out[b] = u;
    float thr = u * sum;
    int pick = K - 1;
    for (int i = 0; i < K; i++) {
        thr -= literal_walk ? 1.0f : expf((v[i] - v0) / temperature);
        if (thr < 0.f) {
            pick = i;
            break;
        }
    }
    const int id = topk_id[(size_t)b * K + pick] % vocab_size;
    output_id[b] = id;
    if (output_id2) output_id2[b] = id;
    if (seqlen && finished) {
        seqlen[b] = finished[b] ? seqlen[b] : seqlen[b] + 1;
        finished[b] = (id == end_id) ? 1 : 0;
    }
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_topk(int dtype, const void* logits, int rows, int vocab, int K, float* out_val, int* out_id,
                           int global_ids, void* stream)
{
    ONELLM_REQUIRE(logits && out_val && out_id, ONELLM_ERR_ARG, "topk: null pointer");
    ONELLM_REQUIRE(rows >= 0 && vocab > 0, ONELLM_ERR_ARG, "topk: bad size");
    ONELLM_REQUIRE(K >= 1 && K <= kMaxK && K <= vocab, ONELLM_ERR_UNSUPPORTED, "topk: K=%d outside [1, %d]", K,
                   kMaxK);
    if (rows == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == ONELLM_F16)
        ONELLM_CUDA(launch_pdl(topk_kernel<__half>, dim3(rows), dim3(kTopkThreads), 0, st, (const __half*)logits, vocab, K,
                               out_val, out_id, global_ids));
    else if (dtype == ONELLM_F32)
        ONELLM_CUDA(launch_pdl(topk_kernel<float>, dim3(rows), dim3(kTopkThreads), 0, st, (const float*)logits, vocab, K,
                               out_val, out_id, global_ids));
    else
        ONELLM_REQUIRE(false, ONELLM_ERR_UNSUPPORTED, "topk: dtype %d", dtype);
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

namespace onellm {
// Shared by the C entry point and the model driver; output_id2 (may be NULL) gets a second
// copy of the sampled ids (the next step's input buffer).
int topk_sample_launch(const int* topk_id, const float* topk_val, int B, int K, float temperature, int rng_step,
                       const int* rng_step_dev, int vocab_size, int end_id, int literal_walk, int* output_id,
                       int* seqlen, unsigned char* finished, float* u_out, int* output_id2, cudaStream_t st)
{
    ONELLM_REQUIRE(topk_id && topk_val && output_id, ONELLM_ERR_ARG, "topk_sample: null pointer");
    ONELLM_REQUIRE(B >= 0 && K >= 1 && vocab_size > 0 && temperature > 0.f, ONELLM_ERR_ARG,
                   "topk_sample: bad size or temperature");
    ONELLM_REQUIRE((seqlen == nullptr) == (finished == nullptr), ONELLM_ERR_ARG,
                   "topk_sample: seqlen and finished must be given together");
    if (B == 0) return ONELLM_OK;
    ONELLM_CUDA(launch_pdl(sample_kernel, dim3(B), dim3(32), 0, st, topk_id, topk_val, K, temperature, rng_step,
                           rng_step_dev, vocab_size, end_id, literal_walk, output_id, seqlen, finished, u_out,
                           output_id2));
    return ONELLM_OK;
}
}  // namespace onellm

extern "C" int onellm_topk_sample(const int* topk_id, const float* topk_val, int B, int K, float temperature,
                                  int rng_step, const int* rng_step_dev, int vocab_size, int end_id,
                                  int literal_walk, int* output_id, int* seqlen, unsigned char* finished,
                                  float* u_out, void* stream)
{
    return topk_sample_launch(topk_id, topk_val, B, K, temperature, rng_step, rng_step_dev, vocab_size, end_id,
                              literal_walk, output_id, seqlen, finished, u_out, nullptr,
                              reinterpret_cast<cudaStream_t>(stream));
}
