// Top-K selection and top-K sampling for sm_100a.
//
// Top-K generalises the reference's two-round block top-K with K fixed at 2
// (src/kernels/beamsearch_topK.cu:20-119, struct topK in src/kernels/beamsearch_topK.h:3-33)
// to 1 <= K <= 64 with a defined order for ties (lower column first).  Sampling restates
// SamplingKernel (src/kernels/topK_sampling.cu:6-41) with the same cuRAND call sequence.
//
// One thread block per row, over an order-preserving integer image of the logits (NaN lowest).  Rows of up to
// 32768 logits (topk_reg_kernel) are read once, 32 consecutive keys per thread in registers: the K-th largest of
// the per-thread maxima bounds the K-th largest key from below, the few keys that reach it are gathered and ranked
// against each other; rows with long runs of equal keys fall back to a bisection over all keys.  Neither step
// uses a histogram: logits share their leading bits, and a 256-bin histogram in shared memory serialises on a
// handful of bins.  Longer rows (topk_kernel) are a radix select, 8 bits per pass, re-reading the logits from L2.
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


template <typename T>
__device__ __forceinline__ uint32_t logit_key(T v);
template <>
__device__ __forceinline__ uint32_t logit_key<float>(float v) { return float_key(v); }
template <>
__device__ __forceinline__ uint32_t logit_key<__half>(__half v)
{
    // 16-bit image in the upper half of the key: same order as the float image, two radix passes
    const uint32_t u = __half_as_ushort(v);
    if ((u & 0x7fffu) > 0x7c00u) return 0u;  // NaN
    return ((u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u)) << 16;
}
template <typename T>
__device__ __forceinline__ float key_value(uint32_t k);
template <>
__device__ __forceinline__ float key_value<float>(uint32_t k) { return key_float(k); }
template <>
__device__ __forceinline__ float key_value<__half>(uint32_t k)
{
    const uint32_t k16 = k >> 16;
    const uint32_t u = (k16 & 0x8000u) ? (k16 & 0x7fffu) : (~k16 & 0xffffu);
    return __half2float(__ushort_as_half((unsigned short)u));
}

constexpr int kTopkPer = 32;  // keys per thread held in registers
constexpr int kTopkCand = 512;  // gathered keys the short way ranks; >= kMaxK

template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
topk_reg_kernel(const T* __restrict__ logits, int vocab, int K, float* __restrict__ out_val, int* __restrict__ out_id,
                int global_ids)
{
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const T* x = logits + (size_t)row * vocab;
    __shared__ int s_count;
    __shared__ int warp_tot[kTopkThreads / 32];
    __shared__ uint32_t cand_key[kTopkCand];
    __shared__ int cand_id[kTopkCand];

    // thread t owns columns [t*32, t*32 + 32): a contiguous slice, so ranks inside a tie follow the columns
    const int c0 = threadIdx.x * kTopkPer;
    const int n_mine = max(0, min(kTopkPer, vocab - c0));
    uint32_t key[kTopkPer];
    constexpr int VEC = 16 / sizeof(T);
    if (n_mine == kTopkPer && ((reinterpret_cast<uintptr_t>(x + c0) & 15u) == 0)) {
#pragma unroll
        for (int j = 0; j < kTopkPer; j += VEC) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + c0 + j);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int q = 0; q < VEC; q++) key[j + q] = logit_key<T>(e[q]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kTopkPer; j++) key[j] = j < n_mine ? logit_key<T>(x[c0 + j]) : 0u;
    }
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();

    constexpr int kLowBit = sizeof(T) == 2 ? 16 : 0;  // fp16 keys live in the upper half
    __shared__ int bit_tot[2][kTopkThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int it = 0;

    // 0. The short way, which nearly every row of logits takes.  The K-th largest of the 1024 per-thread maxima is
    // a lower bound of the K-th largest key (K threads hold a key that large), and for logits hardly more than K
    // keys reach it.  One bisection over ONE key per thread finds it (a ballot per warp, one block barrier per bit);
    // the keys that reach it are gathered (a few dozen shared-memory atomics) and ranked against each other, larger
    // key first, lower column first among equals: rank r < K is output slot r.  Rows with many equal keys, where
    // the gathered set would be large, take the bisection over all keys below instead.
    {
        uint32_t mk = 0u;  // padding and NaN have key 0
#pragma unroll
        for (int j = 0; j < kTopkPer; j++) mk = max(mk, key[j]);
        uint32_t low = 0u;
#pragma unroll 1
        for (int bit = 31; bit >= kLowBit; bit--, it++) {
            const uint32_t t = low | (1u << bit);
            const int c = __popc(__ballot_sync(0xffffffffu, mk >= t));
            if (lane == 0) bit_tot[it & 1][wid] = c;
            __syncthreads();
            if (__reduce_add_sync(0xffffffffu, bit_tot[it & 1][lane]) >= K) low = t;
        }
        if (mk >= low) {
#pragma unroll
            for (int j = 0; j < kTopkPer; j++) {
                if (j < n_mine && key[j] >= low) {
                    const int pos = atomicAdd(&s_count, 1);
                    if (pos < kTopkCand) {
                        cand_key[pos] = key[j];
                        cand_id[pos] = c0 + j;
                    }
                }
            }
        }
        __syncthreads();
        const int n_c = s_count;  // >= K: K threads hold a real key >= low (or low == 0 and every column counts)
        if (n_c <= kTopkCand) {
            if ((int)threadIdx.x < n_c) {
                const uint32_t k = cand_key[threadIdx.x];
                const int id = cand_id[threadIdx.x];
                int r = 0;
                for (int j = 0; j < n_c; j++) r += (cand_key[j] > k) || (cand_key[j] == k && cand_id[j] < id);
                if (r < K) {
                    out_val[(size_t)row * K + r] = (k == 0u) ? -INFINITY : key_value<T>(k);
                    out_id[(size_t)row * K + r] = global_ids ? row * vocab + id : id;
                }
            }
            return;
        }
        __syncthreads();  // everyone has read s_count
        if (threadIdx.x == 0) s_count = 0;
        __syncthreads();
    }

    // 1. K-th largest key by bisection on its bits, from the top: the largest t with at least K keys >= t.  Every thread
    // counts its 32 keys in registers, a warp adds up with one reduction, the 32 warp sums meet in shared memory (two
    // buffers in turn: one block barrier per bit) and every thread takes the same decision, so nothing is broadcast
    // and no shared-memory atomic is used (a 256-bin histogram of logits has a handful of hot bins: the radix form
    // of this step spent most of its 39 us waiting for them).
    auto block_count = [&](auto pred, int buf) {
        int c = 0;
#pragma unroll
        for (int j = 0; j < kTopkPer; j++) c += (j < n_mine && pred(key[j])) ? 1 : 0;
        c = __reduce_add_sync(0xffffffffu, c);
        if (lane == 0) bit_tot[buf][wid] = c;
        __syncthreads();
        return __reduce_add_sync(0xffffffffu, bit_tot[buf][lane]);
    };
    uint32_t kth = 0u;
#pragma unroll 1
    for (int bit = 31; bit >= kLowBit; bit--, it++) {
        const uint32_t t = kth | (1u << bit);
        if (block_count([t](uint32_t k) { return k >= t; }, it & 1) >= K) kth = t;
    }
    const int need_ties = K - block_count([kth](uint32_t k) { return k > kth; }, it & 1);

    // 2. gather: everything above the K-th key (any order), then the lowest-indexed ties
    int ties = 0;
#pragma unroll
    for (int j = 0; j < kTopkPer; j++) {
        if (j < n_mine && key[j] > kth) {
            const int pos = atomicAdd(&s_count, 1);
            cand_key[pos] = key[j];
            cand_id[pos] = c0 + j;
        }
        ties += (j < n_mine && key[j] == kth);
    }
    __syncthreads();
    const int n_above = s_count;  // == K - need_ties
    {
        int incl = ties;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((threadIdx.x & 31) >= o) incl += v;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            const int v = warp_tot[threadIdx.x];
            int inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, inc, o);
                if ((int)threadIdx.x >= o) inc += u;
            }
            warp_tot[threadIdx.x] = inc - v;  // exclusive
        }
        __syncthreads();
        int rank = warp_tot[threadIdx.x >> 5] + incl - ties;
        if (ties > 0 && rank < need_ties) {
#pragma unroll
            for (int j = 0; j < kTopkPer; j++) {
                if (j < n_mine && key[j] == kth && rank < need_ties) {
                    cand_key[n_above + rank] = kth;
                    cand_id[n_above + rank] = c0 + j;
                    rank++;
                }
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
        out_val[(size_t)row * K + r] = (k == 0u) ? -INFINITY : key_value<T>(k);
        out_id[(size_t)row * K + r] = global_ids ? row * vocab + id : id;
    }
}

// The draw of (step, row) is curand_init(step, row, 0) + curand_uniform, as src/kernels/topK_sampling.cu:29-30 of the
// reference takes it.  For row > 0 nearly all of its time is the skip-ahead to sub-sequence `row`: a linear map
// (over GF(2)) of the 160 xorshift bits of the XORWOW state, which cuRAND applies bit by bit in one thread, 10-15 us
// per set bit of the row index.  The map depends on the row only, so a caller that draws for the same rows at
// every step can have it tabulated once (build_skip_table: the image of each of the 160 unit vectors under
// skipahead_sequence(row), 3200 bytes per row, and the change of the additive counter `d`); the draw is then
// curand_init(step, 0, 0), which skips nothing, and an XOR of the columns the state's set bits select, five bits per
// lane.  The table is checked against the direct form when it is built and not used if a single draw differs.
constexpr int kSkipBits = 160, kSkipWords = 5;
constexpr int kSkipRowWords = kSkipBits * kSkipWords + 1;  // a row's columns, then its counter change

__global__ void skip_table_kernel(uint32_t* __restrict__ tab)
{
    const int b = blockIdx.x, i = threadIdx.x;  // one row per block, one state bit per thread
    curandStateXORWOW_t s;
    s.d = 0u;
    for (int w = 0; w < kSkipWords; w++) s.v[w] = 0u;
    s.boxmuller_flag = 0;
    s.boxmuller_flag_double = 0;
    s.boxmuller_extra = 0.f;
    s.boxmuller_extra_double = 0.0;
    s.v[i >> 5] = 1u << (i & 31);
    skipahead_sequence((unsigned long long)b, &s);
    uint32_t* row = tab + (size_t)b * kSkipRowWords;
    for (int w = 0; w < kSkipWords; w++) row[i * kSkipWords + w] = s.v[w];
    if (i == 0) row[kSkipBits * kSkipWords] = s.d;
}

// Whole warp; the result is valid in lane 0.
__device__ __forceinline__ float draw_with_table(int seed, int b, const uint32_t* __restrict__ tab)
{
    const uint32_t* row = tab + (size_t)b * kSkipRowWords;
    const int lane = threadIdx.x & 31;
    curandStateXORWOW_t s;
    uint32_t v[kSkipWords] = {0u, 0u, 0u, 0u, 0u};
    if (lane == 0) {
        curand_init((unsigned long long)seed, 0ULL, 0ULL, &s);
#pragma unroll
        for (int w = 0; w < kSkipWords; w++) v[w] = s.v[w];
    }
#pragma unroll
    for (int w = 0; w < kSkipWords; w++) v[w] = __shfl_sync(0xffffffffu, v[w], 0);
    uint32_t acc[kSkipWords] = {0u, 0u, 0u, 0u, 0u};
#pragma unroll
    for (int q = 0; q < kSkipBits / 32; q++) {
        const int bit = q * 32 + lane;  // word q, bit `lane`
        if ((v[q] >> lane) & 1u) {
            const uint32_t* col = row + bit * kSkipWords;
#pragma unroll
            for (int w = 0; w < kSkipWords; w++) acc[w] ^= col[w];
        }
    }
#pragma unroll
    for (int w = 0; w < kSkipWords; w++) acc[w] = __reduce_xor_sync(0xffffffffu, acc[w]);
    float u = 0.f;
    if (lane == 0) {
#pragma unroll
        for (int w = 0; w < kSkipWords; w++) s.v[w] = acc[w];
        s.d += row[kSkipBits * kSkipWords];
        u = curand_uniform(&s);
    }
    return u;
}

__global__ void skip_table_check_kernel(const uint32_t* __restrict__ tab, int* __restrict__ mismatches)
{
    const int b = blockIdx.x;
    const int seeds[6] = {0, 1, 2, 515, 12345, 0x7fffffff};
    for (int i = 0; i < 6; i++) {
        const float fast = draw_with_table(seeds[i], b, tab);
        if (threadIdx.x == 0) {
            curandState_t state;
            curand_init((unsigned long long)seeds[i], (unsigned long long)b, 0ULL, &state);
            if (curand_uniform(&state) != fast) atomicAdd(mismatches, 1);
        }
    }
}

__global__ void sample_kernel(const int* __restrict__ topk_id, const float* __restrict__ topk_val, int K,
                              float temperature, int rng_step, const int* __restrict__ rng_step_dev,
                              int vocab_size, int end_id, int literal_walk, int* __restrict__ output_id, int* __restrict__ seqlen,
                              unsigned char* __restrict__ finished, float* __restrict__ u_out,
                              int* __restrict__ output_id2, int early_seed, const uint32_t* __restrict__ skip_tab)
{
    pdl_launch_dependents();
    const int b = blockIdx.x;
    // The draw depends on (step, row) only, and seeding the generator (a sequence skip-ahead) is by far
    // the longest part of this kernel.  early_seed: do it before waiting for the candidates; the caller
    // vouches that *rng_step_dev was written by work that completed long before (the model's step
    // counter is advanced by the first kernel of a step, and the layer projections between it and this
    // kernel release their dependents only after passing their own griddepcontrol.wait).
    float u = 0.f;
    auto draw = [&]() {  // whole warp (blockDim.x == 32); u is valid in thread 0
        const int seed = rng_step_dev ? *rng_step_dev : rng_step;
        if (skip_tab) {
            u = draw_with_table(seed, b, skip_tab);
        } else if (threadIdx.x == 0) {
            curandState_t state;
            curand_init((unsigned long long)seed, (unsigned long long)b, 0ULL, &state);
            u = curand_uniform(&state);
        }
    };
    if (early_seed) draw();
    pdl_wait();
    if (!early_seed) draw();
    if (threadIdx.x != 0) return;
    const float* v = topk_val + (size_t)b * K;
    const float v0 = v[0];
    float sum = 0.f;
    for (int i = 0; i < K; i++) sum += expf((v[i] - v0) / temperature);
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
    const bool in_regs = vocab <= kTopkPer * kTopkThreads;
    if (dtype == ONELLM_F16)
        ONELLM_CUDA(launch_pdl(in_regs ? topk_reg_kernel<__half> : topk_kernel<__half>, dim3(rows), dim3(kTopkThreads), 0, st,
                               (const __half*)logits, vocab, K, out_val, out_id, global_ids));
    else if (dtype == ONELLM_F32)
        ONELLM_CUDA(launch_pdl(in_regs ? topk_reg_kernel<float> : topk_kernel<float>, dim3(rows), dim3(kTopkThreads), 0, st,
                               (const float*)logits, vocab, K, out_val, out_id, global_ids));
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
                       int* seqlen, unsigned char* finished, float* u_out, int* output_id2, bool early_seed,
                       const uint32_t* skip_table, cudaStream_t st)
{
    ONELLM_REQUIRE(topk_id && topk_val && output_id, ONELLM_ERR_ARG, "topk_sample: null pointer");
    ONELLM_REQUIRE(B >= 0 && K >= 1 && vocab_size > 0 && temperature > 0.f, ONELLM_ERR_ARG,
                   "topk_sample: bad size or temperature");
    ONELLM_REQUIRE((seqlen == nullptr) == (finished == nullptr), ONELLM_ERR_ARG,
                   "topk_sample: seqlen and finished must be given together");
    if (B == 0) return ONELLM_OK;
    ONELLM_CUDA(launch_pdl(sample_kernel, dim3(B), dim3(32), 0, st, topk_id, topk_val, K, temperature, rng_step,
                           rng_step_dev, vocab_size, end_id, literal_walk, output_id, seqlen, finished, u_out,
                           output_id2, early_seed ? 1 : 0, skip_table));
    return ONELLM_OK;
}

// Words a skip table for `rows` rows takes.
size_t skip_table_words(int rows) { return (size_t)rows * kSkipRowWords; }

// Fills `table` (device memory, skip_table_words(rows) words) for rows 0..rows-1 and checks it against the direct
// draw; waits for the stream.  *usable = 0 when a draw differed (the caller then passes no table).  A table built
// for `rows` rows serves launches of up to that many rows.
int build_skip_table(uint32_t* table, int rows, int* usable, cudaStream_t st)
{
    ONELLM_REQUIRE(table && usable && rows > 0, ONELLM_ERR_ARG, "skip table: bad argument");
    int* d_bad = nullptr;
    ONELLM_CUDA(cudaMalloc(&d_bad, sizeof(int)));
    cudaError_t e = cudaMemsetAsync(d_bad, 0, sizeof(int), st);
    if (e == cudaSuccess) {
        skip_table_kernel<<<rows, kSkipBits, 0, st>>>(table);
        skip_table_check_kernel<<<rows, 32, 0, st>>>(table, d_bad);
        e = cudaGetLastError();
    }
    int bad = 1;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&bad, d_bad, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_bad);
    ONELLM_CUDA(e);
    *usable = bad == 0 ? 1 : 0;
    return ONELLM_OK;
}
}  // namespace onellm

extern "C" int onellm_topk_sample(const int* topk_id, const float* topk_val, int B, int K, float temperature,
                                  int rng_step, const int* rng_step_dev, int vocab_size, int end_id,
                                  int literal_walk, int* output_id, int* seqlen, unsigned char* finished,
                                  float* u_out, void* stream)
{
    return topk_sample_launch(topk_id, topk_val, B, K, temperature, rng_step, rng_step_dev, vocab_size, end_id,
                              literal_walk, output_id, seqlen, finished, u_out, nullptr, /*early_seed=*/false,
                              /*skip_table=*/nullptr, reinterpret_cast<cudaStream_t>(stream));
}
