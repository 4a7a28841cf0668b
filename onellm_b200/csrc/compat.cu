// One-to-one replacements for the reference launchers that the fused context-phase kernels make
// unnecessary.  They exist so that LLaMAContextAttentionLayer::forward
// (src/layers/attention/context_attention.cpp:101-158 of the reference) can keep its nine-step
// sequence unchanged on top of this library; new code should call onellm_qkv_bias_rope_kvcache and
// onellm_context_attn instead.  All are plain HBM-bound kernels (fp32 or fp16).
//   onellm_cal_padding_offset       launchCalPaddingoffset           src/kernels/cal_paddingoffset.cu:9-46
//   onellm_build_causal_mask        launchBuildCausalMasks           src/kernels/build_casual_mask.cu:27-60
//   onellm_qkv_bias_rope_transpose  launchAddFusedQKVBiasTransposeAndRoPE  src/kernels/qkv_bias_and_RoPE.cu:74-207
//   onellm_append_kv_cache          launchAppendKVCache              src/kernels/append_to_kvcache.cu:8-114
//   onellm_repeat_kv                launchTransposeKVCache           src/kernels/transpose_kernel.cu:7-88
//   onellm_batched_gemm             launchLinearStridedBatchGemm     src/kernels/qkv_linear.cu:67-120
//   onellm_scale_mask_softmax       launchScaleMaskAndSoftmax        src/kernels/attn_softmax_kernel.cu:45-176
//   onellm_transpose_remove_padding launchTransposeOutRemovePadding  src/kernels/fused_transpose_reshape_remv_pad.cu:5-51
#include <math.h>

#include "common.cuh"

namespace onellm {

constexpr int kPairs = 128;
struct RopeDenoms {
    float d[kPairs];
};

__global__ void padding_offset_kernel(int* __restrict__ padding_offset, int* __restrict__ cum_seqlens,
                                      const int* __restrict__ seq_lens, int B, int max_q_len, int* __restrict__ token_num)
{
    // thread 0 takes the exclusive prefix sums of the (at most 64) lengths; the block then writes the offsets
    __shared__ int cum[65];
    if (threadIdx.x == 0) {
        int total = 0;
        for (int b = 0; b < B; b++) {
            cum[b] = total;
            total += seq_lens[b];
        }
        cum[B] = total;
        if (token_num) *token_num = total;
    }
    __syncthreads();
    for (int b = threadIdx.x; b <= B; b += blockDim.x) cum_seqlens[b] = cum[b];
    for (int b = 0; b < B; b++) {
        const int off = b * max_q_len - cum[b];  // padding in front of sequence b
        for (int i = threadIdx.x; i < cum[b + 1] - cum[b]; i += blockDim.x) padding_offset[cum[b] + i] = off;
    }
}

template <typename T>
__global__ void causal_mask_kernel(T* __restrict__ mask, const int* __restrict__ q_lens, const int* __restrict__ k_lens,
                                   int max_q, int max_k, int attend_history)
{
    const int b = blockIdx.y, ql = q_lens[b], kl = k_lens[b];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < max_q * max_k; i += gridDim.x * blockDim.x) {
        const int q = i / max_k, k = i % max_k;
        bool one = q < ql && k < kl && k <= q + (kl - ql);
        if (!attend_history) one = one && k >= kl - ql;  // the shipped predicate, build_casual_mask.cu:40-43
        mask[(size_t)b * max_q * max_k + i] = (T)(one ? 1.f : 0.f);
    }
}

template <typename T>
__global__ void qkv_rope_transpose_kernel(T* __restrict__ q_buf, T* __restrict__ k_buf, T* __restrict__ v_buf,
                                          const T* __restrict__ QKV, const T* __restrict__ bias,
                                          const int* __restrict__ padding_offset, const int* __restrict__ history, int B,
                                          int seq_len, int H, int Hkv, int D, int rot_dim, const RopeDenoms rd)
{
    const int t = blockIdx.x;
    const int dst_tok = t + padding_offset[t];
    const int b = dst_tok / seq_len, local = dst_tok % seq_len;
    if (b >= B) return;
    const float pos = (float)(history[b] + local);
    const int QH = H + 2 * Hkv, half_d = D / 2;
    const T* row = QKV + (size_t)t * QH * D;
    for (int idx = threadIdx.x; idx < QH * half_d; idx += blockDim.x) {
        const int head = idx / half_d, pr = idx % half_d;
        float x = (float)row[head * D + 2 * pr], y = (float)row[head * D + 2 * pr + 1];
        if (bias) {
            x += (float)bias[head * D + 2 * pr];
            y += (float)bias[head * D + 2 * pr + 1];
        }
        if (head < H + Hkv && 2 * pr < rot_dim) {
            float sn, cs;
            sincosf(pos / rd.d[pr], &sn, &cs);
            const float xr = cs * x - sn * y, yr = cs * y + sn * x;
            x = xr;
            y = yr;
        }
        T* dst;
        if (head < H) dst = q_buf + (((size_t)b * H + head) * seq_len + local) * D;
        else if (head < H + Hkv) dst = k_buf + (((size_t)b * Hkv + head - H) * seq_len + local) * D;
        else dst = v_buf + (((size_t)b * Hkv + head - H - Hkv) * seq_len + local) * D;
        dst[2 * pr] = (T)x;
        dst[2 * pr + 1] = (T)y;
    }
}

template <typename T>
__global__ void append_kv_kernel(T* __restrict__ dst, const T* __restrict__ src, const int* __restrict__ cur_len,
                                 const int* __restrict__ history, int Hkv, int max_q_len, int max_seq_len, int D,
                                 int* __restrict__ overflow)
{
    const int tok = blockIdx.x, b = blockIdx.y, hk = blockIdx.z;
    if (tok >= cur_len[b]) return;
    const int row = history[b] + tok;
    if (row >= max_seq_len) {
        if (overflow && threadIdx.x == 0) atomicExch(overflow, 1);
        return;
    }
    const T* s = src + (((size_t)b * Hkv + hk) * max_q_len + tok) * D;
    T* d = dst + (((size_t)b * Hkv + hk) * max_seq_len + row) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) d[i] = s[i];
}

template <typename T>
__global__ void repeat_kv_kernel(T* __restrict__ dst, const T* __restrict__ src, const int* __restrict__ context_len, int H,
                                 int Hkv, int max_k_len, int max_seq_len, int D)
{
    const int b = blockIdx.y, h = blockIdx.z, hk = h / (H / Hkv);
    const int n = min(context_len[b], max_k_len) * D;
    const T* s = src + ((size_t)b * Hkv + hk) * max_seq_len * D;
    T* d = dst + ((size_t)b * H + h) * max_k_len * D;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) d[i] = s[i];
}

// C[b](i,j) = alpha * sum_k A[b](i,k) * B[b](k,j) + beta * C[b](i,j) with every operand addressed through
// element strides, so one kernel serves row-major, column-major and transposed callers.
struct GemmStrides {
    long a_i, a_k, a_b, b_k, b_j, b_b, c_i, c_j, c_b;
};

template <typename T>
__global__ void strided_gemm_kernel(const T* __restrict__ A, const T* __restrict__ Bm, T* __restrict__ Cm, int m, int n, int k,
                                    GemmStrides s, float alpha, float beta)
{
    __shared__ float as[16][17], bs[16][17];
    const long batch = blockIdx.z;
    const T* a = A + batch * s.a_b;
    const T* b = Bm + batch * s.b_b;
    T* c = Cm + batch * s.c_b;
    const int row = blockIdx.y * 16 + threadIdx.y, col = blockIdx.x * 16 + threadIdx.x;
    float acc = 0.f;
    for (int k0 = 0; k0 < k; k0 += 16) {
        const int ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        as[threadIdx.y][threadIdx.x] = (row < m && ka < k) ? (float)a[row * s.a_i + ka * s.a_k] : 0.f;
        bs[threadIdx.y][threadIdx.x] = (col < n && kb < k) ? (float)b[kb * s.b_k + col * s.b_j] : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) acc = fmaf(as[threadIdx.y][kk], bs[kk][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < m && col < n) {
        T* dst = c + row * s.c_i + col * s.c_j;
        *dst = (T)(beta == 0.f ? alpha * acc : alpha * acc + beta * (float)*dst);
    }
}

template <typename T>
static cudaError_t launch_strided_gemm(const void* A, const void* Bm, void* Cm, int batch, int m, int n, int k, GemmStrides s,
                                       float alpha, float beta, cudaStream_t st)
{
    const dim3 grid((n + 15) / 16, (m + 15) / 16, batch), block(16, 16);
    strided_gemm_kernel<T><<<grid, block, 0, st>>>((const T*)A, (const T*)Bm, (T*)Cm, m, n, k, s, alpha, beta);
    return cudaPeekAtLastError();
}

// one warp per (b, h, q) row: softmax(scale * qk) over the columns the mask keeps
template <typename T>
__global__ void scale_mask_softmax_kernel(T* __restrict__ out, const T* __restrict__ qk, const T* __restrict__ mask, int H,
                                          int q_len, int k_len, float scale, size_t rows)
{
    const size_t r = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const size_t b = r / ((size_t)H * q_len);
    const int q = (int)(r % q_len);
    const T* in = qk + r * k_len;
    const T* m = mask + (b * q_len + q) * k_len;
    float mx = -INFINITY;
    for (int k = lane; k < k_len; k += 32)
        if ((float)m[k] != 0.f) mx = fmaxf(mx, scale * (float)in[k]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int k = lane; k < k_len; k += 32)
        if ((float)m[k] != 0.f) sum += expf(scale * (float)in[k] - mx);
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    for (int k = lane; k < k_len; k += 32)
        out[r * k_len + k] = (T)(((float)m[k] != 0.f) ? expf(scale * (float)in[k] - mx) * inv : 0.f);
}

template <typename T>
__global__ void transpose_remove_padding_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                const int* __restrict__ padding_offset, int B, int S, int H, int D)
{
    const int t = blockIdx.x;
    const int p = t + padding_offset[t];
    const int b = p / S, s = p % S;
    if (b >= B) return;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const int h = i / D, d = i % D;
        dst[(size_t)t * H * D + i] = src[(((size_t)b * H + h) * S + s) * D + d];
    }
}

}  // namespace onellm

using namespace onellm;

#define DISPATCH(dtype, who, F16_CALL, F32_CALL)                                   \
    do {                                                                           \
        note_launch();                                                             \
        if ((dtype) == ONELLM_F16) { F16_CALL; }                                   \
        else if ((dtype) == ONELLM_F32) { F32_CALL; }                              \
        else ONELLM_REQUIRE(false, ONELLM_ERR_UNSUPPORTED, who ": dtype %d", dtype); \
        ONELLM_CHECK_LAUNCH();                                                     \
    } while (0)

extern "C" int onellm_cal_padding_offset(int* padding_offset, int* cum_seqlens, const int* seq_lens, int B, int max_q_len,
                                         int* host_token_num, void* stream)
{
    ONELLM_REQUIRE(padding_offset && cum_seqlens && seq_lens, ONELLM_ERR_ARG, "cal_padding_offset: null pointer");
    ONELLM_REQUIRE(B >= 1 && B <= 64 && max_q_len >= 1, ONELLM_ERR_ARG, "cal_padding_offset: batch must be in [1,64]");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* d_total = nullptr;
    if (host_token_num) ONELLM_CUDA(cudaMallocAsync(&d_total, sizeof(int), st));
    note_launch();
    padding_offset_kernel<<<1, 256, 0, st>>>(padding_offset, cum_seqlens, seq_lens, B, max_q_len, d_total);
    ONELLM_CHECK_LAUNCH();
    if (host_token_num) {
        // unlike the reference (cal_paddingoffset.cu:42-45) the count is read back after the kernel has finished
        ONELLM_CUDA(cudaMemcpyAsync(host_token_num, d_total, sizeof(int), cudaMemcpyDeviceToHost, st));
        ONELLM_CUDA(cudaStreamSynchronize(st));
        ONELLM_CUDA(cudaFreeAsync(d_total, st));
    }
    return ONELLM_OK;
}

extern "C" int onellm_build_causal_mask(int dtype, void* mask, const int* q_lens, const int* k_lens, int max_q_len,
                                        int max_k_len, int B, int attend_history, void* stream)
{
    ONELLM_REQUIRE(mask && q_lens && k_lens && B > 0 && max_q_len > 0 && max_k_len > 0, ONELLM_ERR_ARG, "build_causal_mask: bad argument");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((max_q_len * max_k_len + 255) / 256 < 1024 ? (max_q_len * max_k_len + 255) / 256 : 1024, B);
    DISPATCH(dtype, "build_causal_mask",
             (causal_mask_kernel<__half><<<grid, 256, 0, st>>>((__half*)mask, q_lens, k_lens, max_q_len, max_k_len, attend_history)),
             (causal_mask_kernel<float><<<grid, 256, 0, st>>>((float*)mask, q_lens, k_lens, max_q_len, max_k_len, attend_history)));
    return ONELLM_OK;
}

extern "C" int onellm_qkv_bias_rope_transpose(int dtype, void* q_buf, void* k_buf, void* v_buf, const void* QKV, const void* bias,
                                              const int* padding_offset, const int* history_length, int B, int seq_len,
                                              int num_tokens, int H, int Hkv, int D, int rot_dim, float rope_base, void* stream)
{
    ONELLM_REQUIRE(q_buf && k_buf && v_buf && QKV && padding_offset && history_length, ONELLM_ERR_ARG, "qkv_bias_rope_transpose: null pointer");
    ONELLM_REQUIRE(B > 0 && seq_len > 0 && num_tokens >= 0 && H > 0 && Hkv > 0 && D > 0 && D % 2 == 0 && rot_dim / 2 <= kPairs &&
                       rope_base > 0.f,
                   ONELLM_ERR_ARG, "qkv_bias_rope_transpose: bad size");
    if (num_tokens == 0) return ONELLM_OK;
    RopeDenoms rd;
    const int r = rot_dim < D ? rot_dim : D;
    for (int i = 0; i < kPairs; i++) rd.d[i] = (2 * i < r) ? powf(rope_base, (float)(2 * i) / (float)rot_dim) : 1.f;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    DISPATCH(dtype, "qkv_bias_rope_transpose",
             (qkv_rope_transpose_kernel<__half><<<num_tokens, 256, 0, st>>>((__half*)q_buf, (__half*)k_buf, (__half*)v_buf, (const __half*)QKV,
                                                                          (const __half*)bias, padding_offset, history_length, B,
                                                                          seq_len, H, Hkv, D, r, rd)),
             (qkv_rope_transpose_kernel<float><<<num_tokens, 256, 0, st>>>((float*)q_buf, (float*)k_buf, (float*)v_buf, (const float*)QKV,
                                                                         (const float*)bias, padding_offset, history_length, B, seq_len,
                                                                         H, Hkv, D, r, rd)));
    return ONELLM_OK;
}

extern "C" int onellm_append_kv_cache(int dtype, void* dst, const void* src, const int* cur_query_length,
                                      const int* history_length, int B, int Hkv, int max_q_len, int max_seq_len, int D,
                                      int* overflow_flag, void* stream)
{
    ONELLM_REQUIRE(dst && src && cur_query_length && history_length, ONELLM_ERR_ARG, "append_kv_cache: null pointer");
    ONELLM_REQUIRE(B > 0 && Hkv > 0 && max_q_len > 0 && max_seq_len > 0 && D > 0 && B <= 65535 && Hkv <= 65535, ONELLM_ERR_ARG,
                   "append_kv_cache: bad size");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(max_q_len, B, Hkv);
    DISPATCH(dtype, "append_kv_cache",
             (append_kv_kernel<__half><<<grid, 128, 0, st>>>((__half*)dst, (const __half*)src, cur_query_length, history_length, Hkv,
                                                           max_q_len, max_seq_len, D, overflow_flag)),
             (append_kv_kernel<float><<<grid, 128, 0, st>>>((float*)dst, (const float*)src, cur_query_length, history_length, Hkv,
                                                          max_q_len, max_seq_len, D, overflow_flag)));
    return ONELLM_OK;
}

extern "C" int onellm_repeat_kv(int dtype, void* dst, const void* src, const int* context_length, int B, int H, int Hkv,
                                int max_k_len, int max_seq_len, int D, void* stream)
{
    ONELLM_REQUIRE(dst && src && context_length, ONELLM_ERR_ARG, "repeat_kv: null pointer");
    ONELLM_REQUIRE(B > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && max_k_len > 0 && max_k_len <= max_seq_len && D > 0 && B <= 65535 &&
                       H <= 65535,
                   ONELLM_ERR_ARG, "repeat_kv: bad size");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((max_k_len * D + 255) / 256, B, H);
    DISPATCH(dtype, "repeat_kv",
             (repeat_kv_kernel<__half><<<grid, 256, 0, st>>>((__half*)dst, (const __half*)src, context_length, H, Hkv, max_k_len, max_seq_len, D)),
             (repeat_kv_kernel<float><<<grid, 256, 0, st>>>((float*)dst, (const float*)src, context_length, H, Hkv, max_k_len, max_seq_len, D)));
    return ONELLM_OK;
}

extern "C" int onellm_batched_gemm(int dtype, const void* A, const void* Bm, void* Cm, int batch, int m, int n, int k, int trans_a,
                                   int trans_b, void* stream)
{
    ONELLM_REQUIRE(A && Bm && Cm && batch > 0 && m > 0 && n > 0 && k > 0 && batch <= 65535, ONELLM_ERR_ARG, "batched_gemm: bad argument");
    ONELLM_REQUIRE((m + 15) / 16 <= 65535, ONELLM_ERR_UNSUPPORTED, "batched_gemm: m too large");
    GemmStrides s;
    s.a_i = trans_a ? 1 : k;  s.a_k = trans_a ? m : 1;  s.a_b = (long)m * k;
    s.b_k = trans_b ? 1 : n;  s.b_j = trans_b ? k : 1;  s.b_b = (long)k * n;
    s.c_i = n;  s.c_j = 1;  s.c_b = (long)m * n;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    DISPATCH(dtype, "batched_gemm", (void)launch_strided_gemm<__half>(A, Bm, Cm, batch, m, n, k, s, 1.f, 0.f, st),
             (void)launch_strided_gemm<float>(A, Bm, Cm, batch, m, n, k, s, 1.f, 0.f, st));
    return ONELLM_OK;
}

extern "C" int onellm_gemm_strided_batched(int dtype, int trans_a, int trans_b, int m, int n, int k, const void* A, int lda,
                                           long stride_a, const void* Bm, int ldb, long stride_b, void* Cm, int ldc, long stride_c,
                                           int batch, float alpha, float beta, void* stream)
{
    ONELLM_REQUIRE(A && Bm && Cm && batch > 0 && m > 0 && n > 0 && k > 0 && batch <= 65535, ONELLM_ERR_ARG,
                   "gemm_strided_batched: bad argument");
    ONELLM_REQUIRE(lda >= (trans_a ? k : m) && ldb >= (trans_b ? n : k) && ldc >= m, ONELLM_ERR_ARG,
                   "gemm_strided_batched: leading dimension too small (lda %d ldb %d ldc %d)", lda, ldb, ldc);
    ONELLM_REQUIRE((m + 15) / 16 <= 65535, ONELLM_ERR_UNSUPPORTED, "gemm_strided_batched: m too large");
    GemmStrides s;  // column-major operands, as the BLAS convention has them
    s.a_i = trans_a ? lda : 1;  s.a_k = trans_a ? 1 : lda;  s.a_b = stride_a;
    s.b_k = trans_b ? ldb : 1;  s.b_j = trans_b ? 1 : ldb;  s.b_b = stride_b;
    s.c_i = 1;  s.c_j = ldc;  s.c_b = stride_c;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    DISPATCH(dtype, "gemm_strided_batched", (void)launch_strided_gemm<__half>(A, Bm, Cm, batch, m, n, k, s, alpha, beta, st),
             (void)launch_strided_gemm<float>(A, Bm, Cm, batch, m, n, k, s, alpha, beta, st));
    return ONELLM_OK;
}

extern "C" int onellm_scale_mask_softmax(int dtype, void* attn_score, const void* qk, const void* mask, int B, int H, int q_len,
                                         int k_len, float scale, void* stream)
{
    ONELLM_REQUIRE(attn_score && qk && mask && B > 0 && H > 0 && q_len > 0 && k_len > 0, ONELLM_ERR_ARG, "scale_mask_softmax: bad argument");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t rows = (size_t)B * H * q_len;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    DISPATCH(dtype, "scale_mask_softmax",
             (scale_mask_softmax_kernel<__half><<<blocks, 256, 0, st>>>((__half*)attn_score, (const __half*)qk, (const __half*)mask, H, q_len,
                                                                      k_len, scale, rows)),
             (scale_mask_softmax_kernel<float><<<blocks, 256, 0, st>>>((float*)attn_score, (const float*)qk, (const float*)mask, H, q_len, k_len,
                                                                     scale, rows)));
    return ONELLM_OK;
}

extern "C" int onellm_transpose_remove_padding(int dtype, void* dst, const void* src, const int* padding_offset, int num_tokens,
                                               int B, int S, int H, int D, void* stream)
{
    ONELLM_REQUIRE(dst && src && padding_offset && num_tokens >= 0 && B > 0 && S > 0 && H > 0 && D > 0, ONELLM_ERR_ARG,
                   "transpose_remove_padding: bad argument");
    if (num_tokens == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    DISPATCH(dtype, "transpose_remove_padding",
             (transpose_remove_padding_kernel<__half><<<num_tokens, 256, 0, st>>>((__half*)dst, (const __half*)src, padding_offset, B, S, H, D)),
             (transpose_remove_padding_kernel<float><<<num_tokens, 256, 0, st>>>((float*)dst, (const float*)src, padding_offset, B, S, H, D)));
    return ONELLM_OK;
}
