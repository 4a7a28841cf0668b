// Context-phase (prefill) kernels for sm_100a: QKV bias + RoPE + KV-cache write, and causal attention.
//
// Together they replace, for one layer, the reference's chain
//   launchAddFusedQKVBiasTransposeAndRoPE  (src/kernels/qkv_bias_and_RoPE.cu:74-207)
//   launchAppendKVCache                     (src/kernels/append_to_kvcache.cu:8-114)
//   launchTransposeKVCache                  (src/kernels/transpose_kernel.cu:7-88)
//   launchLinearStridedBatchGemm x2, launchScaleMaskAndSoftmax, launchBuildCausalMasks
//                                           (src/kernels/qkv_linear.cu:67-120, attn_softmax_kernel.cu:45-176,
//                                            build_casual_mask.cu:27-60)
//   launchTransposeOutRemovePadding         (src/kernels/fused_transpose_reshape_remv_pad.cu:5-51)
// as sequenced by LLaMAContextAttentionLayer::forward (src/layers/attention/context_attention.cpp:101-158),
// without the padded / transposed / repeated copies and without the [B,H,Sq,Sk] score matrix:
//   1. qkv_rope_kvcache_kernel: q <- RoPE(q + bias) in place in the packed [T, H+2Hkv, D] buffer;
//      k <- RoPE(k + bias), v <- v + bias written straight into the layer's cache at row
//      history + local position.  HBM-bound, one pass.
//   2. context_attn_kernel: flash-style attention with mma.m16n8k16: a block owns 64 query rows of one
//      (sequence, head), streams 64-row K/V tiles of the cache through a cp.async double buffer, keeps
//      the running softmax and the output in registers, reads the KV head h / (H/Hkv) directly and
//      writes [T, H*D].  Token i of a sequence attends cache rows 0 .. history + i (causal predicate
//      of build_casual_mask.cu:40-43 with the history columns attended).
#include <math.h>

#include "common.cuh"

namespace onellm {

constexpr int kMaxPairs = 128;

struct RopeTable {
    float denom[kMaxPairs];
};

// token t of the packed batch -> (sequence b, local index i) by scanning cu_seqlens [B+1]
__device__ __forceinline__ void locate_token(const int* __restrict__ cu, int B, int t, int& b, int& i)
{
    b = 0;
    while (b + 1 < B && t >= cu[b + 1]) b++;
    i = t - cu[b];
}

template <typename T>
__global__ void __launch_bounds__(256)
qkv_rope_kvcache_kernel(T* __restrict__ qkv, const T* __restrict__ bias, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ history, T* __restrict__ k_cache, T* __restrict__ v_cache, long cs_b,
                        long cs_h, long cs_s, int B, int H, int Hkv, int D, int rot_dim, int max_seq, const RopeTable rt,
                        int* __restrict__ overflow_flag)
{
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int b, i;
    locate_token(cu_seqlens, B, t, b, i);
    const int pos = history[b] + i;
    if (pos >= max_seq) {  // the cache has no such row: record it, leave q alone
        if (threadIdx.x == 0 && overflow_flag) atomicExch(overflow_flag, 1);
        return;
    }
    const int QH = H + 2 * Hkv, half_d = D / 2;
    T* row = qkv + (size_t)t * QH * D;
    for (int idx = threadIdx.x; idx < QH * half_d; idx += blockDim.x) {
        const int head = idx / half_d, pr = idx % half_d;
        float x = (float)row[head * D + 2 * pr], y = (float)row[head * D + 2 * pr + 1];
        if (bias) {
            x += (float)bias[head * D + 2 * pr];
            y += (float)bias[head * D + 2 * pr + 1];
        }
        if (head < H + Hkv && 2 * pr < rot_dim) {  // q and k heads rotate, v heads do not
            float sn, cs;
            sincosf((float)pos / rt.denom[pr], &sn, &cs);
            const float xr = cs * x - sn * y, yr = cs * y + sn * x;
            x = xr;
            y = yr;
        }
        if (head < H) {
            row[head * D + 2 * pr] = (T)x;
            row[head * D + 2 * pr + 1] = (T)y;
        } else {
            const int hk = head < H + Hkv ? head - H : head - H - Hkv;
            T* dst = (head < H + Hkv ? k_cache : v_cache) + b * cs_b + hk * cs_h + (long)pos * cs_s + 2 * pr;
            dst[0] = (T)x;
            dst[1] = (T)y;
        }
    }
}

// The same with 16-byte accesses and one sincosf per (token, pair) instead of one per (token, head, pair):
// the angles of a token are shared by all its heads, and sincosf on arguments of thousands of radians is
// the slow path of the math library.  Needs D, the cache strides and all pointers aligned to 16 bytes.
template <typename T>
__global__ void __launch_bounds__(256)
qkv_rope_kvcache_vec_kernel(T* __restrict__ qkv, const T* __restrict__ bias, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ history, T* __restrict__ k_cache, T* __restrict__ v_cache, long cs_b,
                            long cs_h, long cs_s, int B, int H, int Hkv, int D, int rot_dim, int max_seq, const RopeTable rt,
                            int* __restrict__ overflow_flag)
{
    constexpr int N = Vec16<T>::N;
    __shared__ float s_sin[kMaxPairs], s_cos[kMaxPairs];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int b, i;
    locate_token(cu_seqlens, B, t, b, i);
    const int pos = history[b] + i;
    if (pos >= max_seq) {  // the cache has no such row: record it, leave q alone
        if (threadIdx.x == 0 && overflow_flag) atomicExch(overflow_flag, 1);
        return;
    }
    const int QH = H + 2 * Hkv, half_d = D / 2;
    for (int pr = threadIdx.x; pr < half_d; pr += blockDim.x) {
        float sn = 0.f, cs = 1.f;  // pairs beyond the rotary dimension pass through
        if (2 * pr < rot_dim) sincosf((float)pos / rt.denom[pr], &sn, &cs);
        s_sin[pr] = sn;
        s_cos[pr] = cs;
    }
    __syncthreads();
    T* row = qkv + (size_t)t * QH * D;
    const int vec_per_head = D / N;
    for (int idx = threadIdx.x; idx < QH * vec_per_head; idx += blockDim.x) {
        const int head = idx / vec_per_head, e0 = (idx % vec_per_head) * N;
        float f[N];
        Vec16<T>::load(row + head * D + e0, f);
        if (bias) {
            float bb[N];
            Vec16<T>::load(bias + head * D + e0, bb);
#pragma unroll
            for (int e = 0; e < N; e++) f[e] += bb[e];
        }
        if (head < H + Hkv) {  // q and k heads rotate, v heads do not
#pragma unroll
            for (int p = 0; p < N / 2; p++) {
                const float cs = s_cos[e0 / 2 + p], sn = s_sin[e0 / 2 + p];
                const float x = f[2 * p], y = f[2 * p + 1];
                f[2 * p] = cs * x - sn * y;
                f[2 * p + 1] = cs * y + sn * x;
            }
        }
        T* dst;
        if (head < H) {
            dst = row + head * D + e0;
        } else {
            const int hk = head < H + Hkv ? head - H : head - H - Hkv;
            dst = (head < H + Hkv ? k_cache : v_cache) + b * cs_b + hk * cs_h + (long)pos * cs_s + e0;
        }
        *reinterpret_cast<uint4*>(dst) = Vec16<T>::pack(f);
    }
}

// ---- causal attention over the cache, fp16, D = 64 or 128 ---------------------------------------------
constexpr int kCtxQ = 64;    // query rows per block (4 warps x 16)
constexpr int kCtxKV = 64;   // cache rows per tile

template <int D>
__global__ void __launch_bounds__(128)
context_attn_kernel(const __half* __restrict__ q, long q_ld, const __half* __restrict__ k_cache,
                    const __half* __restrict__ v_cache, long cs_b, long cs_h, long cs_s,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ history, int H, int Hkv, float scale_log2e,
                    __half* __restrict__ out)
{
    constexpr int ROWB = D * 2, CH = D / 8, KS = D / 16;
    constexpr int QT = kCtxQ * ROWB;           // Q tile bytes
    constexpr int KVT = 2 * kCtxKV * ROWB;     // K tile then V tile
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sKV = sQ + QT;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (H / Hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    pdl_launch_dependents();
    pdl_wait();
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0, hist = history[b];
    const int q0 = blockIdx.x * kCtxQ;
    if (q0 >= q_len) return;
    const int q_rows = min(kCtxQ, q_len - q0);
    const int kv_end = hist + q0 + q_rows;  // rows any query of this block may attend
    const int n_tiles = (kv_end + kCtxKV - 1) / kCtxKV;
    const __half* kc = k_cache + b * cs_b + hk * cs_h;
    const __half* vc = v_cache + b * cs_b + hk * cs_h;

    // Q tile (rows beyond the sequence are zero) and the first K/V tile
    for (int c = threadIdx.x; c < kCtxQ * CH; c += 128) {
        const int r = c / CH, ch = c % CH;
        const bool ok = r < q_rows;
        const __half* src = ok ? q + (size_t)(tok0 + q0 + r) * q_ld + (size_t)h * D + ch * 8 : q;
        cp_async16(sQ + r * ROWB + ((ch ^ (r & 7)) << 4), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int tile, int buf) {
        if (tile < n_tiles) {
            const uint32_t sb = sKV + (uint32_t)(buf * KVT);
            for (int c = threadIdx.x; c < kCtxKV * CH; c += 128) {
                const int r = c / CH, ch = c % CH;
                const int rr = tile * kCtxKV + r;
                const bool ok = rr < kv_end;
                const long off = ok ? (long)rr * cs_s + ch * 8 : 0;
                const uint32_t dst = sb + r * ROWB + ((ch ^ (r & 7)) << 4);
                cp_async16(dst, kc + off, ok ? 16 : 0);
                cp_async16(dst + kCtxKV * ROWB, vc + off, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };
    load_kv(0, 0);  // group 0 also carries the Q tile

    // per-lane ldmatrix coordinates
    const int lr = lane & 7, mi = lane >> 3;
    const int a_row = warp * 16 + lr + (mi & 1) * 8, a_chunk = mi >> 1;   // Q: (rows 0-7 | 8-15) x (chunk 2ks | 2ks+1)
    const int k_row = lr + (mi >> 1) * 8, k_chunk = mi & 1;                // K: two 8-row n tiles x two chunks
    const int v_row = lr + (mi & 1) * 8, v_chunk = mi >> 1;                // V (transposed): 16 rows x two chunks

    float O[2 * KS][4];
#pragma unroll
    for (int j = 0; j < 2 * KS; j++) O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8 of this warp's 16
    uint32_t qa[KS][4];
    const int qpos0 = hist + q0 + warp * 16 + g;  // cache row of query row g (row g+8: +8)

    for (int tile = 0; tile < n_tiles; tile++) {
        load_kv(tile + 1, (tile + 1) & 1);
        cp_async_wait<1>();
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const int c = 2 * ks + a_chunk;
                ldsm_x4(qa[ks], sQ + a_row * ROWB + ((c ^ (a_row & 7)) << 4));
            }
        }
        const uint32_t sb = sKV + (uint32_t)((tile & 1) * KVT);
        const int kv0 = tile * kCtxKV;
        // a warp whose 16 queries all precede this tile has nothing to add (causal)
        if (kv0 <= hist + q0 + warp * 16 + 15) {
            float S[kCtxKV / 8][4];
#pragma unroll
            for (int j = 0; j < kCtxKV / 8; j++) S[j][0] = S[j][1] = S[j][2] = S[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
#pragma unroll
                for (int jj = 0; jj < kCtxKV / 16; jj++) {
                    uint32_t kb[4];
                    const int r = 16 * jj + k_row, c = 2 * ks + k_chunk;
                    ldsm_x4(kb, sb + r * ROWB + ((c ^ (r & 7)) << 4));
                    mma_f16(S[2 * jj], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
                    mma_f16(S[2 * jj + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
                }
            }
            // scale, causal mask, running softmax (log2 domain) for rows g and g+8
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < kCtxKV / 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int kv = kv0 + 8 * j + 2 * t + (e & 1);
                    const int qp = qpos0 + ((e & 2) ? 8 : 0);
                    const float s = (kv <= qp) ? S[j][e] * scale_log2e : -INFINITY;
                    S[j][e] = s;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s);
                }
            float corr[2], ms[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float mn = fmaxf(m_run[r], mx[r]);
                ms[r] = (mn == -INFINITY) ? 0.f : mn;
                corr[r] = fast_exp2(m_run[r] - ms[r]);
                m_run[r] = mn;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int j = 0; j < kCtxKV / 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float pv = fast_exp2(S[j][e] - ms[e >> 1]);
                    S[j][e] = pv;
                    l_run[e >> 1] += pv;
                }
#pragma unroll
            for (int j = 0; j < 2 * KS; j++) {
                O[j][0] *= corr[0];
                O[j][1] *= corr[0];
                O[j][2] *= corr[1];
                O[j][3] *= corr[1];
            }
            // O += P . V
#pragma unroll
            for (int kk = 0; kk < kCtxKV / 16; kk++) {
                const uint32_t pa0 = pack_h2(S[2 * kk][0], S[2 * kk][1]), pa1 = pack_h2(S[2 * kk][2], S[2 * kk][3]);
                const uint32_t pa2 = pack_h2(S[2 * kk + 1][0], S[2 * kk + 1][1]), pa3 = pack_h2(S[2 * kk + 1][2], S[2 * kk + 1][3]);
#pragma unroll
                for (int jp = 0; jp < KS; jp++) {
                    uint32_t vb[4];
                    const int r = 16 * kk + v_row, c = 2 * jp + v_chunk;
                    ldsm_x4_t(vb, sb + (kCtxKV + r) * ROWB + ((c ^ (r & 7)) << 4));
                    mma_f16(O[2 * jp], pa0, pa1, pa2, pa3, vb[0], vb[1]);
                    mma_f16(O[2 * jp + 1], pa0, pa1, pa2, pa3, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();  // the other buffer is refilled at the top of the next iteration
    }
    cp_async_wait<0>();

    // normalise and store rows g and g+8
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int qi = warp * 16 + g + 8 * r;
        if (qi < q_rows) {
            const float inv = 1.f / l_run[r];
            __half* dst = out + ((size_t)(tok0 + q0 + qi) * H + h) * D;
#pragma unroll
            for (int j = 0; j < 2 * KS; j++)
                *reinterpret_cast<__half2*>(dst + 8 * j + 2 * t) = __floats2half2_rn(O[j][2 * r] * inv, O[j][2 * r + 1] * inv);
        }
    }
}

static void fill_rope(RopeTable& rt, int rot_dim, float base)
{
    for (int i = 0; i < kMaxPairs; i++) rt.denom[i] = (2 * i < rot_dim) ? powf(base, (float)(2 * i) / (float)rot_dim) : 1.f;
}

// context_attn_tc.cu
int context_attn_tc_launch(const __half* q, long q_ld, const __half* k_cache, const __half* v_cache, int S_max, long cache_rows,
                           const int* cu_seqlens, const int* history, int B, int max_q_len, int H, int Hkv, float scale, __half* out,
                           cudaStream_t st);

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_qkv_bias_rope_kvcache(int dtype, void* qkv, const void* bias, const int* cu_seqlens,
                                            const int* history_length, void* k_cache, void* v_cache, long cs_b, long cs_h,
                                            long cs_s, int num_tokens, int B, int H, int Hkv, int D, int rot_dim,
                                            float rope_base, int max_seq_len, int* overflow_flag, void* stream)
{
    ONELLM_REQUIRE(qkv && cu_seqlens && history_length && k_cache && v_cache, ONELLM_ERR_ARG, "qkv_bias_rope_kvcache: null pointer");
    ONELLM_REQUIRE(num_tokens >= 0 && B > 0 && H > 0 && Hkv > 0 && D > 0 && D % 2 == 0 && max_seq_len > 0, ONELLM_ERR_ARG,
                   "qkv_bias_rope_kvcache: bad size");
    ONELLM_REQUIRE(rot_dim >= 0 && rot_dim / 2 <= kMaxPairs && rope_base > 0.f, ONELLM_ERR_ARG,
                   "qkv_bias_rope_kvcache: bad rotary parameters");
    ONELLM_REQUIRE(dtype == ONELLM_F16 || dtype == ONELLM_F32, ONELLM_ERR_UNSUPPORTED, "qkv_bias_rope_kvcache: dtype %d", dtype);
    if (num_tokens == 0) return ONELLM_OK;
    RopeTable rt;
    fill_rope(rt, rot_dim < D ? rot_dim : D, rope_base);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int rd = rot_dim < D ? rot_dim : D;
    const long vec = dtype == ONELLM_F16 ? 8 : 4;  // elements per 16 bytes
    const bool aligned = D % vec == 0 && cs_b % vec == 0 && cs_h % vec == 0 && cs_s % vec == 0 && aligned16(qkv) && aligned16(k_cache) &&
                         aligned16(v_cache) && (!bias || aligned16(bias));
    if (dtype == ONELLM_F16)
        ONELLM_CUDA(launch_pdl(aligned ? qkv_rope_kvcache_vec_kernel<__half> : qkv_rope_kvcache_kernel<__half>, dim3(num_tokens), dim3(256), 0,
                               st, (__half*)qkv, (const __half*)bias, cu_seqlens, history_length, (__half*)k_cache, (__half*)v_cache,
                               cs_b, cs_h, cs_s, B, H, Hkv, D, rd, max_seq_len, rt, overflow_flag));
    else
        ONELLM_CUDA(launch_pdl(aligned ? qkv_rope_kvcache_vec_kernel<float> : qkv_rope_kvcache_kernel<float>, dim3(num_tokens), dim3(256), 0,
                               st, (float*)qkv, (const float*)bias, cu_seqlens, history_length, (float*)k_cache, (float*)v_cache, cs_b,
                               cs_h, cs_s, B, H, Hkv, D, rd, max_seq_len, rt, overflow_flag));
    return ONELLM_OK;
}

extern "C" int onellm_context_attn(int dtype, const void* q, long q_ld, const void* k_cache, const void* v_cache, long cs_b,
                                   long cs_h, long cs_s, const int* cu_seqlens, const int* history_length, int B,
                                   int max_q_len, int H, int Hkv, int D, float scale, void* out, void* stream)
{
    ONELLM_REQUIRE(q && k_cache && v_cache && cu_seqlens && history_length && out, ONELLM_ERR_ARG, "context_attn: null pointer");
    ONELLM_REQUIRE(B > 0 && max_q_len > 0 && H > 0 && Hkv > 0 && H % Hkv == 0, ONELLM_ERR_ARG, "context_attn: bad size");
    ONELLM_REQUIRE(dtype == ONELLM_F16 && (D == 64 || D == 128), ONELLM_ERR_UNSUPPORTED,
                   "context_attn: fp16 with head size 64 or 128 only");
    ONELLM_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && aligned16(out) && q_ld % 8 == 0 &&
                       cs_b % 8 == 0 && cs_h % 8 == 0 && cs_s % 8 == 0,
                   ONELLM_ERR_ARG, "context_attn: pointers and strides must keep rows 16-byte aligned");
    ONELLM_REQUIRE(B <= 65535 && H <= 65535, ONELLM_ERR_UNSUPPORTED, "context_attn: grid too large");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // head size 128 and the cache in its standard [B, Hkv, S, D] order: tcgen05 tiles (context_attn_tc.cu)
    if (D == 128 && cs_s == D && cs_h % D == 0 && cs_b == (long)Hkv * cs_h && max_q_len >= 32)
        return context_attn_tc_launch((const __half*)q, q_ld, (const __half*)k_cache, (const __half*)v_cache, (int)(cs_h / D),
                                      (long)B * Hkv * (cs_h / D), cu_seqlens, history_length, B, max_q_len, H, Hkv, scale, (__half*)out, st);
    const dim3 grid((max_q_len + kCtxQ - 1) / kCtxQ, H, B);
    const float sl = scale * 1.4426950408889634f;
    static DeviceOnce attr64, attr128;
    if (D == 128) {
        const size_t smem = (size_t)kCtxQ * 256 + 2 * 2 * kCtxKV * 256;
        ONELLM_CUDA(attr128.run([smem] { return cudaFuncSetAttribute(context_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
        ONELLM_CUDA(launch_pdl(context_attn_kernel<128>, grid, dim3(128), smem, st, (const __half*)q, q_ld, (const __half*)k_cache,
                               (const __half*)v_cache, cs_b, cs_h, cs_s, cu_seqlens, history_length, H, Hkv, sl, (__half*)out));
    } else {
        const size_t smem = (size_t)kCtxQ * 128 + 2 * 2 * kCtxKV * 128;
        ONELLM_CUDA(attr64.run([smem] { return cudaFuncSetAttribute(context_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }));
        ONELLM_CUDA(launch_pdl(context_attn_kernel<64>, grid, dim3(128), smem, st, (const __half*)q, q_ld, (const __half*)k_cache,
                               (const __half*)v_cache, cs_b, cs_h, cs_s, cu_seqlens, history_length, H, Hkv, sl, (__half*)out));
    }
    return ONELLM_OK;
}
