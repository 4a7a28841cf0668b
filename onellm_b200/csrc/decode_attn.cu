// Decode-step fused masked self-attention with RoPE for sm_100a: split-KV, HBM-bound.
//
// Replaces masked_MHA_kernel (src/kernels/decoder_masked_attn.cu:136-268 of the reference).
//
// Work split: grid = (n_split, H / G, B).  A thread block owns G query heads that share one
// KV head and one contiguous chunk of cached rows.  Inside the block a "lane group" of LPR
// lanes owns a row at a time: each lane holds 16 bytes of the row (8 halfs / 4 floats), so one
// warp load instruction fetches whole 128-byte lines; U rows of K and of V are in flight per
// lane group before the first is consumed.  Scores are reduced with xor-shuffles over the
// LPR lanes, the softmax is the running (max, sum) form kept in registers in the log2
// domain, and the V accumulator stays in registers.  Lane groups are merged through shared
// memory; splits are merged by a second, tiny kernel reading fp32 partials from scratch.
//
// The block that owns the last chunk also adds bias to the new k / v, rotates k, stores both
// in cache row step-1 and attends to them from registers, so no other block ever reads a row
// that is being written.  The RoPE denominators base^(2i/rot_dim) come in as kernel
// parameters computed by the host's powf, so the angle pos / denom is the same float the
// reference's CPU arithmetic produces.
#include <math.h>

#include <map>
#include <mutex>

#include "common.cuh"

namespace onellm {

constexpr int kMaxRopePairs = 128;     // D <= 256
constexpr int kAttnThreads = 128;      // 4 warps
constexpr int kRowsPerGroup = 2;       // U: rows a lane group takes from one stage
constexpr int kAttnStageBytes = 8192;  // K and V rows of one stage (always 256 + 256 chunks of 16 bytes)
constexpr int kMinChunkRows = 64;

struct DecodeAttnParams {
    const void *q, *k, *v;
    long q_sb, k_sb, v_sb;
    const void *bq, *bk, *bv;
    void *kc, *vc;
    long cs_b, cs_h, cs_s;
    int B, H, Hkv, D;
    int step;
    const int* step_dev;
    int rope_delta;  // position = step + rope_delta
    int rot_dim;
    float scale_log2e;
    void* out;
    long out_sb;
    float* part_acc;  // [B, H, n_split, D]
    float* part_ml;   // [B, H, n_split, 2]
    int n_split;      // grid.x
    int chunk;        // rows per split
    int nst;          // depth of the shared-memory ring
    float rope_denom[kMaxRopePairs];
};

__device__ __forceinline__ int effective_splits(int n_cached, int chunk)
{
    const int s = (n_cached + chunk - 1) / chunk;
    return s < 1 ? 1 : s;
}

template <typename T, int LPR, int G>
__global__ void __launch_bounds__(kAttnThreads) decode_attn_kernel(const DecodeAttnParams p)
{
    constexpr int VEC = Vec16<T>::N;
    constexpr int D = LPR * VEC;
    constexpr int GPW = 32 / LPR;                      // lane groups per warp
    constexpr int NG = (kAttnThreads / 32) * GPW;      // lane groups per block
    constexpr int U = kRowsPerGroup;
    constexpr int SR = NG * U;                         // rows per stage
    constexpr int ROWB = LPR * 16;                     // bytes per row

    const int split = blockIdx.x;
    const int h0 = blockIdx.y * G;  // first query head of this block
    const int b = blockIdx.z;
    const int qpk = p.H / p.Hkv;
    const int hk = h0 / qpk;
    const bool writes_cache = (h0 % qpk) == 0;

    const int step = p.step_dev ? *p.step_dev : p.step;
    const float pos = (float)(step + p.rope_delta);
    const int n_cached = step - 1;
    const int n_split = effective_splits(n_cached, p.chunk);
    if (split >= n_split) {
        pdl_launch_dependents();
        pdl_wait();
        return;
    }
    const bool owns_new = (split == n_split - 1);
    const int row0 = split * p.chunk;
    const int row1 = min(row0 + p.chunk, n_cached);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = warp * GPW + lane / LPR;
    const int d0 = (lane % LPR) * VEC;

    // rotation coefficients for this lane's pairs
    float cs[VEC / 2], sn[VEC / 2];
#pragma unroll
    for (int i = 0; i < VEC / 2; i++) {
        const int d = d0 + 2 * i;
        if (d < p.rot_dim) {
            const float ang = pos / p.rope_denom[d >> 1];
            sincosf(ang, &sn[i], &cs[i]);
        } else {
            cs[i] = 1.f;
            sn[i] = 0.f;
        }
    }

    float m[G], l[G], acc[G][VEC];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[g][i] = 0.f;
    }

    // K/V rows come through a ring of shared-memory stages filled by 16-byte cp.async copies
    // (each warp-wide copy covers whole 128-byte lines), so the bytes in flight per SM are set
    // by the ring depth, not by registers.  A stage holds SR rows of K, then SR rows of V.
    extern __shared__ __align__(16) unsigned char ring[];
    const uint32_t ring_base = (uint32_t)__cvta_generic_to_shared(ring);
    const T* kc = reinterpret_cast<const T*>(p.kc) + b * p.cs_b + hk * p.cs_h;
    const T* vc = reinterpret_cast<const T*>(p.vc) + b * p.cs_b + hk * p.cs_h;
    const int n_iter = row1 > row0 ? (row1 - row0 + SR - 1) / SR : 0;
    const int nst = p.nst;
    auto issue = [&](int it, int buf) {
        if (it < n_iter) {
            const int r0 = row0 + it * SR;
            const uint32_t sb = ring_base + (uint32_t)(buf * kAttnStageBytes);
#pragma unroll
            for (int i = 0; i < (SR * LPR) / kAttnThreads; i++) {
                const int c = threadIdx.x + kAttnThreads * i;
                const int row = c / LPR, ch = c % LPR;
                const int rr = r0 + row;
                const bool ok = rr < row1;
                const long off = ok ? (long)rr * p.cs_s + ch * VEC : 0;
                cp_async16(sb + row * ROWB + ch * 16, kc + off, ok ? 16 : 0);
                cp_async16(sb + (SR + row) * ROWB + ch * 16, vc + off, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };
    for (int s = 0; s < nst - 1; s++) issue(s, s);
    int buf = 0, fill = nst - 1;

    // Nothing above reads what the previous kernel in the stream wrote (cache rows below
    // step-1 are older than that); q, k and v do.  The next kernel is released after the main
    // loop: released earlier, its blocks would take residency this kernel's single wave needs.
    pdl_wait();

    // q: bias, rotate
    float qf[G][VEC];
#pragma unroll
    for (int g = 0; g < G; g++) {
        Vec16<T>::load(reinterpret_cast<const T*>(p.q) + b * p.q_sb + (long)(h0 + g) * D + d0, qf[g]);
        if (p.bq) {
            float bb[VEC];
            Vec16<T>::load(reinterpret_cast<const T*>(p.bq) + (long)(h0 + g) * D + d0, bb);
#pragma unroll
            for (int i = 0; i < VEC; i++) qf[g][i] += bb[i];
        }
#pragma unroll
        for (int i = 0; i < VEC / 2; i++) {
            const float x = qf[g][2 * i], y = qf[g][2 * i + 1];
            qf[g][2 * i] = cs[i] * x - sn[i] * y;
            qf[g][2 * i + 1] = cs[i] * y + sn[i] * x;
        }
    }


    // the trip count is the same for every thread: the barrier and the shuffles below are safe
    for (int it = 0; it < n_iter; it++) {
        cp_async_wait_dyn(nst - 2);
        __syncthreads();
        issue(it + nst - 1, fill);
        const unsigned char* sb = ring + buf * kAttnStageBytes;
        buf = buf + 1 == nst ? 0 : buf + 1;
        fill = fill + 1 == nst ? 0 : fill + 1;
        const int r = row0 + it * SR + grp;
        uint4 kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int srow = grp + u * NG;
            kk[u] = *reinterpret_cast<const uint4*>(sb + srow * ROWB + (lane % LPR) * 16);
            vv[u] = *reinterpret_cast<const uint4*>(sb + (SR + srow) * ROWB + (lane % LPR) * 16);
        }
        float s[U][G];
#pragma unroll
        for (int u = 0; u < U; u++) {
            float kf[VEC];
            Vec16<T>::unpack(kk[u], kf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; i++) a = fmaf(qf[g][i], kf[i], a);
                s[u][g] = a;
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int g = 0; g < G; g++) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
#pragma unroll
        for (int u = 0; u < U; u++) {
            const bool valid = (r + u * NG) < row1;
#pragma unroll
            for (int g = 0; g < G; g++) s[u][g] = valid ? s[u][g] * p.scale_log2e : -INFINITY;
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < U; u++) mn = fmaxf(mn, s[u][g]);
            // a lane group that has seen no valid row yet keeps m = -inf; subtract 0 then, so
            // that every exponent below is -inf (weight 0) instead of inf - inf
            const float ms = (mn == -INFINITY) ? 0.f : mn;
            const float corr = fast_exp2(m[g] - ms);
            m[g] = mn;
            l[g] *= corr;
#pragma unroll
            for (int i = 0; i < VEC; i++) acc[g][i] *= corr;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const float pr = fast_exp2(s[u][g] - ms);
                l[g] += pr;
                float vf[VEC];
                Vec16<T>::unpack(vv[u], vf);
#pragma unroll
                for (int i = 0; i < VEC; i++) acc[g][i] = fmaf(pr, vf[i], acc[g][i]);
            }
        }
    }

    cp_async_wait<0>();
    pdl_launch_dependents();

    // the new token's row: lane group 0 of the block that owns the last chunk
    if (owns_new && grp == 0) {
        // only lanes 0..LPR-1 of warp 0 are here
        constexpr unsigned kGroup0Mask = (LPR == 32) ? 0xffffffffu : ((1u << LPR) - 1u);
        float kf[VEC], vf[VEC];
        Vec16<T>::load(reinterpret_cast<const T*>(p.k) + b * p.k_sb + (long)hk * D + d0, kf);
        Vec16<T>::load(reinterpret_cast<const T*>(p.v) + b * p.v_sb + (long)hk * D + d0, vf);
        if (p.bk) {
            float bb[VEC];
            Vec16<T>::load(reinterpret_cast<const T*>(p.bk) + (long)hk * D + d0, bb);
#pragma unroll
            for (int i = 0; i < VEC; i++) kf[i] += bb[i];
        }
        if (p.bv) {
            float bb[VEC];
            Vec16<T>::load(reinterpret_cast<const T*>(p.bv) + (long)hk * D + d0, bb);
#pragma unroll
            for (int i = 0; i < VEC; i++) vf[i] += bb[i];
        }
#pragma unroll
        for (int i = 0; i < VEC / 2; i++) {
            const float x = kf[2 * i], y = kf[2 * i + 1];
            kf[2 * i] = cs[i] * x - sn[i] * y;
            kf[2 * i + 1] = cs[i] * y + sn[i] * x;
        }
        // attend to exactly what later steps will read back: the stored (rounded) values
        const uint4 kp = Vec16<T>::pack(kf), vp = Vec16<T>::pack(vf);
        if (writes_cache) {
            T* kd = reinterpret_cast<T*>(p.kc) + b * p.cs_b + hk * p.cs_h + (long)(step - 1) * p.cs_s + d0;
            T* vd = reinterpret_cast<T*>(p.vc) + b * p.cs_b + hk * p.cs_h + (long)(step - 1) * p.cs_s + d0;
            *reinterpret_cast<uint4*>(kd) = kp;
            *reinterpret_cast<uint4*>(vd) = vp;
        }
        Vec16<T>::unpack(kp, kf);
        Vec16<T>::unpack(vp, vf);
#pragma unroll
        for (int g = 0; g < G; g++) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; i++) a = fmaf(qf[g][i], kf[i], a);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) a += __shfl_xor_sync(kGroup0Mask, a, o);
            a *= p.scale_log2e;
            const float mn = fmaxf(m[g], a);
            const float corr = fast_exp2(m[g] - mn);
            const float pr = fast_exp2(a - mn);
            m[g] = mn;
            l[g] = l[g] * corr + pr;
#pragma unroll
            for (int i = 0; i < VEC; i++) acc[g][i] = fmaf(pr, vf[i], acc[g][i] * corr);
        }
    }

    // merge the lane groups of this block
    __shared__ float sm_acc[NG][G][D];
    __shared__ float sm_m[NG][G], sm_l[NG][G];
#pragma unroll
    for (int g = 0; g < G; g++) {
#pragma unroll
        for (int i = 0; i < VEC; i++) sm_acc[grp][g][d0 + i] = acc[g][i];
        if ((lane % LPR) == 0) {
            sm_m[grp][g] = m[g];
            sm_l[grp][g] = l[g];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
        const int g = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < NG; i++) M = fmaxf(M, sm_m[i][g]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int i = 0; i < NG; i++) {
            const float w = fast_exp2(sm_m[i][g] - M);  // empty groups: exp2(-inf) = 0
            L = fmaf(sm_l[i][g], w, L);
            O = fmaf(sm_acc[i][g][d], w, O);
        }
        const int h = h0 + g;
        if (n_split == 1) {
            reinterpret_cast<T*>(p.out)[b * p.out_sb + (long)h * D + d] = (T)(O / L);
        } else {
            const long base = ((long)b * p.H + h) * p.n_split + split;
            p.part_acc[base * D + d] = O;
            if (d == 0) {
                p.part_ml[base * 2] = M;
                p.part_ml[base * 2 + 1] = L;
            }
        }
    }
}

// Merges the per-split partials: out = sum_i O_i 2^(m_i - M) / sum_i L_i 2^(m_i - M).
template <typename T>
__global__ void decode_attn_combine_kernel(const DecodeAttnParams p)
{
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int step = p.step_dev ? *p.step_dev : p.step;
    const int n_split = effective_splits(step - 1, p.chunk);
    if (n_split == 1) return;  // the attention kernel wrote the output itself
    const long base = ((long)b * p.H + h) * p.n_split;
    float M = -INFINITY;
    for (int i = 0; i < n_split; i++) M = fmaxf(M, p.part_ml[(base + i) * 2]);
    float L = 0.f;
    for (int i = 0; i < n_split; i++)
        L = fmaf(p.part_ml[(base + i) * 2 + 1], fast_exp2(p.part_ml[(base + i) * 2] - M), L);
    const float invL = 1.f / L;
    for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
        float O = 0.f;
        for (int i = 0; i < n_split; i++)
            O = fmaf(p.part_acc[(base + i) * p.D + d], fast_exp2(p.part_ml[(base + i) * 2] - M), O);
        reinterpret_cast<T*>(p.out)[b * p.out_sb + (long)h * p.D + d] = (T)(O * invL);
    }
}

constexpr int kMaxSplits = 32;

// Upper bound on the splits any plan uses for `step` rows.
static int max_splits(int step)
{
    const int n_cached = step > 1 ? step - 1 : 0;
    int m = (n_cached + kMinChunkRows - 1) / kMinChunkRows;
    if (m < 1) m = 1;
    return m > kMaxSplits ? kMaxSplits : m;
}

struct AttnPlan {
    int n_split, chunk, nst;
    size_t dyn_smem;
};

// Splits, rows per split and ring depth for `step` rows.
//   regs_per_sm : blocks per SM the kernel's registers allow
//   static_smem : its static shared memory
//   row_bytes   : bytes of one K (or V) row; a stage holds kAttnStageBytes of K+V rows
// The bandwidth a launch reaches grows with the bytes it keeps in flight (resident blocks x
// ring depth x stage size, bounded by shared memory); a last wave of blocks that is nearly
// empty costs as much as a full one; every split adds partials to write and merge.  The
// plan enumerates (blocks per SM, splits) and takes the cheapest by that model.
static AttnPlan plan_attention(int B, int n_head_blocks, int step, int regs_per_sm, size_t static_smem,
                               size_t row_bytes)
{
    const int n_cached = step > 1 ? step - 1 : 0;
    const long base = (long)B * n_head_blocks;
    const int ms = max_splits(step);
    const int sms = num_sms();
    const int stage_rows = (int)(kAttnStageBytes / (2 * row_bytes));
    const double rows_per_us = 6.5e6 / (2.0 * (double)row_bytes);  // all blocks together, at peak
    AttnPlan best = {1, kMinChunkRows, 2, 2 * (size_t)kAttnStageBytes};
    double best_t = 1e30;
    for (int r = regs_per_sm; r >= 1; r--) {
        const long smem_block = (long)(227 * 1024) / r - (long)static_smem - 1024;
        int nst_cap = (int)(smem_block / kAttnStageBytes);
        if (nst_cap > kMaxStages) nst_cap = kMaxStages;
        if (nst_cap < 2) continue;
        const long slots = (long)r * sms;
        for (int n = 1; n <= ms; n++) {
            int c = (n_cached + n - 1) / n;
            c = (c + 31) / 32 * 32;
            if (c < kMinChunkRows) c = kMinChunkRows;
            int ns = (n_cached + c - 1) / c;
            if (ns < 1) ns = 1;
            const long total = base * ns;
            const long waves = (total + slots - 1) / slots;
            const long resident = total < slots ? total : slots;
            int nst = (c + stage_rows - 1) / stage_rows + 1;
            if (nst > nst_cap) nst = nst_cap;
            if (nst < 2) nst = 2;
            const double inflight = (double)resident * (nst - 1) * kAttnStageBytes;
            // share of peak bandwidth: bounded by the bytes in flight and by what one block can
            // consume (about 11.5 GB/s measured: its softmax chain is latency-bound)
            double bw = inflight / 28e6;
            const double by_blocks = (double)resident * 11.5e3 / 6.5e6;
            if (by_blocks < bw) bw = by_blocks;
            bw = bw > 1.0 ? 1.0 : (bw < 0.02 ? 0.02 : bw);
            // microseconds: streaming + per-block start-up per wave + merge of the partials
            const double t = (double)waves * ((double)resident * c / (rows_per_us * bw) + 1.5) +
                             (ns > 1 ? 2.5 + 0.05 * ns : 0.0);
            if (t < best_t) {
                best_t = t;
                best = {ns, c, nst, (size_t)nst * kAttnStageBytes};
            }
        }
    }
    return best;
}

static int pick_group(int qpk)
{
    if (qpk % 8 == 0) return 8;
    if (qpk % 4 == 0) return 4;
    if (qpk % 2 == 0) return 2;
    return 1;
}

using AttnKernel = void (*)(const DecodeAttnParams);

template <typename T, int LPR>
static AttnKernel attn_kernel_for(int G)
{
    switch (G) {
        case 8: return decode_attn_kernel<T, LPR, 8>;
        case 4: return decode_attn_kernel<T, LPR, 4>;
        case 2: return decode_attn_kernel<T, LPR, 2>;
        default: return decode_attn_kernel<T, LPR, 1>;
    }
}

template <typename T>
static AttnKernel attn_kernel_for(int lpr, int G)
{
    switch (lpr) {
        case 4: return attn_kernel_for<T, 4>(G);
        case 8: return attn_kernel_for<T, 8>(G);
        case 16: return attn_kernel_for<T, 16>(G);
        default: return attn_kernel_for<T, 32>(G);
    }
}

struct AttnKernelInfo {
    int blocks_per_sm_regs;  // residency allowed by registers and threads
    size_t static_smem;
};

// Per-kernel facts the planner needs (queried once; also raises the dynamic shared-memory cap).
static AttnKernelInfo kernel_info(AttnKernel k)
{
    static std::map<AttnKernel, AttnKernelInfo> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(k);
    if (it != cache.end()) return it->second;
    AttnKernelInfo info = {4, 4096};
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, k) == cudaSuccess) {
        info.static_smem = fa.sharedSizeBytes;
        int by_regs = fa.numRegs > 0 ? 65536 / (fa.numRegs * kAttnThreads) : 4;
        if (by_regs > 2048 / kAttnThreads) by_regs = 2048 / kAttnThreads;
        if (by_regs < 1) by_regs = 1;
        info.blocks_per_sm_regs = by_regs;
        (void)cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(227 * 1024 - fa.sharedSizeBytes));
    }
    (void)cudaGetLastError();
    cache[k] = info;
    return info;
}

}  // namespace onellm

using namespace onellm;

extern "C" size_t onellm_decode_attn_workspace_bytes(int B, int H, int D, int max_step)
{
    if (B <= 0 || H <= 0 || D <= 0 || max_step <= 0) return 0;
    const size_t worst = (size_t)B * H * max_splits(max_step) * (D + 2) * sizeof(float);
    return worst + 256;
}

extern "C" int onellm_decode_attn(int dtype, const void* q, const void* k, const void* v, long q_stride_b,
                                  long k_stride_b, long v_stride_b, const void* bias_q,
                                  const void* bias_k, const void* bias_v, void* k_cache, void* v_cache,
                                  long cs_b, long cs_h, long cs_s, int B, int H, int Hkv, int D, int step,
                                  const int* step_dev, int rope_pos, int rot_dim, float rope_base,
                                  float scale, void* out, long out_stride_b, void* workspace,
                                  size_t workspace_bytes, void* stream)
{
    ONELLM_REQUIRE(q && k && v && k_cache && v_cache && out, ONELLM_ERR_ARG, "decode_attn: null pointer");
    ONELLM_REQUIRE(B > 0 && H > 0 && Hkv > 0 && D > 0 && step > 0, ONELLM_ERR_ARG,
                   "decode_attn: non-positive size (B=%d H=%d Hkv=%d D=%d step=%d)", B, H, Hkv, D, step);
    ONELLM_REQUIRE(H % Hkv == 0, ONELLM_ERR_ARG, "decode_attn: H=%d is not a multiple of Hkv=%d", H, Hkv);
    const size_t es = dtype_size(dtype);
    ONELLM_REQUIRE(es != 0, ONELLM_ERR_UNSUPPORTED, "decode_attn: dtype %d", dtype);
    const size_t row_bytes = (size_t)D * es;
    ONELLM_REQUIRE(row_bytes == 64 || row_bytes == 128 || row_bytes == 256 || row_bytes == 512,
                   ONELLM_ERR_UNSUPPORTED, "decode_attn: head row of %zu bytes (need 64/128/256/512)",
                   row_bytes);
    ONELLM_REQUIRE(rot_dim >= 0 && rot_dim / 2 <= kMaxRopePairs && rope_base > 0.f, ONELLM_ERR_ARG,
                   "decode_attn: bad rotary parameters");
    const long vec = (long)(16 / es);
    ONELLM_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache) &&
                       aligned16(out) && (!bias_q || aligned16(bias_q)) && (!bias_k || aligned16(bias_k)) &&
                       (!bias_v || aligned16(bias_v)),
                   ONELLM_ERR_ARG, "decode_attn: pointers must be 16-byte aligned");
    ONELLM_REQUIRE(q_stride_b % vec == 0 && k_stride_b % vec == 0 && v_stride_b % vec == 0 &&
                       cs_b % vec == 0 && cs_h % vec == 0 && cs_s % vec == 0 && out_stride_b % vec == 0,
                   ONELLM_ERR_ARG, "decode_attn: strides must keep rows 16-byte aligned");

    DecodeAttnParams p;
    p.q = q; p.k = k; p.v = v;
    p.q_sb = q_stride_b; p.k_sb = k_stride_b; p.v_sb = v_stride_b;
    p.bq = bias_q; p.bk = bias_k; p.bv = bias_v;
    p.kc = k_cache; p.vc = v_cache;
    p.cs_b = cs_b; p.cs_h = cs_h; p.cs_s = cs_s;
    p.B = B; p.H = H; p.Hkv = Hkv; p.D = D;
    p.step = step;
    p.step_dev = step_dev;
    p.rope_delta = rope_pos - step;
    p.rot_dim = rot_dim < D ? rot_dim : D;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.out = out;
    p.out_sb = out_stride_b;
    for (int i = 0; i < kMaxRopePairs; i++)
        p.rope_denom[i] = (2 * i < p.rot_dim) ? powf(rope_base, (float)(2 * i) / (float)rot_dim) : 1.f;

    const int G = pick_group(H / Hkv);
    const int lpr = (int)(row_bytes / 16);
    const AttnKernel kern = dtype == ONELLM_F16 ? attn_kernel_for<__half>(lpr, G) : attn_kernel_for<float>(lpr, G);
    const AttnKernelInfo info = kernel_info(kern);
    const AttnPlan plan = plan_attention(B, H / G, step, info.blocks_per_sm_regs, info.static_smem, row_bytes);
    p.n_split = plan.n_split;
    p.chunk = plan.chunk;
    p.nst = plan.nst;
    p.part_acc = nullptr;
    p.part_ml = nullptr;
    if (p.n_split > 1) {
        const size_t need_acc = (size_t)B * H * p.n_split * D * sizeof(float);
        const size_t need = need_acc + (size_t)B * H * p.n_split * 2 * sizeof(float);
        ONELLM_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need, ONELLM_ERR_WORKSPACE,
                       "decode_attn: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        p.part_acc = reinterpret_cast<float*>(workspace);
        p.part_ml = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + need_acc);
    }
    ONELLM_REQUIRE(B <= 65535 && H / G <= 65535, ONELLM_ERR_UNSUPPORTED, "decode_attn: grid too large");

    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    ONELLM_CUDA(launch_pdl(kern, dim3(p.n_split, H / G, B), dim3(kAttnThreads), plan.dyn_smem, st, p));
    if (p.n_split > 1) {
        if (dtype == ONELLM_F16)
            ONELLM_CUDA(launch_pdl(decode_attn_combine_kernel<__half>, dim3(H, B), dim3(128), 0, st, p));
        else
            ONELLM_CUDA(launch_pdl(decode_attn_combine_kernel<float>, dim3(H, B), dim3(128), 0, st, p));
    }
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library hand every byte of device memory out themselves and are not able
// to call cudaMalloc for a kernel's scratch: a serving process whose memory pool was sized and
// pinned at start-up, a plugin running inside another framework's allocator, code running where
// the CUDA allocator must not be re-entered.  For them the split-KV partials of the attention
// kernel live in a fixed array inside the library image instead of a caller-provided workspace.
// Every GPU that loads the library holds these kStaticScratchBytes until the process exits.
//
// In host code `g_attn_scratch` is only a handle for the symbol, not a device address: passing it
// to a kernel would fault or silently use the wrong memory.  Its device address is looked up once
// per device with cudaGetSymbolAddress, with that device current, on the first call made on that
// device; that first call should therefore happen before any stream capture.
//
// All calls share the one array and it keeps the previous call's contents.  Nothing in it has to
// start at zero (every partial that is read was written by the same launch), but two calls that
// overlap on the GPU (different streams, or different host threads) race on it: serialise them.
// ---------------------------------------------------------------------------------------------
namespace onellm {
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticScratchBytes];

// device address of g_attn_scratch on the current device (looked up once per device)
static int static_scratch(void** out)
{
    constexpr int kMaxDevices = 64;
    static void* addr[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    ONELLM_CUDA(cudaGetDevice(&dev));
    ONELLM_REQUIRE(dev >= 0 && dev < kMaxDevices, ONELLM_ERR_UNSUPPORTED, "decode_attn_static: device index %d", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        ONELLM_CUDA(cudaGetSymbolAddress(&p, g_attn_scratch));
        addr[dev] = p;
    }
    *out = addr[dev];
    return ONELLM_OK;
}
}  // namespace onellm

extern "C" size_t onellm_decode_attn_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int onellm_decode_attn_static(int dtype, const void* q, const void* k, const void* v, long q_stride_b,
                                         long k_stride_b, long v_stride_b, const void* bias_q, const void* bias_k,
                                         const void* bias_v, void* k_cache, void* v_cache, long cs_b, long cs_h,
                                         long cs_s, int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         int rope_pos, int rot_dim, float rope_base, float scale, void* out,
                                         long out_stride_b, void* stream)
{
    // The bound is the documented worst case for the shape, not what this launch happens to use,
    // so that a shape is either always accepted or always refused.
    const size_t bound = onellm_decode_attn_workspace_bytes(B, H, D, step);
    ONELLM_REQUIRE(bound != 0 && bound <= kStaticScratchBytes, ONELLM_ERR_WORKSPACE,
                   "decode_attn_static: B=%d H=%d D=%d step=%d may need %zu bytes of split-KV scratch, the array "
                   "built into the library holds %zu; use onellm_decode_attn with a caller workspace",
                   B, H, D, step, bound, kStaticScratchBytes);
    void* scratch = nullptr;
    const int rc0 = static_scratch(&scratch);
    if (rc0) return rc0;
    const int rc = onellm_decode_attn(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache,
                                      v_cache, cs_b, cs_h, cs_s, B, H, Hkv, D, step, step_dev, rope_pos, rot_dim,
                                      rope_base, scale, out, out_stride_b, scratch, kStaticScratchBytes, stream);
    return rc;
}
