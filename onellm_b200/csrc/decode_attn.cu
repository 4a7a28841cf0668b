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
    const int* step_offset;  // optional, per sequence: its step is the common step + step_offset[b] (<= 0)
    int rope_delta;  // position = step + rope_delta
    int rot_dim;
    float scale_log2e;
    void* out;
    long out_sb;
    float* part_acc;  // [B, H, n_split, D]
    float* part_ml;   // [B, H, n_split, 2]
    int* tickets;     // optional [B, H / G], zero between launches: the last block of a (sequence, head group) to
                      // arrive merges the splits itself and no merge kernel follows
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

// Split launches without a merge kernel.  Every block of a (sequence, head group) takes a ticket once its partials
// are written and fenced; the one that draws the last ticket knows that all the others' partials are visible, merges
// them (the arithmetic of decode_attn_combine_kernel, operation for operation: the results are bit-identical) and
// puts the ticket counter back to zero for the next launch.  Nobody waits for anybody.  The partials are read
// past L1 (ld.cg): the same addresses held an earlier launch's partials.  Called by all threads of the block.
template <typename T>
__device__ __forceinline__ void merge_by_last_block(const DecodeAttnParams& p, int b, int h0, int G, int n_split)
{
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* t = p.tickets + (size_t)b * gridDim.y + blockIdx.y;
        const int last = atomicAdd(t, 1) == n_split - 1;
        if (last) atomicExch(t, 0);
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * p.D; idx += blockDim.x) {
        const int h = h0 + idx / p.D, d = idx % p.D;
        const long base = ((long)b * p.H + h) * p.n_split;
        float M = -INFINITY;
        for (int i = 0; i < n_split; i++) M = fmaxf(M, __ldcg(&p.part_ml[(base + i) * 2]));
        float L = 0.f;
        for (int i = 0; i < n_split; i++)
            L = fmaf(__ldcg(&p.part_ml[(base + i) * 2 + 1]), fast_exp2(__ldcg(&p.part_ml[(base + i) * 2]) - M), L);
        const float invL = 1.f / L;
        float O = 0.f;
        for (int i = 0; i < n_split; i++)
            O = fmaf(__ldcg(&p.part_acc[(base + i) * p.D + d]), fast_exp2(__ldcg(&p.part_ml[(base + i) * 2]) - M), O);
        reinterpret_cast<T*>(p.out)[b * p.out_sb + (long)h * p.D + d] = (T)(O * invL);
    }
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

    const int step = (p.step_dev ? *p.step_dev : p.step) + (p.step_offset ? p.step_offset[b] : 0);
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
    if (n_split > 1 && p.tickets) merge_by_last_block<T>(p, b, h0, G, n_split);
}

// Merges the per-split partials: out = sum_i O_i 2^(m_i - M) / sum_i L_i 2^(m_i - M).
template <typename T>
__global__ void decode_attn_combine_kernel(const DecodeAttnParams p)
{
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int step = (p.step_dev ? *p.step_dev : p.step) + (p.step_offset ? p.step_offset[b] : 0);
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

// ---------------------------------------------------------------------------------------------
// Tensor-core variant for fp16 caches with D = 64 or 128.
//
// Same contract as decode_attn_kernel.  The SIMT kernel above spends ~45 instructions per row
// and lane group on conversions, FMAs and shuffles and ends up bounded by instruction issue
// (67 % issue-slot use at 5.2 TB/s); here a warp handles a 16-row tile with 2 * D/8 mma.m16n8k16:
//   S^T[head, row] = q[head, :] . K[row, :]^T      (A = q from registers, B = K rows via ldmatrix)
//   O[head, :]    += P[head, row] . V[row, :]      (A = P straight from the S accumulators,
//                                                   B = V rows via ldmatrix.trans)
// The up to 8 query heads that share a KV head sit on the M axis (rows 8..15 of every tile are
// padding), so K and V are read once per group.  Each WARP owns a contiguous range of the
// block's rows and its own ring of cp.async stages: there is no block-wide barrier in the main
// loop.  With about two blocks per SM the whole context of a (sequence, KV head) pair fits one
// block, so large batches need no split and no merge kernel.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaWarps = 4;
constexpr int kMmaTileRows = 16;

template <int D, int G>
__global__ void __launch_bounds__(kMmaWarps * 32) decode_attn_mma_kernel(const DecodeAttnParams p)
{
    constexpr int ROWB = D * 2;                       // bytes per K or V row
    constexpr int CH = D / 8;                         // 16-byte chunks per row
    constexpr int TILE = 2 * kMmaTileRows * ROWB;     // K rows then V rows of one stage
    constexpr int KS = D / 16;                        // k-steps of q.K^T, pairs of d tiles of P.V
    constexpr int EPL = D / 32;                       // elements of a row per lane (new-row path)
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(16) __half q_s[8][D];
    __shared__ float sm_m[kMmaWarps][G], sm_l[kMmaWarps][G];
    // per-warp accumulators for the final merge reuse the ring once the main loop is over
    float (*sm_acc)[G][D] = reinterpret_cast<float (*)[G][D]>(ring);

    const int split = blockIdx.x;
    const int h0 = blockIdx.y * G;
    const int b = blockIdx.z;
    const int qpk = p.H / p.Hkv;
    const int hk = h0 / qpk;
    const bool writes_cache = (h0 % qpk) == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    const int step = (p.step_dev ? *p.step_dev : p.step) + (p.step_offset ? p.step_offset[b] : 0);
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
    const int row1 = min(row0 + p.chunk, n_cached) + (owns_new ? 1 : 0);  // the new row rides at the end
    // rows of this warp: contiguous, whole tiles except at the end
    const int rows_total = row1 - row0;
    int per_warp = (rows_total + kMmaWarps - 1) / kMmaWarps;
    per_warp = (per_warp + kMmaTileRows - 1) / kMmaTileRows * kMmaTileRows;
    const int wr0 = min(row0 + warp * per_warp, row1);
    const int wr1 = min(wr0 + per_warp, row1);
    const int n_tiles = (wr1 - wr0 + kMmaTileRows - 1) / kMmaTileRows;

    const __half* kc = reinterpret_cast<const __half*>(p.kc) + b * p.cs_b + hk * p.cs_h;
    const __half* vc = reinterpret_cast<const __half*>(p.vc) + b * p.cs_b + hk * p.cs_h;
    const int nst = p.nst;
    const uint32_t ring_base = (uint32_t)__cvta_generic_to_shared(ring) + (uint32_t)(warp * nst * TILE);
    unsigned char* ring_gen = ring + (size_t)warp * nst * TILE;

    // this lane's copies of a tile: chunk id = lane + 32*i -> row id/CH, chunk id%CH (a warp-wide
    // copy covers whole rows); rows at or beyond n_cached are not in the cache yet: zero-filled
    auto issue = [&](int tile, int buf) {
        if (tile < n_tiles) {
            const int r0 = wr0 + tile * kMmaTileRows;
            const uint32_t sb = ring_base + (uint32_t)(buf * TILE);
#pragma unroll
            for (int i = 0; i < (kMmaTileRows * CH) / 32; i++) {
                const int id = lane + 32 * i;
                const int row = id / CH, c = id % CH;
                const int rr = r0 + row;
                const bool ok = rr < wr1 && rr < n_cached;
                const long off = ok ? (long)rr * p.cs_s + c * 8 : 0;
                const uint32_t dst = sb + row * ROWB + ((c ^ (row & 7)) << 4);
                cp_async16(dst, kc + off, ok ? 16 : 0);
                cp_async16(dst + kMmaTileRows * ROWB, vc + off, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };
    for (int s = 0; s < nst - 1; s++) issue(s, s);

    // rotation coefficients of the pairs this THREAD rotates when it prepares q (and the new k)
    // q: thread handles elements (head = threadIdx/ (D/2) ... ) -- see below
    pdl_wait();

    // q -> bias, RoPE, fp16 into q_s[head][d]; heads >= G are zero
    for (int idx = threadIdx.x; idx < 8 * (D / 2); idx += kMmaWarps * 32) {
        const int head = idx / (D / 2), pr = idx % (D / 2);
        float x = 0.f, y = 0.f;
        if (head < G) {
            const __half* qp = reinterpret_cast<const __half*>(p.q) + b * p.q_sb + (long)(h0 + head) * D + 2 * pr;
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(qp));
            x = v.x;
            y = v.y;
            if (p.bq) {
                const float2 bb = __half22float2(
                    *reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(p.bq) + (long)(h0 + head) * D + 2 * pr));
                x += bb.x;
                y += bb.y;
            }
            if (2 * pr < p.rot_dim) {
                float sn, cs;
                sincosf(pos / p.rope_denom[pr], &sn, &cs);
                const float xr = cs * x - sn * y, yr = cs * y + sn * x;
                x = xr;
                y = yr;
            }
        }
        *reinterpret_cast<__half2*>(&q_s[head][2 * pr]) = __floats2half2_rn(x, y);
    }
    __syncthreads();
    uint32_t qa[KS][2];  // A fragments of q: (head g, d 16ks+2t..) and (head g, d 16ks+8+2t..)
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(&q_s[g][16 * ks + 2 * t]);
        qa[ks][1] = *reinterpret_cast<const uint32_t*>(&q_s[g][16 * ks + 8 + 2 * t]);
    }

    float O[2 * KS][2];  // (head g, d 8j+2t, 8j+2t+1); the accumulator halves of heads 8..15 are dropped
#pragma unroll
    for (int j = 0; j < 2 * KS; j++) O[j][0] = O[j][1] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's share of the row sum

    // ldmatrix lane addressing inside a tile (K part): matrix mi = lane/8
    const int mi = lane >> 3, lr = lane & 7;
    const int k_row = lr + (mi >> 1) * 8, k_chunk = mi & 1;   // S: (rows 0-7 | 8-15) x (chunk 2ks | 2ks+1)
    const int v_row = lr + (mi & 1) * 8, v_chunk = mi >> 1;   // PV: (rows 0-7 | 8-15) x (chunk 2jp | 2jp+1)

    int buf = 0, fill = nst - 1;
    for (int tile = 0; tile < n_tiles; tile++) {
        cp_async_wait_dyn(nst - 2);
        __syncwarp();
        const int r0 = wr0 + tile * kMmaTileRows;
        const uint32_t sb = ring_base + (uint32_t)(buf * TILE);
        // the new token's row, if it lies in this tile: bias, RoPE, round, store to the tile and the cache
        if (owns_new && n_cached >= r0 && n_cached < r0 + kMmaTileRows && n_cached < wr1) {
            const int row = n_cached - r0, d0 = lane * EPL;
            float kf[EPL], vf[EPL];
#pragma unroll
            for (int e = 0; e < EPL; e++) {
                kf[e] = __half2float(reinterpret_cast<const __half*>(p.k)[b * p.k_sb + (long)hk * D + d0 + e]);
                vf[e] = __half2float(reinterpret_cast<const __half*>(p.v)[b * p.v_sb + (long)hk * D + d0 + e]);
                if (p.bk) kf[e] += __half2float(reinterpret_cast<const __half*>(p.bk)[(long)hk * D + d0 + e]);
                if (p.bv) vf[e] += __half2float(reinterpret_cast<const __half*>(p.bv)[(long)hk * D + d0 + e]);
            }
#pragma unroll
            for (int e = 0; e < EPL; e += 2) {
                if (d0 + e < p.rot_dim) {
                    float sn, cs;
                    sincosf(pos / p.rope_denom[(d0 + e) >> 1], &sn, &cs);
                    const float x = kf[e], y = kf[e + 1];
                    kf[e] = cs * x - sn * y;
                    kf[e + 1] = cs * y + sn * x;
                }
            }
            unsigned char* krow = ring_gen + (size_t)buf * TILE + row * ROWB + ((((d0 >> 3) ^ (row & 7))) << 4) + (d0 & 7) * 2;
            unsigned char* vrow = krow + kMmaTileRows * ROWB;
            __half* kd = reinterpret_cast<__half*>(p.kc) + b * p.cs_b + hk * p.cs_h + (long)n_cached * p.cs_s + d0;
            __half* vd = reinterpret_cast<__half*>(p.vc) + b * p.cs_b + hk * p.cs_h + (long)n_cached * p.cs_s + d0;
#pragma unroll
            for (int e = 0; e < EPL; e += 2) {
                const __half2 kh = __floats2half2_rn(kf[e], kf[e + 1]), vh = __floats2half2_rn(vf[e], vf[e + 1]);
                *reinterpret_cast<__half2*>(krow + e * 2) = kh;
                *reinterpret_cast<__half2*>(vrow + e * 2) = vh;
                if (writes_cache) {
                    *reinterpret_cast<__half2*>(kd + e) = kh;
                    *reinterpret_cast<__half2*>(vd + e) = vh;
                }
            }
            __syncwarp();
        }
        issue(tile + nst - 1, fill);
        buf = buf + 1 == nst ? 0 : buf + 1;
        fill = fill + 1 == nst ? 0 : fill + 1;

        // S^T = q . K^T for the 16 rows of the tile: s0 = rows 0-7, s1 = rows 8-15
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t kb[4];
            const int c = 2 * ks + k_chunk;
            ldsm_x4(kb, sb + k_row * ROWB + ((c ^ (k_row & 7)) << 4));
            mma_f16(s0, qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
            mma_f16(s1, qa[ks][0], 0u, qa[ks][1], 0u, kb[2], kb[3]);
        }
        // scale, mask rows beyond the range, running softmax for head g (log2 domain)
        const int valid = wr1 - r0;  // rows of this tile that exist
        float sc[4];
        sc[0] = (2 * t < valid) ? s0[0] * p.scale_log2e : -INFINITY;
        sc[1] = (2 * t + 1 < valid) ? s0[1] * p.scale_log2e : -INFINITY;
        sc[2] = (8 + 2 * t < valid) ? s1[0] * p.scale_log2e : -INFINITY;
        sc[3] = (9 + 2 * t < valid) ? s1[1] * p.scale_log2e : -INFINITY;
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float ms = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = fast_exp2(m_run - ms);
        m_run = m_new;
        float pr[4];
#pragma unroll
        for (int e = 0; e < 4; e++) pr[e] = fast_exp2(sc[e] - ms);
        l_run = l_run * corr + (pr[0] + pr[1] + pr[2] + pr[3]);
        const uint32_t pa0 = pack_h2(pr[0], pr[1]), pa2 = pack_h2(pr[2], pr[3]);
#pragma unroll
        for (int j = 0; j < 2 * KS; j++) {
            O[j][0] *= corr;
            O[j][1] *= corr;
        }
        // O += P . V
#pragma unroll
        for (int jp = 0; jp < KS; jp++) {
            uint32_t vb[4];
            const int c = 2 * jp + v_chunk;
            ldsm_x4_t(vb, sb + (kMmaTileRows + v_row) * ROWB + ((c ^ (v_row & 7)) << 4));
            float o0[4] = {O[2 * jp][0], O[2 * jp][1], 0.f, 0.f}, o1[4] = {O[2 * jp + 1][0], O[2 * jp + 1][1], 0.f, 0.f};
            mma_f16(o0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
            mma_f16(o1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
            O[2 * jp][0] = o0[0];
            O[2 * jp][1] = o0[1];
            O[2 * jp + 1][0] = o1[0];
            O[2 * jp + 1][1] = o1[1];
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    __syncthreads();  // every warp is done with its ring before the ring is reused below

    // per-warp results -> shared memory, then the same merge as the SIMT kernel
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < G) {
#pragma unroll
        for (int j = 0; j < 2 * KS; j++) {
            sm_acc[warp][g][8 * j + 2 * t] = O[j][0];
            sm_acc[warp][g][8 * j + 2 * t + 1] = O[j][1];
        }
        if (t == 0) {
            sm_m[warp][g] = m_run;
            sm_l[warp][g] = l_run;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += kMmaWarps * 32) {
        const int gg = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < kMmaWarps; i++) M = fmaxf(M, sm_m[i][gg]);
        float L = 0.f, Ov = 0.f;
#pragma unroll
        for (int i = 0; i < kMmaWarps; i++) {
            const float w = fast_exp2(sm_m[i][gg] - M);  // warps without rows: exp2(-inf) = 0
            L = fmaf(sm_l[i][gg], w, L);
            Ov = fmaf(sm_acc[i][gg][d], w, Ov);
        }
        const int h = h0 + gg;
        if (n_split == 1) {
            reinterpret_cast<__half*>(p.out)[b * p.out_sb + (long)h * D + d] = __float2half_rn(Ov / L);
        } else {
            const long base = ((long)b * p.H + h) * p.n_split + split;
            p.part_acc[base * D + d] = Ov;
            if (d == 0) {
                p.part_ml[base * 2] = M;
                p.part_ml[base * 2 + 1] = L;
            }
        }
    }
    if (n_split > 1 && p.tickets) merge_by_last_block<__half>(p, b, h0, G, n_split);
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

// Plan for the tensor-core kernel: blocks per SM r in {3, 2, 1} fix the ring depth shared memory allows (2, 3, 6
// stages per warp at D = 128).  For every split count the launch's time is estimated from what was measured
// to bound it on B200:
//   - a warp takes its tiles one after the other, so with `depth` tiles in flight it moves at most
//     depth * tile / latency (latency under load about 2.3 us): shallow rings need many resident warps;
//   - a warp needs about 0.9 us of issue time per 16-row tile (D = 128), and an SM gains little beyond 8 warps:
//     one block per SM cannot reach the HBM rate however deep its ring is;
//   - the blocks should fill the waves they need, each wave has a fixed cost (q, RoPE, the warps' merge), and a
//     split launch pays for the merge kernel behind it.
// Many (sequence, head) pairs on few slots, e.g. 320 pairs per GPU of an 8-way split 13B model at batch 64, are
// split so that the last wave is full instead of running one shallow ring per pair.
static int g_plan_force_r = 0, g_plan_force_n = 0;  // onellm_decode_attn_plan_override (tuning aid)

static AttnPlan plan_attention_mma(int B, int n_head_blocks, int step, int D, int regs_per_sm)
{
    const int n_cached = step > 1 ? step - 1 : 0;
    const long base = (long)B * n_head_blocks;
    const int ms = max_splits(step);
    const int sms = num_sms();
    const size_t tile = (size_t)2 * kMmaTileRows * D * 2;
    const int rows_all = (n_cached + 63) / 64 * 64 < kMinChunkRows ? kMinChunkRows : (n_cached + 63) / 64 * 64;
    // fallback (never taken while any ring fits): one split over all rows, two stages
    AttnPlan best = {1, rows_all, 2, 2 * kMmaWarps * tile};
    double best_t = 1.0e300;
    const double bytes = 2.0 * (double)n_cached * (double)base * D * 2.0;
    // the merge kernel costs a launch boundary in a step, not only its run time (merging inside the attention kernel,
    // onellm_decode_attn_merged, measured no cheaper: every block then ends with a fence and a ticket)
    constexpr double kPeak = 6.5e12, kLatency = 2.3e-6, kWaveCost = 1.0e-6, kMergeCost = 6.0e-6;
    const double t_tile = 0.9e-6 * (double)D / 128.0;
    // Two blocks per SM (three stages per warp at D = 128) won or tied every sweep over (blocks per SM, splits) on B200,
    // from 32 to 2560 (sequence, head) pairs and 520 to 2040 rows: three blocks leave one tile in flight per warp, one
    // block has too few warps to issue.  The other values are only tried on request or when two blocks do not fit.
    const int r_default = regs_per_sm >= 2 ? 2 : 1;
    for (int r = regs_per_sm < 3 ? regs_per_sm : 3; r >= 1; r--) {
        if (r != (g_plan_force_r > 0 ? g_plan_force_r : r_default)) continue;
        const size_t budget = (size_t)(227 * 1024) / r - 4096;
        int nst = (int)(budget / (kMmaWarps * tile));
        if (nst > 8) nst = 8;
        if (nst < 2) continue;
        const long slots = (long)r * sms;
        int last_ns = 0;
        for (int n = 1; n <= ms && n <= 16; n++) {
            if (g_plan_force_n > 0 && n != g_plan_force_n) continue;
            int c = (n_cached + n - 1) / n;
            c = (c + 63) / 64 * 64;  // whole tiles for each of the four warps
            if (c < kMinChunkRows) c = kMinChunkRows;
            int ns = (n_cached + c - 1) / c;
            if (ns < 1) ns = 1;
            if (ns == last_ns) continue;  // the same launch as the split count before
            last_ns = ns;
            const long total = base * ns;
            const long waves = (total + slots - 1) / slots;
            const long resident = total < slots ? total : slots;
            const double fill = total <= slots ? 1.0 : (double)total / (double)(waves * slots);
            const int tiles_per_warp = (c / kMmaWarps + kMmaTileRows - 1) / kMmaTileRows;
            const int depth = nst - 1 < tiles_per_warp ? nst - 1 : tiles_per_warp;
            const double by_latency = (double)resident * kMmaWarps * depth * (double)tile / kLatency;
            const long sms_used = (resident + r - 1) / r < sms ? (resident + r - 1) / r : sms;
            const int warps_sm = r * kMmaWarps < 8 ? r * kMmaWarps : 8;
            const double by_issue = (double)sms_used * warps_sm * (double)tile / t_tile;
            double rate = kPeak * fill;
            if (by_latency < rate) rate = by_latency;
            if (by_issue < rate) rate = by_issue;
            const double t = bytes / rate + kWaveCost * (double)waves + (ns > 1 ? kMergeCost : 0.0);
            if (t < best_t) {
                best_t = t;
                best = {ns, c, nst, (size_t)nst * kMmaWarps * tile};
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
    static std::map<std::pair<AttnKernel, int>, AttnKernelInfo> cache;  // per (kernel, device): the attribute is set per device
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair(k, current_device());
    auto it = cache.find(key);
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
        (void)prefer_max_shared((const void*)k);  // same L1 / shared-memory split as the projections around it
    }
    (void)cudaGetLastError();
    cache[key] = info;
    return info;
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_decode_attn_plan_override(int blocks_per_sm, int splits)
{
    ONELLM_REQUIRE(blocks_per_sm >= 0 && blocks_per_sm <= 3 && splits >= 0 && splits <= 16, ONELLM_ERR_ARG,
                   "decode_attn_plan_override: blocks per SM in 0..3, splits in 0..16 (0 = the planner decides)");
    g_plan_force_r = blocks_per_sm;
    g_plan_force_n = splits;
    return ONELLM_OK;
}

extern "C" size_t onellm_decode_attn_workspace_bytes(int B, int H, int D, int max_step)
{
    if (B <= 0 || H <= 0 || D <= 0 || max_step <= 0) return 0;
    const size_t worst = (size_t)B * H * max_splits(max_step) * (D + 2) * sizeof(float);
    return worst + 256;
}

static int decode_attn_impl(int dtype, const void* q, const void* k, const void* v, long q_stride_b, long k_stride_b,
                            long v_stride_b, const void* bias_q, const void* bias_k, const void* bias_v, void* k_cache,
                            void* v_cache, long cs_b, long cs_h, long cs_s, int B, int H, int Hkv, int D, int step,
                            const int* step_dev, const int* step_offset, int rope_pos, int rot_dim, float rope_base,
                            float scale, void* out, long out_stride_b, void* workspace, size_t workspace_bytes,
                            int* tickets, void* stream)
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
    p.step_offset = step_offset;
    p.rope_delta = rope_pos - step;
    p.rot_dim = rot_dim < D ? rot_dim : D;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.out = out;
    p.out_sb = out_stride_b;
    for (int i = 0; i < kMaxRopePairs; i++)
        p.rope_denom[i] = (2 * i < p.rot_dim) ? powf(rope_base, (float)(2 * i) / (float)rot_dim) : 1.f;

    const int G = pick_group(H / Hkv);
    const int lpr = (int)(row_bytes / 16);
    const bool use_mma = dtype == ONELLM_F16 && (D == 64 || D == 128);
    AttnKernel kern;
    AttnPlan plan;
    if (use_mma) {
        kern = D == 128 ? (G == 8 ? decode_attn_mma_kernel<128, 8> : G == 4 ? decode_attn_mma_kernel<128, 4>
                                   : G == 2 ? decode_attn_mma_kernel<128, 2> : decode_attn_mma_kernel<128, 1>)
                        : (G == 8 ? decode_attn_mma_kernel<64, 8> : G == 4 ? decode_attn_mma_kernel<64, 4>
                                   : G == 2 ? decode_attn_mma_kernel<64, 2> : decode_attn_mma_kernel<64, 1>);
        const AttnKernelInfo info = kernel_info(kern);  // also raises the dynamic shared-memory limit once
        plan = plan_attention_mma(B, H / G, step, D, info.blocks_per_sm_regs);
    } else {
        kern = dtype == ONELLM_F16 ? attn_kernel_for<__half>(lpr, G) : attn_kernel_for<float>(lpr, G);
        const AttnKernelInfo info = kernel_info(kern);
        plan = plan_attention(B, H / G, step, info.blocks_per_sm_regs, info.static_smem, row_bytes);
    }
    p.n_split = plan.n_split;
    p.chunk = plan.chunk;
    p.nst = plan.nst;
    // the kernels derive their split count from `chunk`: it must cover every cached row within the
    // launched grid, or a block would take itself for a partial and write to a missing workspace
    ONELLM_REQUIRE((long)plan.chunk * plan.n_split >= step - 1 && plan.nst >= 2, ONELLM_ERR_UNSUPPORTED,
                   "decode_attn: internal plan does not cover the rows (chunk=%d splits=%d step=%d)", plan.chunk,
                   plan.n_split, step);
    p.part_acc = nullptr;
    p.part_ml = nullptr;
    p.tickets = tickets;
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
    if (p.n_split > 1 && !tickets) {
        if (dtype == ONELLM_F16)
            ONELLM_CUDA(launch_pdl(decode_attn_combine_kernel<__half>, dim3(H, B), dim3(128), 0, st, p));
        else
            ONELLM_CUDA(launch_pdl(decode_attn_combine_kernel<float>, dim3(H, B), dim3(128), 0, st, p));
    }
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

extern "C" int onellm_decode_attn(int dtype, const void* q, const void* k, const void* v, long q_stride_b,
                                  long k_stride_b, long v_stride_b, const void* bias_q,
                                  const void* bias_k, const void* bias_v, void* k_cache, void* v_cache,
                                  long cs_b, long cs_h, long cs_s, int B, int H, int Hkv, int D, int step,
                                  const int* step_dev, int rope_pos, int rot_dim, float rope_base,
                                  float scale, void* out, long out_stride_b, void* workspace,
                                  size_t workspace_bytes, void* stream)
{
    return decode_attn_impl(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache, cs_b,
                            cs_h, cs_s, B, H, Hkv, D, step, step_dev, nullptr, rope_pos, rot_dim, rope_base, scale, out,
                            out_stride_b, workspace, workspace_bytes, nullptr, stream);
}

// Sequences of different lengths in one batch: sequence b attends step + step_offset[b] rows (the new one included),
// its new row goes to cache row step + step_offset[b] - 1 and its position moves with it.
extern "C" int onellm_decode_attn_ragged(int dtype, const void* q, const void* k, const void* v, long q_stride_b,
                                         long k_stride_b, long v_stride_b, const void* bias_q, const void* bias_k,
                                         const void* bias_v, void* k_cache, void* v_cache, long cs_b, long cs_h,
                                         long cs_s, int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         const int* step_offset, int rope_pos, int rot_dim, float rope_base,
                                         float scale, void* out, long out_stride_b, void* workspace,
                                         size_t workspace_bytes, void* stream)
{
    return decode_attn_impl(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache, cs_b,
                            cs_h, cs_s, B, H, Hkv, D, step, step_dev, step_offset, rope_pos, rot_dim, rope_base, scale, out,
                            out_stride_b, workspace, workspace_bytes, nullptr, stream);
}

// The same call with the splits merged inside the attention kernel (one launch whatever the plan): `tickets` is
// B * H ints of device memory that are zero before the first call; every call leaves them zero.  Calls that share a
// ticket array must not overlap on the GPU.  Same plan and same bits as the two-launch form.  On B200 it measured
// SLOWER than the two-launch form wherever a plan splits (inside a decoder layer 1.5-4 us at the 7B shape over 2-8
// GPUs, 7-11 us at the 13B shape, batch 64: every block of a split launch ends with a fence, a barrier and an
// atomic, which costs more over several waves of blocks than one small merge launch), so the model class keeps the
// two-launch form; the entry point stays for hosts where a launch is dearer than that.
extern "C" int onellm_decode_attn_merged(int dtype, const void* q, const void* k, const void* v, long q_stride_b,
                                         long k_stride_b, long v_stride_b, const void* bias_q, const void* bias_k,
                                         const void* bias_v, void* k_cache, void* v_cache, long cs_b, long cs_h,
                                         long cs_s, int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         const int* step_offset, int rope_pos, int rot_dim, float rope_base,
                                         float scale, void* out, long out_stride_b, void* workspace,
                                         size_t workspace_bytes, int* tickets, void* stream)
{
    ONELLM_REQUIRE(tickets, ONELLM_ERR_ARG, "decode_attn_merged: null ticket array");
    return decode_attn_impl(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache, cs_b,
                            cs_h, cs_s, B, H, Hkv, D, step, step_dev, step_offset, rope_pos, rot_dim, rope_base, scale, out,
                            out_stride_b, workspace, workspace_bytes, tickets, stream);
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
