// Shared by the two weight-streaming projection kernels (skinny_gemm_staged.cu: mma.sync, at most 16 tokens per
// 8-token block row; skinny_gemm_tc.cu: tcgen05, up to 64 tokens): the epilogue options and the split-K reduction
// over a thread-block cluster with everything that follows it (RMS scale, SwiGLU, tensor-parallel exchange,
// residual and bias).
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace onellm {

constexpr int kBN = 128;          // output columns per block
constexpr int kRedLd = kBN + 1;   // row stride of the partial tile in shared memory (floats)

// Options of the plain (not FUSED) kernel that let a decoder layer run without norm kernels:
//   rms:   the result is scaled per token by rsqrt(mean_over_K(x^2) + rms_eps), i.e. the projection of
//          RMSNorm(x) when the norm's gamma has been multiplied into the rows of W beforehand.  The sum
//          of squares is taken from the activations as they pass through the ring (no extra reads).
//   resid: y = resid + bias + result (bias may be NULL); resid may be y itself (each element is read
//          and written by the same thread).
struct EpilogueArgs {
    const __half* resid;  // [M, N] or NULL
    const __half* bias;   // [N] or NULL
    float rms_eps;
    int rms;
    int early_dependents;  // release the next kernel before the main loop (it then shares the SM with this one)
    TpEpilogue tp;         // tensor parallel: y = resid + bias + sum over ranks of this projection (see common.cuh)
};

// `red` holds this block's partial tile as [NW][MP][kRedLd] floats followed by MP partial sums of squares (used
// when ep.rms is set); the blocks of the cluster (rank = blockIdx.y of gridDim.y) hold the other K ranges of the
// same tile.  Sums them in rank order and finishes the tile; every thread of the block (NT of them) calls it.
// WIDE (tcgen05 kernel, no tensor-parallel exchange): the second half of `red` is not a second weight but the next
// 128 output columns of the same weight (a block owns 256 columns and reads its activations once for both).
template <int MP, bool DUAL, bool FUSED, int NT, bool WIDE = false>
__device__ __forceinline__ void splitk_epilogue(float* red, cg::cluster_group& cluster, __half* y, int M, int N, int K, int n0,
                                                const EpilogueArgs& ep)
{
    static_assert(!(DUAL && WIDE), "two weights or two column tiles, not both");
    constexpr int NW = (DUAL || WIDE) ? 2 : 1;
    const int KS = gridDim.y, rank = blockIdx.y, tid = threadIdx.x;
    // tensor parallel: this block's sequence number for the call (blocks pair up by index across the ranks)
    __shared__ uint32_t s_seq;
    const bool tp = !FUSED && !WIDE && ep.tp.world > 1;
    if (tp && tid == 0) {
        int* ctr = ep.tp.counters + blockIdx.y * gridDim.x + blockIdx.x;
        const int n = *ctr + 1;
        *ctr = n;
        s_seq = 0x80000000u | (uint32_t)n;  // the high bit keeps these apart from the numbers of the stand-alone all-reduce
    }
    cluster.sync();
    const uint32_t seq = tp ? s_seq : 0u;
    // every rank of the cluster finishes an even-sized slice of the tile, two adjacent columns per thread
    const int per_rank = (((MP * kBN + KS - 1) / KS) + 1) & ~1;
    const int e_begin = rank * per_rank, e_end = min(e_begin + per_rank, MP * kBN);
    const long long t_start = clock64();
    // The value this block contributes to elements (tok, c) and (tok, c + 1): the K ranges of the cluster added in rank
    // order, the RMS scale, SwiGLU.  False when the pair lies outside the matrix.
    auto partial = [&](int e, float& v0, float& v1, float& w0, float& w1) {
        const int tok = e / kBN, c = e % kBN;
        // all remote loads are issued before the first is used (a cluster has at most 8 ranks): summing as
        // they are requested would pay one distributed-shared-memory round trip per rank
        float2 p0[8], p1[8];
        float ps[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            p0[r] = p1[r] = make_float2(0.f, 0.f);
            ps[r] = 0.f;
            if (r < KS) {
                const float* peer = cluster.map_shared_rank(red, r);
                p0[r] = make_float2(peer[tok * kRedLd + c], peer[tok * kRedLd + c + 1]);
                if (NW == 2) p1[r] = make_float2(peer[(MP + tok) * kRedLd + c], peer[(MP + tok) * kRedLd + c + 1]);
                if (!FUSED && ep.rms) ps[r] = peer[NW * MP * kRedLd + tok];
            }
        }
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < 8; r++) {  // rank order: the sum does not depend on which block does it
            s0.x += p0[r].x;
            s0.y += p0[r].y;
            s1.x += p1[r].x;
            s1.y += p1[r].y;
            ss += ps[r];
        }
        if (!(tok < M && n0 + c < N)) return false;  // N is even: the second column is inside too
        if (!FUSED && ep.rms) {
            const float inv = rsqrtf(ss / (float)K + ep.rms_eps);
            s0.x *= inv;
            s0.y *= inv;
            s1.x *= inv;
            s1.y *= inv;
        }
        v0 = DUAL ? (s0.x / (1.0f + __expf(-s0.x))) * s1.x : s0.x;
        v1 = DUAL ? (s0.y / (1.0f + __expf(-s0.y))) * s1.y : s0.y;
        w0 = s1.x;  // WIDE: the same pair 128 columns further
        w1 = s1.y;
        return true;
    };
    // one bounded poll of a tagged word: returns the data word once it carries this call's sequence number
    auto await = [&](const uint2* src) {
        uint32_t w, got;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(w), "=r"(got) : "l"(src) : "memory");
            if (got == seq) break;
            if (clock64() - t_start > 2000LL * 1000 * 1000) {  // about a second: give up, say so, go on
                atomicExch(ep.tp.error, 1);
                break;
            }
        }
        return w;
    };
    auto send = [&](uint2* dst, uint32_t w) {
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(dst), "r"(w), "r"(seq) : "memory");
    };
    // this rank's fp16 partial `word` of a pair -> the partials of all ranks added in rank order
    auto gather = [&](size_t idx, uint32_t word, float& v0, float& v1) {
        v0 = v1 = 0.f;
#pragma unroll
        for (int r = 0; r < 8; r++)
            if (r < ep.tp.world) {
                const uint32_t w = r == ep.tp.rank ? word : await(ep.tp.mine + (size_t)r * ep.tp.slot_words + idx / 2);
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
                v0 += f.x;
                v1 += f.y;
            }
    };
    // residual and bias, then the store; returns what was stored
    auto finish = [&](size_t idx, int c, float v0, float v1) {
        if (!FUSED && ep.resid) {
            const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(ep.resid + idx));
            v0 += rr.x;
            v1 += rr.y;
            if (ep.bias) {
                const float2 bb = __half22float2(*reinterpret_cast<const __half2*>(ep.bias + n0 + c));
                v0 += bb.x;
                v1 += bb.y;
            }
        }
        const __half2 out = __floats2half2_rn(v0, v1);
        *reinterpret_cast<__half2*>(y + idx) = out;
        return *reinterpret_cast<const uint32_t*>(&out);
    };

    if (tp && ep.tp.two_shot) {
        // Three passes, so that the two hops of all of a thread's pairs overlap: (1) every partial of a row that
        // belongs to another rank goes to that rank; (2) the rows of this rank: gather, finish, store, and the
        // finished value to everybody; (3) the other rows: store what their owners sent.
        constexpr int kPairs = (MP * kBN / 2 + NT - 1) / NT;  // pairs a thread handles at most (K split of one)
        uint32_t mine[kPairs];
        unsigned valid = 0u;  // kPairs <= 32
        static_assert(kPairs <= 32, "pair bookkeeping is one bit per pair");
        int it = 0;
        for (int e = e_begin + 2 * tid; e < e_end; e += 2 * NT, it++) {
            float v0, v1, w0, w1;
            if (!partial(e, v0, v1, w0, w1)) continue;
            const int tok = e / kBN, c = e % kBN;
            const __half2 own = __floats2half2_rn(v0, v1);
            mine[it] = *reinterpret_cast<const uint32_t*>(&own);
            valid |= 1u << it;
            const int owner = tok % ep.tp.world;
            if (owner != ep.tp.rank) send(ep.tp.push[owner] + ((size_t)tok * N + n0 + c) / 2, mine[it]);
        }
        it = 0;
        for (int e = e_begin + 2 * tid; e < e_end; e += 2 * NT, it++) {
            const int tok = e / kBN, c = e % kBN;
            if (!((valid >> it) & 1u) || tok % ep.tp.world != ep.tp.rank) continue;
            const size_t idx = (size_t)tok * N + n0 + c;
            float v0, v1;
            gather(idx, mine[it], v0, v1);
            const uint32_t w = finish(idx, c, v0, v1);
#pragma unroll
            for (int r = 0; r < 8; r++)
                if (r < ep.tp.world && r != ep.tp.rank) send(ep.tp.final_push[r] + idx / 2, w);
        }
        it = 0;
        for (int e = e_begin + 2 * tid; e < e_end; e += 2 * NT, it++) {
            const int tok = e / kBN, c = e % kBN;
            if (!((valid >> it) & 1u) || tok % ep.tp.world == ep.tp.rank) continue;
            const size_t idx = (size_t)tok * N + n0 + c;
            *reinterpret_cast<uint32_t*>(y + idx) = await(ep.tp.final_mine + idx / 2);
        }
        return;
    }
    for (int e = e_begin + 2 * tid; e < e_end; e += 2 * NT) {
        float v0, v1, w0, w1;
        if (!partial(e, v0, v1, w0, w1)) continue;
        const int tok = e / kBN, c = e % kBN;
        const size_t idx = (size_t)tok * N + n0 + c;
        if (WIDE && n0 + kBN + c < N) (void)finish(idx + kBN, c + kBN, w0, w1);
        if (tp) {
            // one-shot: this rank's value of the two elements to every peer, then theirs
            const __half2 own = __floats2half2_rn(v0, v1);
            const uint32_t word = *reinterpret_cast<const uint32_t*>(&own);
#pragma unroll
            for (int r = 0; r < 8; r++)
                if (r < ep.tp.world && r != ep.tp.rank) send(ep.tp.push[r] + idx / 2, word);
            gather(idx, word, v0, v1);
        }
        (void)finish(idx, c, v0, v1);
    }
}

}  // namespace onellm
