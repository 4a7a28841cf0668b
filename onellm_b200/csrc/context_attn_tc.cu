// Context-phase causal attention on the 5th-generation tensor cores (fp16, head size 128, cache in its
// standard [B, Hkv, S, D] order).  Same arithmetic and interface as context_attn_kernel in prefill.cu (which
// stays for other head sizes and cache orders); replaces launchLinearStridedBatchGemm x2 +
// launchScaleMaskAndSoftmax + launchTransposeOutRemovePadding of
// src/layers/attention/context_attention.cpp:137-151 without the score matrix.
//
// A block owns 128 query rows of one (sequence, head) and walks the cache in tiles of 64 rows:
//   S = Q . K_tile^T      tcgen05.mma M128 N64 K16 x 8, Q and K_tile in shared memory (128-byte swizzle, both
//                         K-major; K by TMA), S in tensor memory (64 columns of fp32, two accumulators so that
//                         the next tile's product runs under this tile's softmax)
//   P = exp2(S - ref)     four warps, one query row per thread: the row is read from tensor memory once and kept
//                         in registers; P goes back as fp16 (two per 32-bit column) over the first 32 columns of
//                         the accumulator its scores came from (tcgen05.st)
//   O += P . V_tile       tcgen05.mma again with the A operand read from tensor memory (no shared-memory copy of P,
//                         no proxy fence); V_tile (rows of the cache, head dimension contiguous) is the MN-major B
//                         operand, exactly as the [K,N] weights of the projections.  O stays in tensor memory (128
//                         columns) over all tiles.  `ref` is the row maximum the exponentials are taken against; it
//                         follows the true running maximum only when that has grown by more than 8 (P stays below
//                         2^8), and only then does a thread wait for the previous product and rescale O in place.
// The MMAs of one thread run in issue order, which is what lets S of tile j + 2 overwrite the accumulator P of tile j
// was read from without a wait in between.
// A fifth warp issues the TMA loads (K and V tiles double-buffered) and the MMAs.  96 KB of shared memory and 256
// columns of tensor memory per block: two blocks share an SM, so one block's start-up and drain hide under the
// other's steady state.  Every mbarrier wait is bounded; on expiry the block raises the time-out flag, stops, frees
// its tensor memory and returns.
#include <math.h>

#include "tc_common.cuh"

namespace onellm {

constexpr int kAtQ = 128, kAtKV = 64, kAtD = 128;
constexpr int kAtSoftmaxThreads = 128;              // one query row per thread
constexpr int kAtThreads = kAtSoftmaxThreads + 32;  // + one control warp (TMA and MMA issue)
constexpr int kAtQTile = kAtQ * kAtD * 2;           // 32 KB: two 64-column chunks of [128 rows x 128 bytes]
constexpr int kAtQChunk = kAtQTile / 2;
constexpr int kAtKVTile = kAtKV * kAtD * 2;         // 16 KB: two 64-column chunks of [64 rows x 128 bytes]
constexpr int kAtKVChunk = kAtKVTile / 2;
// Q, two K and two V buffers, barriers: 96.25 KB, two blocks per SM; the dynamic array is declared 1024-byte aligned
// instead of carrying slack for it
constexpr int kAtSmemBytes = kAtQTile + 4 * kAtKVTile + 256;
constexpr uint32_t kAtTmemCols = 256;  // S0 at column 0, S1 at 64, O at 128

// D[tmem] (+)= A[tmem] . B[smem]: the A operand (M rows = lanes, K elements packed two fp16 per 32-bit column) comes
// from tensor memory
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(kAtThreads, 2)
context_attn_tc_kernel(const __half* __restrict__ q, long q_ld, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ history, int H, int Hkv, int S_max, float scale_log2e, __half* __restrict__ out)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];  // the 128-byte swizzle works on shared-window address bits
    unsigned char* sQ = smem_raw;
    unsigned char* sK = sQ + kAtQTile;       // two buffers
    unsigned char* sV = sK + 2 * kAtKVTile;  // two buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kAtKVTile);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    // Every per-tile barrier comes as a pair: tile j uses slot j & 1 and waits for phase (j >> 1) & 1 of it.  A
    // parity wait only tells "this phase" from "the next one", so a single barrier would be wrong as soon as its
    // producer can get two phases ahead of a waiter: the softmax warps may finish tile j + 1 (its scores were issued
    // before the control warp waits for P of tile j) before a delayed control warp has looked at P of tile j, and
    // the last P.V product may still be in flight behind the one before it when the softmax warps look for it.
    // With two slots a slot's next phase (tile j + 2) can only start after its waiter has seen tile j.
    const uint32_t q_full = smem_u32(bars), k_full0 = smem_u32(bars + 1), s_full0 = smem_u32(bars + 3), v_full0 = smem_u32(bars + 5),
                   p_full0 = smem_u32(bars + 7), o_full0 = smem_u32(bars + 9);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (H / Hkv);

    if (smem_u32(smem_raw) & 1023u) {  // never seen; the tiles would be read with the wrong swizzle
        if (threadIdx.x == 0) atomicExch(&g_tc_timeout_flag, 1);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, kAtSoftmaxThreads);
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1);
            mbar_init(p_full0 + 8 * s, kAtSoftmaxThreads);
            mbar_init(o_full0 + 8 * s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kAtTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    pdl_wait();  // q and the cache rows come from the kernel before this one
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0, hist = history[b];
    // the blocks with the most cache tiles first: the last query rows of a sequence
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kAtQ;
    const bool active = q0 < q_len;  // uniform over the block
    const int q_rows = active ? min(kAtQ, q_len - q0) : 0;
    const int kv_end = hist + q0 + q_rows;  // rows any query of this block may attend
    const int n_tiles = active ? (kv_end + kAtKV - 1) / kAtKV : 0;
    const int cache_row0 = (b * Hkv + hk) * S_max;

    if (warp == 4 && active) {
        // ---- control: TMA loads and MMA issue.  The whole warp runs this code and one elected lane issues the
        // single-thread instructions: with warp-uniform control flow the descriptors and addresses stay in uniform
        // registers, which is where tcgen05.mma takes them from (under a divergent `lane == 0` branch every operand
        // of every MMA was moved there one by one, ~100 cycles per instruction).
        uint32_t leader;
        asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(leader));
        bool ok = true;
        auto load_k = [&](int j) {
            const int s = j & 1;
            if (leader) {
                mbar_expect_tx(k_full0 + 8 * s, kAtKVTile);
#pragma unroll
                for (int c = 0; c < 2; c++)
                    tma_load_2d(smem_u32(sK + s * kAtKVTile + c * kAtKVChunk), &map_k, 64 * c, cache_row0 + j * kAtKV, k_full0 + 8 * s);
            }
        };
        auto load_v = [&](int j) {
            const int s = j & 1;
            if (leader) {
                mbar_expect_tx(v_full0 + 8 * s, kAtKVTile);
#pragma unroll
                for (int c = 0; c < 2; c++)
                    tma_load_2d(smem_u32(sV + s * kAtKVTile + c * kAtKVChunk), &map_v, 64 * c, cache_row0 + j * kAtKV, v_full0 + 8 * s);
            }
        };
        auto wait_all = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); };
        // instruction descriptors: D = f32, A = B = f16, M = 128; S: N = 64, B K-major; O: N = 128, B MN-major
        const uint32_t idesc_s = (1u << 4) | (0u << 16) | ((uint32_t)(kAtKV >> 3) << 17) | ((uint32_t)(kAtQ >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(kAtD >> 3) << 17) | ((uint32_t)(kAtQ >> 4) << 24);
        // Shared-memory descriptors are built once; a step inside a tile only adds (bytes >> 4) to the address field in
        // the low word (the field holds any shared-memory address, so the add never carries out of it).
        const uint64_t dq = umma_desc(smem_u32(sQ), 16, 1024), dk = umma_desc(smem_u32(sK), 16, 1024),
                       dv = umma_desc(smem_u32(sV), kAtKVChunk, 1024);
        auto issue_s = [&](int j) {  // S_j = Q . K_j^T into accumulator j & 1
            const int s = j & 1;
            if (!wait_all(k_full0 + 8 * s, (uint32_t)(j >> 1) & 1u)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t dks = dk + (uint64_t)(s * (kAtKVTile >> 4));
            const uint32_t acc = tmem_base + (uint32_t)(s * kAtKV);
            if (leader) {
#pragma unroll
                for (int kk = 0; kk < kAtD / 16; kk++) {
                    // both K-major: 64-column chunk kk/4, 32 bytes per 16 k inside the 128-byte row, 8-row groups 1024 bytes apart
                    umma_f16(acc, dq + (uint64_t)(((kk >> 2) * kAtQChunk + (kk & 3) * 32) >> 4),
                             dks + (uint64_t)(((kk >> 2) * kAtKVChunk + (kk & 3) * 32) >> 4), idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(s_full0 + 8 * s);
            }
            __syncwarp();
            return true;
        };
        load_k(0);
        load_v(0);
        if (n_tiles > 1) {
            load_k(1);
            load_v(1);
        }
        ok = wait_all(q_full, 0) && issue_s(0);
        for (int j = 0; j < n_tiles && ok; j++) {
            const int s = j & 1;
            // the next tile's scores while the softmax warps work on this one (its accumulator was last read for
            // tile j - 1, whose P has been waited for in the previous round)
            if (j + 1 < n_tiles) ok = issue_s(j + 1);
            // K buffer s is free once S_j is complete
            ok = ok && wait_all(s_full0 + 8 * s, (uint32_t)(j >> 1) & 1u);
            if (ok && j + 2 < n_tiles) load_k(j + 2);
            ok = ok && wait_all(p_full0 + 8 * s, (uint32_t)(j >> 1) & 1u) && wait_all(v_full0 + 8 * s, (uint32_t)(j >> 1) & 1u);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t dvs = dv + (uint64_t)(s * (kAtKVTile >> 4));
            if (leader) {
#pragma unroll
                for (int kk = 0; kk < kAtKV / 16; kk++) {
                    // O += P . V_tile.  A = P, K-major over the 64 cache rows of the tile (one 128-byte row per query); B =
                    // V_tile, MN-major: 64-column chunks 8 KB apart (LBO), 8-row groups 1024 bytes apart (SBO), 16 rows =
                    // 2048 bytes further
                    umma_f16_ta(tmem_base + 128u, tmem_base + (uint32_t)(s * kAtKV + kk * 8), dvs + (uint64_t)((kk * 2048) >> 4), idesc_o,
                             (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(o_full0 + 8 * s);
            }
            __syncwarp();
            if (j + 2 < n_tiles) {
                ok = wait_all(o_full0 + 8 * s, (uint32_t)(j >> 1) & 1u);  // V buffer s is free again
                if (ok) load_v(j + 2);
            }
        }
    } else if (warp < 4 && active) {
        // ---- softmax and output, one query row per thread
        const int r = threadIdx.x;                  // tensor-memory lane = query row (warp w reaches lanes 32 w ..)
        const int pos = hist + q0 + r;              // last cache row this query attends
        const bool row_ok = r < q_rows;
        const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t t_o = t_lane + 128u;
        const uint32_t row_off = (r >> 3) * 1024 + (r & 7) * 128;  // this row inside a swizzled [rows x 128-byte] chunk
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        {
            // the query row into the Q tile, in the swizzled K-major form a TMA load would give it (rows behind the
            // end of the sequence are zero): the packed q buffer has no row count the host could put into a tensor map
            // without reading cu_seqlens back
            const __half* qrow = q + (size_t)(tok0 + q0 + r) * q_ld + (size_t)h * kAtD;
#pragma unroll
            for (int u = 0; u < 16; u++) {
                const uint4 v = row_ok ? *reinterpret_cast<const uint4*>(qrow + u * 8) : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(sQ + (u >> 3) * kAtQChunk + row_off + (((u & 7) ^ (r & 7)) << 4)) = v;
            }
            fence_async_smem();
            mbar_arrive(q_full);
        }
        for (int j = 0; j < n_tiles && ok; j++) {
            ok = mbar_wait(s_full0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int kv0 = j * kAtKV;
            const bool need_mask = kv0 + kAtKV - 1 > hist + q0;  // some query of the block cannot see the whole tile
            uint32_t sv[64];
            tmem_ld32(t_lane + (uint32_t)((j & 1) * kAtKV), *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
            tmem_ld32(t_lane + (uint32_t)((j & 1) * kAtKV + 32), *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // Row maximum of the raw scores (the scale is positive, so it commutes with the maximum) on four
            // independent chains; the scale itself is folded into the exponent's multiply-add below.
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    if (kv0 + i > pos) sv[i] = 0xff800000u;  // -inf
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2e;
            const bool grow = mx > m_ref + 8.f;  // always on the first tile: every row sees cache row 0
            float alpha = 1.f;
            if (grow) {
                alpha = fast_exp2(m_ref - mx);  // exp2(-inf) = 0 on the first tile
                m_ref = mx;
                l_run *= alpha;
            }
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const float neg_ref = -m_ref;
#pragma unroll
            for (int i = 0; i < 64; i++) {
                const float pv = fast_exp2(fmaf(__uint_as_float(sv[i]), scale_log2e, neg_ref));  // exp2(-inf) = 0 for masked columns
                sum4[i & 3] += pv;
                sv[i] = __float_as_uint(pv);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l_run += sum;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                ok = mbar_wait(o_full0 + 8 * ((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u);  // P.V of the tile before: O is at rest
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t ov[32];
#pragma unroll 1
                    for (int c = 0; c < kAtD; c += 32) {
                        tmem_ld32(t_o + (uint32_t)c, ov);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                        tmem_st32(t_o + (uint32_t)c, ov);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            // P (fp16, two values per 32-bit column) over the first 32 columns of the score accumulator it came from:
            // the A operand of the P.V product, read from tensor memory
            {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; i++) pk[i] = pack_h2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]));
                tmem_st32(t_lane + (uint32_t)((j & 1) * kAtKV), pk);
            }
            if (kv0 + kAtKV > kv_end) {
                // The tile reaches beyond the rows that exist: what the cache holds there is arbitrary (possibly NaN
                // bit patterns), and 0 x NaN would poison the product.  Thread r < 64 clears cache row r of the V tile.
                ok = mbar_wait(v_full0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (r < kAtKV && kv0 + r >= kv_end) {
#pragma unroll
                    for (int u = 0; u < 16; u++)
                        *reinterpret_cast<uint4*>(sV + (j & 1) * kAtKVTile + (u >> 3) * kAtKVChunk + row_off + (u & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_smem();  // V rows were written through the generic proxy; the MMA reads through the async proxy
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(p_full0 + 8 * (j & 1));
        }
        // the last product; the commit of a product covers every MMA issued before it, the earlier products included
        ok = ok && mbar_wait(o_full0 + 8 * ((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __half* dst = out + (size_t)(tok0 + q0 + r) * H * kAtD + (size_t)h * kAtD;
#pragma unroll 1
            for (int c0 = 0; c0 < kAtD; c0 += 64) {
                uint32_t ov[64];
                tmem_ld32(t_o + (uint32_t)c0, *reinterpret_cast<uint32_t(*)[32]>(&ov[0]));
                tmem_ld32(t_o + (uint32_t)(c0 + 32), *reinterpret_cast<uint32_t(*)[32]>(&ov[32]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 64; c += 8) {
                        *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(
                            pack_h2(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv),
                            pack_h2(__uint_as_float(ov[c + 2]) * inv, __uint_as_float(ov[c + 3]) * inv),
                            pack_h2(__uint_as_float(ov[c + 4]) * inv, __uint_as_float(ov[c + 5]) * inv),
                            pack_h2(__uint_as_float(ov[c + 6]) * inv, __uint_as_float(ov[c + 7]) * inv));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAtTmemCols) : "memory");
    }
}

int attn_tc_timeout_flag() { return tc_flag_read_clear(); }

// Context attention on tensor-core tiles; the caller has checked fp16, D = 128 and the standard cache order.
int context_attn_tc_launch(const __half* q, long q_ld, const __half* k_cache, const __half* v_cache, int S_max, long cache_rows,
                           const int* cu_seqlens, const int* history, int B, int max_q_len, int H, int Hkv,
                           float scale, __half* out, cudaStream_t st)
{
    CUtensorMap map_k, map_v;
    int rc = make_map(&map_k, k_cache, (uint64_t)kAtD, (uint64_t)cache_rows, kAtKV);
    if (rc) return rc;
    rc = make_map(&map_v, v_cache, (uint64_t)kAtD, (uint64_t)cache_rows, kAtKV);
    if (rc) return rc;
    static DeviceOnce smem_attr;
    ONELLM_CUDA(smem_attr.run([] { return cudaFuncSetAttribute(context_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtSmemBytes); }));
    const dim3 grid((max_q_len + kAtQ - 1) / kAtQ, H, B);
    ONELLM_CUDA(launch_pdl(context_attn_tc_kernel, grid, dim3(kAtThreads), kAtSmemBytes, st, q, q_ld, map_k, map_v, cu_seqlens, history, H,
                           Hkv, S_max, scale * 1.4426950408889634f, out));
    return ONELLM_OK;
}

}  // namespace onellm
