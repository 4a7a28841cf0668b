// Context-phase causal attention on the 5th-generation tensor cores (fp16, head size 128, cache in its
// standard [B, Hkv, S, D] order).  Same arithmetic and interface as context_attn_kernel in prefill.cu (which
// stays for other head sizes and cache orders); replaces launchLinearStridedBatchGemm x2 +
// launchScaleMaskAndSoftmax + launchTransposeOutRemovePadding of
// src/layers/attention/context_attention.cpp:137-151 without the score matrix.
//
// A block owns 128 query rows of one (sequence, head) and walks the cache in tiles of 128 rows:
//   S = Q . K_tile^T      tcgen05.mma M128 N128 K16 x 8, Q and K_tile in shared memory (TMA, 128-byte swizzle,
//                         both K-major), S in tensor memory (128 columns of fp32)
//   P = exp2(S - max)     four warps, one query row per thread: the row is read from tensor memory twice
//                         (max, then exponentials), the running max / sum are per-thread scalars, P goes to
//                         shared memory as fp16 in the same swizzled K-major form a TMA load would give it
//   PV = P . V_tile       tcgen05.mma again: P is the A operand, V_tile (rows of the cache, head dimension
//                         contiguous) is the MN-major B operand, exactly as the [K,N] weights of the projections
//   O = O * alpha + PV    in registers (128 floats per thread), PV read from tensor memory
// A fifth warp issues the TMA loads (K and V tiles double-buffered) and the MMAs.  Every mbarrier wait is
// bounded; on expiry the block raises the time-out flag, stops, frees its tensor memory and returns.
#include <math.h>

#include "tc_common.cuh"

namespace onellm {

constexpr int kAtQ = 128, kAtKV = 128, kAtD = 128;
constexpr int kAtSoftmaxThreads = 256;              // eight warps: two threads per query row, 64 columns each
constexpr int kAtThreads = kAtSoftmaxThreads + 32;  // + one control warp (TMA and MMA issue)
constexpr int kAtTile = kAtQ * kAtD * 2;            // 32 KB: two 64-column chunks of [128 rows x 128 bytes]
constexpr int kAtChunk = kAtTile / 2;               // 16 KB
constexpr int kAtSmemBytes = 6 * kAtTile + 1024 /* alignment slack */ + 4096 /* barriers, TMEM address, row exchange */;

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(kAtThreads)
context_attn_tc_kernel(const __half* __restrict__ q, long q_ld, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ history, int H, int Hkv, int S_max, float scale_log2e, __half* __restrict__ out)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem;
    unsigned char* sK = smem + kAtTile;       // two buffers
    unsigned char* sV = smem + 3 * kAtTile;   // two buffers
    unsigned char* sP = smem + 5 * kAtTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kAtTile);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    float* xch = reinterpret_cast<float*>(smem + 6 * kAtTile + 128);  // [2][128]: the two halves of a row meet here
    const uint32_t q_full = smem_u32(bars), k_full0 = smem_u32(bars + 1), v_full0 = smem_u32(bars + 3), s_full0 = smem_u32(bars + 5),
                   p_full = smem_u32(bars + 7), o_full = smem_u32(bars + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (H / Hkv);

    if (threadIdx.x == 0) {
        mbar_init(q_full, kAtSoftmaxThreads);
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1);
        }
        mbar_init(p_full, kAtSoftmaxThreads);
        mbar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        // columns 0-127 and 128-255: two S accumulators (the MMA of the next tile runs under the softmax of this
        // one), 256-383: P.V of the current tile
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    pdl_wait();  // q and the cache rows come from the kernel before this one
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0, hist = history[b];
    const int q0 = blockIdx.x * kAtQ;
    const bool active = q0 < q_len;  // uniform over the block
    const int q_rows = active ? min(kAtQ, q_len - q0) : 0;
    const int kv_end = hist + q0 + q_rows;  // rows any query of this block may attend
    const int n_tiles = active ? (kv_end + kAtKV - 1) / kAtKV : 0;
    const int cache_row0 = (b * Hkv + hk) * S_max;

    if (warp == 8 && lane == 0 && active) {
        // ---- control: TMA loads and MMA issue
        bool ok = true;
        auto load_k = [&](int j) {
            const int s = j & 1;
            mbar_expect_tx(k_full0 + 8 * s, kAtTile);
#pragma unroll
            for (int c = 0; c < 2; c++)
                tma_load_2d(smem_u32(sK + s * kAtTile + c * kAtChunk), &map_k, 64 * c, cache_row0 + j * kAtKV, k_full0 + 8 * s);
        };
        auto load_v = [&](int j) {
            const int s = j & 1;
            mbar_expect_tx(v_full0 + 8 * s, kAtTile);
#pragma unroll
            for (int c = 0; c < 2; c++)
                tma_load_2d(smem_u32(sV + s * kAtTile + c * kAtChunk), &map_v, 64 * c, cache_row0 + j * kAtKV, v_full0 + 8 * s);
        };
        // instruction descriptors: D = f32, A = B = f16, M = 128, N = 128; B K-major for S, MN-major for PV
        const uint32_t idesc_s = (1u << 4) | (0u << 16) | ((uint32_t)(kAtKV >> 3) << 17) | ((uint32_t)(kAtQ >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(kAtD >> 3) << 17) | ((uint32_t)(kAtQ >> 4) << 24);
        auto issue_s = [&](int j) {  // S_j = Q . K_j^T into accumulator j & 1
            const int s = j & 1;
            if (!mbar_wait(k_full0 + 8 * s, (uint32_t)(j >> 1) & 1u)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK + s * kAtTile);
#pragma unroll
            for (int kk = 0; kk < kAtD / 16; kk++) {
                // both K-major: 64-column chunk kk/4, 32 bytes per 16 k inside the 128-byte row, 8-row groups 1024 bytes apart
                const uint32_t off = (kk >> 2) * kAtChunk + (kk & 3) * 32;
                umma_f16(tmem_base + (uint32_t)(s * 128), umma_desc(q_addr + off, 16, 1024), umma_desc(k_addr + off, 16, 1024), idesc_s,
                         kk > 0 ? 1u : 0u);
            }
            umma_commit(s_full0 + 8 * s);
            return true;
        };
        for (int j = 0; j < min(2, n_tiles); j++) {
            load_k(j);
            load_v(j);
        }
        ok = mbar_wait(q_full, 0) && issue_s(0);
        for (int j = 0; j < n_tiles && ok; j++) {
            const int s = j & 1;
            // the next tile's scores while the softmax warps work on this one (its accumulator was last read for
            // tile j - 1, whose P has been waited for in the previous round)
            if (j + 1 < n_tiles) ok = issue_s(j + 1);
            // K buffer s is free once S_j is complete
            ok = ok && mbar_wait(s_full0 + 8 * s, (uint32_t)(j >> 1) & 1u);
            if (ok && j + 2 < n_tiles) load_k(j + 2);
            ok = ok && mbar_wait(p_full, (uint32_t)j & 1u) && mbar_wait(v_full0 + 8 * s, (uint32_t)(j >> 1) & 1u);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t p_addr = smem_u32(sP), v_addr = smem_u32(sV + s * kAtTile);
#pragma unroll
            for (int kk = 0; kk < kAtKV / 16; kk++) {
                // O += P . V_tile.  A = P, K-major over the cache rows of the tile; B = V_tile, MN-major: 64-column
                // chunks 16 KB apart (LBO), 8-row groups 1024 bytes apart (SBO), 16 rows = 2048 bytes further
                const uint32_t aoff = (kk >> 2) * kAtChunk + (kk & 3) * 32;
                umma_f16(tmem_base + 256u, umma_desc(p_addr + aoff, 16, 1024), umma_desc(v_addr + kk * 2048, kAtChunk, 1024), idesc_o,
                         (j > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(o_full);
            if (j + 2 < n_tiles) {
                ok = mbar_wait(o_full, (uint32_t)j & 1u);  // V buffer s is free again
                if (ok) load_v(j + 2);
            }
        }
    } else if (warp < 8 && active) {
        // ---- softmax and output: two threads per query row, columns [64 * half, 64 * half + 64) of every tile.  O stays
        // in tensor memory and the MMA accumulates into it; it is rescaled only when a row's maximum has grown by more
        // than 2^8 over the reference the row's exponentials are taken against (P stays below 256, exact in fp16's range).
        const int r = (warp & 3) * 32 + lane;       // tensor-memory lane = query row (a warp reaches lanes 32 * (warp % 4) ..)
        const int half = warp >> 2;
        const int pos = hist + q0 + r;              // last cache row this query attends
        const bool row_ok = r < q_rows;
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t t_s = t_lane + (uint32_t)(half * 64), t_o = t_lane + 256u + (uint32_t)(half * 64);
        const uint32_t row_off = (r >> 3) * 1024 + (r & 7) * 128;  // this row inside a swizzled [128 x 128-byte] chunk
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        {
            // this thread's half of its query row into the Q tile, in the swizzled K-major form a TMA load would give it
            // (rows behind the end of the sequence are zero): the packed q buffer has no row count the host could put
            // into a tensor map without reading cu_seqlens back
            const __half* qrow = q + (size_t)(tok0 + q0 + r) * q_ld + (size_t)h * kAtD + half * 64;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const uint4 v = row_ok ? *reinterpret_cast<const uint4*>(qrow + u * 8) : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(sQ + half * kAtChunk + row_off + ((u ^ (r & 7)) << 4)) = v;
            }
            fence_async_smem();
            mbar_arrive(q_full);
        }
        for (int j = 0; j < n_tiles; j++) {
            // Every thread passes the named barrier of every tile whatever happens: after a wait that ran out
            // (ok == false) the rest of the work is skipped, never the barrier, so no warp is left waiting for another.
            ok = ok && mbar_wait(s_full0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            uint32_t sv[64];
            float mx = -INFINITY;
            float* slot = xch + (j & 1) * 256;  // the slots alternate, so one barrier per tile is enough
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int kv0 = j * kAtKV + half * 64;  // first cache row of this thread's columns
                const bool need_mask = j * kAtKV + kAtKV - 1 > hist + q0;  // some query of the block cannot see the whole tile
                tmem_ld32(t_s + (uint32_t)((j & 1) * 128), *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
                tmem_ld32(t_s + (uint32_t)((j & 1) * 128 + 32), *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    float x = __uint_as_float(sv[i]) * scale_log2e;
                    if (need_mask && kv0 + i > pos) x = -INFINITY;
                    sv[i] = __float_as_uint(x);
                    mx = fmaxf(mx, x);
                }
                slot[half * 128 + r] = mx;
            }
            softmax_barrier();  // the row maximum over both halves
            if (ok) {
                const float m_row = fmaxf(mx, slot[(half ^ 1) * 128 + r]);  // the same in both threads of the row
                const bool grow = m_row > m_ref + 8.f;  // always on the first tile: every row sees cache row 0
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_ref - m_row);  // exp2(-inf) = 0 on the first tile
                    m_ref = m_row;
                    l_run *= alpha;
                }
                if (j > 0) {
                    ok = mbar_wait(o_full, (uint32_t)(j - 1) & 1u);  // P.V of the tile before: P is free, O is at rest
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok && __any_sync(0xffffffffu, grow)) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        uint32_t ov[32];
#pragma unroll
                        for (int c = 0; c < 64; c += 32) {
                            tmem_ld32(t_o + (uint32_t)c, ov);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                            tmem_st32(t_o + (uint32_t)c, ov);
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    }
                }
            }
            if (ok) {
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    const float pv = fast_exp2(__uint_as_float(sv[i]) - m_ref);  // exp2(-inf) = 0 for masked columns
                    sum += pv;
                    sv[i] = __float_as_uint(pv);
                }
                l_run += sum;  // this thread's half of the row sum; the halves meet at the end
                // P (fp16) into chunk `half` of the P tile: 16-byte unit u of the row, XOR-ed with r % 8
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    *reinterpret_cast<uint4*>(sP + half * kAtChunk + row_off + ((u ^ (r & 7)) << 4)) =
                        make_uint4(pack_h2(__uint_as_float(sv[8 * u]), __uint_as_float(sv[8 * u + 1])),
                                   pack_h2(__uint_as_float(sv[8 * u + 2]), __uint_as_float(sv[8 * u + 3])),
                                   pack_h2(__uint_as_float(sv[8 * u + 4]), __uint_as_float(sv[8 * u + 5])),
                                   pack_h2(__uint_as_float(sv[8 * u + 6]), __uint_as_float(sv[8 * u + 7])));
                }
                if (j * kAtKV + kAtKV > kv_end) {
                    // The tile reaches beyond the rows that exist: what the cache holds there is arbitrary (possibly
                    // NaN bit patterns), and 0 x NaN would poison the product.  Thread (r, half) clears chunk `half`
                    // of cache row r of the V tile.
                    ok = mbar_wait(v_full0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
                    if (ok && j * kAtKV + r >= kv_end) {
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            *reinterpret_cast<uint4*>(sV + (j & 1) * kAtTile + half * kAtChunk + row_off + u * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                if (ok) {
                    fence_async_smem();  // P (and V rows) went through the generic proxy; the MMA reads through the async proxy
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(p_full);
                }
            }
        }
        // the two halves of the row sum, then O out of tensor memory
        softmax_barrier();
        xch[half * 128 + r] = l_run;
        softmax_barrier();
        const float l_row = l_run + xch[(half ^ 1) * 128 + r];
        ok = ok && mbar_wait(o_full, (uint32_t)(n_tiles - 1) & 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t ov[64];
            tmem_ld32(t_o, *reinterpret_cast<uint32_t(*)[32]>(&ov[0]));
            tmem_ld32(t_o + 32u, *reinterpret_cast<uint32_t(*)[32]>(&ov[32]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row_ok) {
                const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
                __half* dst = out + (size_t)(tok0 + q0 + r) * H * kAtD + (size_t)h * kAtD + half * 64;
#pragma unroll
                for (int c = 0; c < 64; c += 8) {
                    *reinterpret_cast<uint4*>(dst + c) = make_uint4(
                        pack_h2(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv),
                        pack_h2(__uint_as_float(ov[c + 2]) * inv, __uint_as_float(ov[c + 3]) * inv),
                        pack_h2(__uint_as_float(ov[c + 4]) * inv, __uint_as_float(ov[c + 5]) * inv),
                        pack_h2(__uint_as_float(ov[c + 6]) * inv, __uint_as_float(ov[c + 7]) * inv));
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
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
    static bool attr_set = false;
    if (!attr_set) {
        ONELLM_CUDA(cudaFuncSetAttribute(context_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtSmemBytes));
        attr_set = true;
    }
    const dim3 grid((max_q_len + kAtQ - 1) / kAtQ, H, B);
    ONELLM_CUDA(launch_pdl(context_attn_tc_kernel, grid, dim3(kAtThreads), kAtSmemBytes, st, q, q_ld, map_k, map_v, cu_seqlens, history, H,
                           Hkv, S_max, scale * 1.4426950408889634f, out));
    return ONELLM_OK;
}

}  // namespace onellm
