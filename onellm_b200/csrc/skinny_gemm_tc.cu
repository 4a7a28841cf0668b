// Decode-time projections with [K, N] weights for 17 to 64 tokens, on the 5th-generation tensor cores.
//
// Same contract as skinny_kn_staged_kernel (skinny_gemm_staged.cu): y = x . W, optionally with the RMS scale,
// SwiGLU of two weights, residual and bias, and the tensor-parallel exchange in the epilogue; replaces the
// cuBLAS GEMM behind launchLinearGemm (src/kernels/qkv_linear.cu:8-65 of the reference) and launchAct
// (src/kernels/activation_kernel.cu:10-21) for these shapes.
//
// The mma.sync kernel spends its time in shared-memory reads once a batch has more than a few 8-token rows: every
// warp re-reads the whole activation tile for its 16 columns (5 bytes of shared-memory traffic per weight byte at
// 64 tokens; measured 0.3 of the HBM rate on the 13B shapes at batch 64).  Here the tensor core reads both operands
// from shared memory itself:
//   D[128 weight columns, 64 tokens] += W_tile^T . x_tile^T        tcgen05.mma M128 N64 K16, kind::f16
// with the WEIGHT tile as the A operand exactly as it lies in memory ([K, N] rows = "MN-major": 64-column TMA boxes,
// 128-byte swizzle), the activations ([tokens, K], K-major) as the B operand, and the accumulator (64 columns, 128
// with two weights) in tensor memory.  One thread issues TMA loads into a ring of 64-row stages, one thread issues
// the MMAs and frees each stage with tcgen05.commit, four warps take the sum of squares of the activations from the
// ring as it passes (RMS option) and afterwards move the accumulator to shared memory, where the split-K reduction
// over the thread-block cluster and the rest of the epilogue are the code shared with the mma.sync kernel.
// Tokens beyond M and rows beyond K are zero-filled by TMA.  Every mbarrier wait is bounded; on expiry the block
// raises the time-out flag and carries on to the cluster barriers, so that no peer waits for it.
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "skinny_common.cuh"
#include "tc_common.cuh"

namespace onellm {

constexpr int kSkThreads = 192;            // producer warp, MMA warp, four auxiliary / epilogue warps
constexpr int kSkTok = 64;                 // token rows of a tile (N of the MMA)
constexpr int kSkBK = 64;                  // K rows per stage
constexpr int kSkWChunk = 64 * kSkBK * 2;  // 8 KB: 64 weight columns x 64 k
constexpr int kSkWTile = 2 * kSkWChunk;    // 16 KB: 128 weight columns x 64 k
constexpr int kSkXTile = kSkTok * kSkBK * 2;  // 8 KB: 64 tokens x 64 k
constexpr int kSkBarBytes = 256;

// WIDE: one weight, 256 output columns per block (the second 128 where DUAL has its second weight): the activation
// tile of a stage, a third of a narrow block's ring, then serves twice the weight bytes.
template <bool DUAL, bool WIDE>
__global__ void __launch_bounds__(kSkThreads)
skinny_tc_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                 const __grid_constant__ CUtensorMap map_x, __half* y, int M, int N, int K, int stages_per_block, int nst,
                 const EpilogueArgs ep)
{
    constexpr int NW = (DUAL || WIDE) ? 2 : 1;
    constexpr int kTileCols = WIDE ? 2 * kBN : kBN;
    constexpr int STAGE = NW * kSkWTile + kSkXTile;
    constexpr uint32_t kCols = NW == 2 ? 128u : 64u;  // tensor-memory columns: gate (or the first 128 outputs) at 0, up (the next 128) at 64
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nst * STAGE);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 12), acc_full = smem_u32(bars + 24);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.y;
    const int n0 = blockIdx.x * kTileCols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_stages = (K + kSkBK - 1) / kSkBK;
    const int s_begin = min(rank * stages_per_block, total_stages);
    const int n_stages = min(stages_per_block, total_stages - s_begin);
    const bool rms = ep.rms != 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, rms ? 5 : 1);  // the MMA thread's commit (+ one arrival per auxiliary warp)
        }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    float ss[4] = {0.f, 0.f, 0.f, 0.f};  // auxiliary warps: sum of squares of token rows (t >> 3) + 16 i, this thread's 16-byte column
    if (warp == 0) {
        if (lane == 0) {
            // producer.  The weights do not depend on the kernel in front of this one, the activations do: the first
            // ring of weight tiles is on its way before the dependency wait.
            auto load_w = [&](int it) {
                const int s = it % nst, k0 = (s_begin + it) * kSkBK;
                const uint32_t dst = smem_u32(smem + (size_t)s * STAGE);
                mbar_expect_tx(full0 + 8 * s, STAGE);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    tma_load_2d(dst + c * kSkWChunk, &map_w0, n0 + 64 * c, k0, full0 + 8 * s);
                    if (DUAL) tma_load_2d(dst + kSkWTile + c * kSkWChunk, &map_w1, n0 + 64 * c, k0, full0 + 8 * s);
                    if (WIDE) tma_load_2d(dst + kSkWTile + c * kSkWChunk, &map_w0, n0 + kBN + 64 * c, k0, full0 + 8 * s);
                }
            };
            auto load_x = [&](int it) {
                const int s = it % nst, k0 = (s_begin + it) * kSkBK;
                tma_load_2d(smem_u32(smem + (size_t)s * STAGE + NW * kSkWTile), &map_x, k0, 0, full0 + 8 * s);
            };
            const int pro = min(nst, n_stages);
            for (int it = 0; it < pro; it++) load_w(it);
            if (ep.early_dependents) pdl_launch_dependents();
            pdl_wait();
            for (int it = 0; it < pro; it++) load_x(it);
            bool ok = true;
            for (int it = pro; it < n_stages && ok; it++) {
                ok = mbar_wait(empty0 + 8 * (it % nst), ((it / nst) - 1) & 1);
                if (!ok) break;
                load_w(it);
                load_x(it);
            }
            if (!ep.early_dependents) pdl_launch_dependents();
        } else {
            pdl_wait();
        }
    } else if (warp == 1) {
        pdl_wait();
        if (lane == 0) {
            // D f32, A and B f16, A (weights) MN-major, B (activations) K-major, N = 64 tokens, M = 128 weight columns
            const uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(kSkTok >> 3) << 17) | ((uint32_t)(kBN >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < n_stages && ok; it++) {
                const int s = it % nst;
                ok = mbar_wait(full0 + 8 * s, (it / nst) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t w_addr = smem_u32(smem + (size_t)s * STAGE), x_addr = w_addr + NW * kSkWTile;
#pragma unroll
                for (int kk = 0; kk < kSkBK / 16; kk++) {
                    // weights: 64-column chunks 8 KB apart, groups of 8 k-rows 1 KB apart, 16 k = two groups further;
                    // activations: rows of 128 bytes, groups of 8 rows 1 KB apart, 16 k = 32 bytes further in the row
                    const uint64_t bdesc = umma_desc(x_addr + kk * 32, 16, 1024);
                    umma_f16(tmem_base, umma_desc(w_addr + kk * 2048, kSkWChunk, 1024), bdesc, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    if (NW == 2)
                        umma_f16(tmem_base + 64u, umma_desc(w_addr + kSkWTile + kk * 2048, kSkWChunk, 1024), bdesc, idesc,
                                 (it > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
            }
            umma_commit(acc_full);  // arrives when everything issued so far has run (also when the loop gave up)
        }
    } else {
        pdl_wait();
        const int t = threadIdx.x - 64;  // 0..127
        if (rms) {
            // sum of squares of the activation rows, taken from the ring: thread t reads 16-byte column t & 7 of rows
            // (t >> 3) + 16 i (a warp covers 512 consecutive bytes: no bank conflicts; the swizzle only permutes the
            // columns of a row, which a sum does not see)
            bool ok = true;
            for (int it = 0; it < n_stages && ok; it++) {
                const int s = it % nst;
                ok = mbar_wait(full0 + 8 * s, (it / nst) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const unsigned char* xt = smem + (size_t)s * STAGE + NW * kSkWTile;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float v[8];
                    Vec16<__half>::load(reinterpret_cast<const __half*>(xt + ((t >> 3) + 16 * i) * 128 + (t & 7) * 16), v);
#pragma unroll
                    for (int e = 0; e < 8; e++) ss[i] = fmaf(v[e], v[e], ss[i]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
            }
        }
        // the accumulator: tensor-memory lane = weight column of the tile, column = token
        const int q = warp & 3;  // this warp may touch lanes 32 q .. 32 q + 31
        const int c = 32 * q + lane;
        float* red = reinterpret_cast<float*>(smem);  // [NW][64][kRedLd], reuses the ring (every MMA has read it by now)
        bool ok = mbar_wait(acc_full, 0);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int w = 0; w < NW; w++)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t r[32];
                if (ok && n_stages > 0) {
                    tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(w * 64 + half * 32), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) r[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 32; i++) red[(w * kSkTok + half * 32 + i) * kRedLd + c] = __uint_as_float(r[i]);
            }
        if (rms) {
            float* red_ss = red + NW * kSkTok * kRedLd;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v = ss[i];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if ((t & 7) == 0) red_ss[(t >> 3) + 16 * i] = v;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
    }
    splitk_epilogue<kSkTok, DUAL, false, kSkThreads, WIDE>(reinterpret_cast<float*>(smem), cluster, y, M, N, K, n0, ep);
    cluster.sync();  // peers may still be reading this block's tile
}

// ---- host side -----------------------------------------------------------------------------------
struct TcPlan {
    int ks, nst, per_block;
    size_t smem;
    cudaError_t status;
};

bool plan_override_lookup(int N, int K, bool dual, int* ks, int* nst);  // skinny_gemm_staged.cu (onellm_gemm_plan_override)

static int g_tc_min_tokens = 33;  // projections of at least this many tokens take this kernel (onellm_gemm_tc_min_tokens)
static int g_tc_wide = 1;         // 256-column blocks where they apply (onellm_gemm_tc_wide)

// Shapes with a tuned plan of the narrow kernel (see plan_tc).
struct TunedTc {
    int N, K;
    bool dual;
    int ks, nst;
};
static const TunedTc kTunedTc[] = {
    {5120, 2560, false, 5, 4}, {5120, 6912, false, 4, 4},  // 2 ways (QKV: 256-column blocks beat the best narrow plan, 21.9 against 27.0 us)
    {3840, 5120, false, 4, 6}, {5120, 1280, false, 5, 3}, {3456, 5120, true, 4, 4}, {5120, 3456, false, 6, 4},  // 4 ways
    {1920, 5120, false, 8, 6}, {5120, 640, false, 5, 3},  {1728, 5120, true, 8, 4}, {5120, 1728, false, 4, 4},  // 8 ways
};

template <bool DUAL, bool WIDE>
static TcPlan plan_tc(int N, int K, bool tp)
{
    auto kern = skinny_tc_kernel<DUAL, WIDE>;
    constexpr int NW = (DUAL || WIDE) ? 2 : 1;
    constexpr int kTileCols = WIDE ? 2 * kBN : kBN;
    constexpr size_t stage = (size_t)NW * kSkWTile + kSkXTile;
    constexpr size_t red = ((size_t)NW * kSkTok * kRedLd + kSkTok) * sizeof(float);
    constexpr size_t cap = 226 * 1024;  // the kernel also has 1 KB of static shared memory
    constexpr int max_nst = (int)((cap - 1024 - kSkBarBytes) / stage);  // 9 (5 with two weights)
    static DeviceOnce attr;
    TcPlan plan = {1, 3, 0, 0, cudaSuccess};
    // the shared-memory carve-out preference comes first: the occupancy queries below answer for the carve-out the
    // kernel currently asks for, and with the default one they see a single block per SM whatever the ring depth
    plan.status = attr.run([kern] {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap);
        return e != cudaSuccess ? e : prefer_max_shared((const void*)kern);
    });
    if (plan.status != cudaSuccess) return plan;
    const int col_tiles = (N + kTileCols - 1) / kTileCols;
    const int total_stages = (K + kSkBK - 1) / kSkBK;
    int oks = 0, onst = 0;
    if (!tp && !WIDE && plan_override_lookup(N, K, DUAL, &oks, &onst)) {  // tuning aid; never cached
        const int per = oks >= 1 ? (total_stages + oks - 1) / oks : 0;
        if (oks < 1 || oks > 8 || oks > total_stages || per * (oks - 1) >= total_stages || onst < 2 || onst > max_nst) {
            plan.status = cudaErrorInvalidValue;
            return plan;
        }
        plan.ks = oks;
        plan.per_block = per;
        plan.nst = onst;
        plan.smem = std::max(stage * onst, red) + 1024 + kSkBarBytes;
        return plan;
    }
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    static std::map<std::tuple<int, int, bool, int>, TcPlan> plans;
    const auto key = std::make_tuple(N, K, tp, current_device());
    auto it = plans.find(key);
    if (it != plans.end()) return it->second;
    // How many clusters of `ks` blocks with an `nst`-stage ring the GPU holds at once (the runtime's answer).
    auto resident_clusters = [&](int ks, int nst) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 1;
        at[0].val.clusterDim.y = ks;
        at[0].val.clusterDim.z = 1;
        cfg.gridDim = dim3(col_tiles, ks, 1);
        cfg.blockDim = dim3(kSkThreads);
        cfg.dynamicSmemBytes = std::max(stage * nst, red) + 1024 + kSkBarBytes;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int clusters = 0;
        const cudaError_t oe = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
        if (oe != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        // The occupancy calculators answer one block per SM for this kernel whatever its shared memory, registers
        // (53-64) and threads would allow: they cannot know how much tensor memory a block allocates at run time.
        // A block takes 64 or 128 of the 512 columns, so two blocks share an SM when their rings fit (what the
        // timings show: the 250-tile LM head runs as one wave with a four-stage ring).  The runtime's figure for the
        // cluster size (which knows how clusters pack into GPCs) is scaled by that.
        const size_t per_block = cfg.dynamicSmemBytes + 2048;  // + static and system-reserved shared memory
        const int by_smem = (int)((size_t)228 * 1024 / per_block);
        const int per_sm = std::min(2, std::max(1, by_smem));
        return clusters * per_sm;
    };
    auto take = [&](int ks, int nst) {
        plan.ks = ks;
        plan.per_block = (total_stages + ks - 1) / ks;
        plan.nst = nst;
        plan.smem = std::max(stage * nst, red) + 1024 + kSkBarBytes;
        if (tp && (long)col_tiles * ks > kTpMaxBlocks) plan.status = cudaErrorInvalidConfiguration;
        plans[key] = plan;
        return plan;
    };
    // Plans found by the sweep of python -m onellm_b200.tune_plans (one decoder layer as a CUDA graph as the objective)
    // for the 13B shape split 2, 4 and 8 ways at 33-64 tokens: a ring of 3-6 stages leaves room for two blocks per
    // SM, which then hide each other's start-up and reduction, and allows a wider K split.  Used when all their
    // blocks are resident at once (which the tensor-parallel epilogue needs in any case).
    for (const TunedTc& t : kTunedTc) {
        if (WIDE || t.N != N || t.K != K || t.dual != DUAL || t.nst > max_nst) continue;
        const int per = (total_stages + t.ks - 1) / t.ks;
        if (t.ks > total_stages || per * (t.ks - 1) >= total_stages) continue;
        if (resident_clusters(t.ks, t.nst) >= col_tiles) return take(t.ks, t.nst);
    }
    // One block per SM (the ring takes the shared memory): the largest K split, of at least two stages per block,
    // whose blocks are all resident at once; the runtime says how many clusters of that size fit.
    int best_ks = 0;
    for (int ks = std::min(8, total_stages); ks >= 1; ks--) {
        const int per = (total_stages + ks - 1) / ks;
        if (ks > 1 && per < 2) continue;
        if ((per * (ks - 1)) >= total_stages) continue;  // the last rank would have no rows
        const int nst = std::min(max_nst, std::max(3, per));
        const size_t smem = std::max(stage * nst, red) + 1024 + kSkBarBytes;
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 1;
        at[0].val.clusterDim.y = ks;
        at[0].val.clusterDim.z = 1;
        cfg.gridDim = dim3(col_tiles, ks, 1);
        cfg.blockDim = dim3(kSkThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            clusters = num_sms() / ks;
        }
        if (clusters >= col_tiles) {
            best_ks = ks;
            break;
        }
    }
    if (best_ks == 0) {
        // More column tiles than SMs (the LM head: 250 tiles).  A four-stage ring lets two blocks share an SM: one wave
        // instead of 1.7 (13B LM head at 64 tokens: 58.6 us instead of 85.9).
        if (!WIDE && resident_clusters(1, 4) >= col_tiles) return take(1, 4);
        // else no K split and several waves (not for the tensor-parallel epilogue, whose blocks wait for the blocks of
        // the same index on the other GPUs)
        if (tp) plan.status = cudaErrorInvalidConfiguration;
        best_ks = 1;
    }
    plan.ks = best_ks;
    plan.per_block = (total_stages + best_ks - 1) / best_ks;
    plan.nst = std::min(max_nst, std::max(3, plan.per_block));
    plan.smem = std::max(stage * plan.nst, red) + 1024 + kSkBarBytes;
    if (plan.status == cudaSuccess && tp && (long)col_tiles * best_ks > kTpMaxBlocks) plan.status = cudaErrorInvalidConfiguration;
    plans[key] = plan;
    return plan;
}

template <bool DUAL, bool WIDE>
static cudaError_t launch_tc(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K, const EpilogueArgs& ep,
                             cudaStream_t st)
{
    constexpr int kTileCols = WIDE ? 2 * kBN : kBN;
    const TcPlan plan = plan_tc<DUAL, WIDE>(N, K, ep.tp.world > 1);
    if (plan.status != cudaSuccess) return plan.status;
    CUtensorMap map_w0, map_w1, map_x;
    if (make_map(&map_w0, W0, (uint64_t)N, (uint64_t)K, kSkBK) != ONELLM_OK) return cudaErrorInvalidValue;
    map_w1 = map_w0;
    if (DUAL && make_map(&map_w1, W1, (uint64_t)N, (uint64_t)K, kSkBK) != ONELLM_OK) return cudaErrorInvalidValue;
    if (make_map(&map_x, x, (uint64_t)K, (uint64_t)M, kSkTok) != ONELLM_OK) return cudaErrorInvalidValue;
    (void)prefer_max_shared((const void*)skinny_tc_kernel<DUAL, WIDE>);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = plan.ks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((N + kTileCols - 1) / kTileCols, plan.ks, 1);
    cfg.blockDim = dim3(kSkThreads);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    note_launch();
    return cudaLaunchKernelEx(&cfg, skinny_tc_kernel<DUAL, WIDE>, map_w0, map_w1, map_x, y, M, N, K, plan.per_block, plan.nst, ep);
}

cudaError_t skinny_tc_plan_query(int N, int K, bool dual, int* ks, int* nst)
{
    const TcPlan p = dual ? plan_tc<true, false>(N, K, false) : plan_tc<false, false>(N, K, false);
    *ks = p.ks;
    *nst = p.nst;
    return p.status;
}

// True when a projection of M tokens goes to this kernel rather than to the mma.sync one.
bool skinny_tc_takes(int M, int N, int K) { return M >= g_tc_min_tokens && M <= kSkTok && K % 8 == 0 && N % 8 == 0; }

cudaError_t skinny_tc_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K, const EpilogueArgs& ep,
                               cudaStream_t st)
{
    if (W1) return launch_tc<true, false>(x, W0, W1, y, M, N, K, ep, st);
    // 256-column blocks for a single weight: not with the tensor-parallel exchange in the epilogue, not where a plan of
    // the narrow kernel was tuned or is forced, and not where the narrow tiles outnumber the SMs (the LM head, which
    // runs as one wave of two narrow blocks per SM)
    bool wide = g_tc_wide != 0 && ep.tp.world <= 1 && N >= 4 * kBN && (N + kBN - 1) / kBN <= num_sms();
    int oks = 0, onst = 0;
    if (wide && plan_override_lookup(N, K, false, &oks, &onst)) wide = false;
    for (const TunedTc& t : kTunedTc)
        if (wide && g_tc_wide < 2 && t.N == N && t.K == K && !t.dual) wide = false;  // 2: sweeps compare against the tuned plans
    return wide ? launch_tc<false, true>(x, W0, nullptr, y, M, N, K, ep, st) : launch_tc<false, false>(x, W0, nullptr, y, M, N, K, ep, st);
}

int skinny_tc_flag() { return tc_flag_read_clear(); }

}  // namespace onellm

extern "C" int onellm_gemm_tc_wide(int enabled)
{
    const int before = onellm::g_tc_wide;
    if (enabled >= 0) onellm::g_tc_wide = enabled > 2 ? 1 : enabled;
    return before;
}

extern "C" int onellm_gemm_tc_min_tokens(int min_tokens)
{
    const int before = onellm::g_tc_min_tokens;
    if (min_tokens >= 1) onellm::g_tc_min_tokens = min_tokens;
    return before;
}
