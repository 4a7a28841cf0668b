// Decode-time projections with [K, N] weights, shared-memory staged: the main weight-streaming
// kernel of a decode step (QKV, o_proj, gate/up + SwiGLU, down_proj at M <= 64 tokens).
//
// Replaces the cuBLAS GEMM behind launchLinearGemm (src/kernels/qkv_linear.cu:8-65 of the
// reference) for these shapes and the SwiGLU of src/kernels/activation_kernel.cu:10-21.
//
// The weight tile of a block is 128 columns wide; it is brought in by 16-byte cp.async copies,
// 32 rows (8 KB) per stage, through a ring of stages deep enough that the bytes in flight per
// SM are set by shared memory, not by registers or by how many warps are resident.  Every
// warp-wide copy instruction covers two whole 256-byte row segments; source pointers are
// set up once and advance by a constant per stage.  The 16-byte chunks of a
// row are XOR-swizzled with the row number so that ldmatrix reads them back without bank
// conflicts; ldmatrix.trans turns the [k][n] tile into the 16x16 "row" operand of
// mma.m16n8k16 (the WEIGHT is the 16-row operand, the 8 tokens of a batch block the 8-column
// operand, so a batch of 8 wastes nothing).  The eight warps of a block split the 128 columns,
// so no cross-warp reduction is needed; K is split across the blocks of a thread-block
// cluster and the partial sums meet in distributed shared memory in a fixed order.
#include <cooperative_groups.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>

#include "skinny_common.cuh"

namespace onellm {

constexpr int kStThreads = 256;
constexpr int kKC = 32;                  // rows per stage
constexpr int kStageBytes = kKC * kBN * 2;  // 8 KB per weight matrix
constexpr int kXRowBytes = kKC * 2 + 16;   // activation rows of a stage, padded: conflict-free fragment reads

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// y[M,N] = x[M,K] . W0                    (DUAL = false)
// y[M,N] = silu(x.W0) * (x.W1)            (DUAL = true)
// grid = (ceil(N/128), KS), cluster (1, KS, 1); 256 threads; M <= 8*MB; K % 16 == 0; N % 8 == 0.
// FUSED: x is not read as is; the block first forms, for its rows of K,
//     r = x + residual (+ bias),   xn = gamma * r * rsqrt(mean_over_K(r^2) + eps)
// (the fused add-bias-residual RMSNorm of src/kernels/fused_addresidual_norm.cu:51-107 in front of
// the projection, as src/layers/decoder/self_decoder.cpp:50-73 sequences them), keeps xn in shared
// memory for the whole kernel and, in the blocks of column tile 0, stores r as the new residual.
// `x` may be NULL (r = residual: the plain RMSNorm in front of layer 0).
struct FusedNormArgs {
    const __half* residual;  // [M, K]
    const __half* bias;      // [K] or NULL
    const __half* gamma;     // [K]
    __half* residual_out;    // [M, K], must not alias residual (other blocks still read it); NULL when x is NULL
    float eps;
};

template <int MB, bool DUAL, bool FUSED>
__global__ void __launch_bounds__(kStThreads)
skinny_kn_staged_kernel(const __half* __restrict__ x, const __half* __restrict__ W0, const __half* __restrict__ W1,
                        __half* y, int M, int N, int K, int stages_per_block, int nst,
                        const FusedNormArgs fn, const EpilogueArgs ep)
{
    constexpr int NW = DUAL ? 2 : 1;
    constexpr int MP = 8 * MB;
    // a stage holds the weights and (not FUSED) the activations of the same 32 rows
    constexpr int STAGE = NW * kStageBytes + (FUSED ? 0 : MP * kXRowBytes);
    constexpr int CPT = (kKC * kBN / 8) / kStThreads;          // 16-byte weight chunks per thread and stage (2)
    extern __shared__ __align__(128) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int KS = gridDim.y, rank = blockIdx.y;
    const int n0 = blockIdx.x * kBN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int k_begin = rank * stages_per_block * kKC;
    const int k_end = min(k_begin + stages_per_block * kKC, K);
    const int n_stages = k_end > k_begin ? (k_end - k_begin + kKC - 1) / kKC : 0;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    // Copy assignments, fixed for the whole kernel: chunk c = tid + 256*i is row c/16 of the stage,
    // 16-byte column c%16.  Source pointers advance by 32 rows per stage; destinations are offsets
    // inside a stage (XOR-swizzled by the row).
    const __half* wsrc[NW][CPT];
    uint32_t wdst[CPT];
    int wrow[CPT];
    bool wcol_ok[CPT];
#pragma unroll
    for (int i = 0; i < CPT; i++) {
        const int c = tid + kStThreads * i;
        const int row = c >> 4, c16 = c & 15;
        const int col = n0 + c16 * 8;
        wrow[i] = row;
        wcol_ok[i] = col < N;
        wdst[i] = row * (kBN * 2) + ((c16 ^ (row & 7)) << 4);
        const size_t off = (size_t)(k_begin + row) * N + (wcol_ok[i] ? col : 0);
        wsrc[0][i] = W0 + off;
        if (DUAL) wsrc[NW - 1][i] = W1 + off;
    }
    const size_t wstep = (size_t)kKC * N;
    // activations: thread tid < 4*MP copies 16 bytes of row tid/4
    const bool x_thread = !FUSED && tid < MP * 4;
    const int x_part = tid & 3;
    const __half* xsrc = FUSED ? x : x + (size_t)min(tid >> 2, M - 1) * K + k_begin + x_part * 8;
    const uint32_t xdst = NW * kStageBytes + (tid >> 2) * kXRowBytes + x_part * 16;

    int w_issued = 0, x_issued = 0;  // stages whose copies have been issued
    auto issue_w = [&](uint32_t sbase) {
        if (w_issued < n_stages) {
            const int rows_left = k_end - (k_begin + w_issued * kKC);
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
                for (int i = 0; i < CPT; i++) {
                    const bool ok = wcol_ok[i] && wrow[i] < rows_left;
                    cp_async16(sbase + w * kStageBytes + wdst[i], ok ? (const void*)wsrc[w][i] : (const void*)W0, ok ? 16 : 0);
                    wsrc[w][i] += wstep;
                }
        }
        w_issued++;
    };
    auto issue_x = [&](uint32_t sbase) {
        if (x_issued < n_stages && x_thread) {
            const bool ok = k_begin + x_issued * kKC + x_part * 8 < k_end;
            cp_async16(sbase + xdst, ok ? (const void*)xsrc : (const void*)x, ok ? 16 : 0);
            xsrc += kKC;
        }
        x_issued++;
    };

    float ssq[MB];  // warp 0: this block's share of sum(x^2) per token (EpilogueArgs::rms)
#pragma unroll
    for (int mb = 0; mb < MB; mb++) ssq[mb] = 0.f;
    float acc[NW][MB][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[w][mb][e] = 0.f;

    // The weights do not depend on the kernel that ran before this one, the activations do:
    // fill the ring with weights first and only then wait for the producer of x (programmatic
    // dependent launch; a no-op for a plain launch).  The next kernel in the stream is released
    // either here (EpilogueArgs::early_dependents: hides its launch latency; measured 2 % faster over
    // a decode step) or after the main loop.
    // one commit group per stage: the first stage can be consumed as soon as ITS weights have landed
    for (int s = 0; s < nst - 1; s++) {
        issue_w(smem_base + (uint32_t)(s * STAGE));
        cp_async_commit();
    }
    if (ep.early_dependents) pdl_launch_dependents();
    pdl_wait();
    // FUSED: normalised activations of this block's K range, [MP][xn_ld] halfs behind the ring
    const int kc = stages_per_block * kKC;               // K range of a block (multiple of 32)
    const int xn_ld = kc + 8;                            // row stride in halfs: an odd number of 16-byte units
    __half* xn = reinterpret_cast<__half*>(smem + (size_t)nst * STAGE);
    if (FUSED) {
        __shared__ float inv_rms[MP];
        // one warp per token row: r = x + residual + bias over the whole row, sum of squares by shuffles
        for (int m = warp; m < MP; m += kStThreads / 32) {
            const int mr = min(m, M - 1);
            const __half* xr = x ? x + (size_t)mr * K : nullptr;
            const __half* rr = fn.residual + (size_t)mr * K;
            float ss = 0.f;
            // loads are issued eight vectors at a time before any of them is used: the row comes
            // from L2 and a load-use-load chain would cost one L2 round trip per vector
            constexpr int NB = 8;
            const int nv = K / 8;
            for (int i0 = lane; i0 < nv; i0 += 32 * NB) {
                uint4 rv[NB], xv[NB], bv[NB];
#pragma unroll
                for (int j = 0; j < NB; j++) {
                    const int i = i0 + 32 * j;
                    const bool in = i < nv;
                    rv[j] = in ? *reinterpret_cast<const uint4*>(rr + (size_t)i * 8) : make_uint4(0, 0, 0, 0);
                    xv[j] = (in && xr) ? *reinterpret_cast<const uint4*>(xr + (size_t)i * 8) : make_uint4(0, 0, 0, 0);
                    bv[j] = (in && xr && fn.bias) ? *reinterpret_cast<const uint4*>(fn.bias + (size_t)i * 8)
                                                  : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < NB; j++) {
                    const int i = i0 + 32 * j;
                    if (i >= nv) break;
                    float v[8], a[8], c[8];
                    Vec16<__half>::unpack(rv[j], v);
                    Vec16<__half>::unpack(xv[j], a);
                    Vec16<__half>::unpack(bv[j], c);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        v[e] = v[e] + a[e] + c[e];
                        ss = fmaf(v[e], v[e], ss);
                    }
                    const int k = i * 8;
                    if (k >= k_begin && k < k_end) {
                        const uint4 packed = Vec16<__half>::pack(v);
                        *reinterpret_cast<uint4*>(xn + (size_t)m * xn_ld + (k - k_begin)) = packed;
                        if (blockIdx.x == 0 && fn.residual_out && m < M)
                            *reinterpret_cast<uint4*>(fn.residual_out + (size_t)m * K + k) = packed;
                    }
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) inv_rms[m] = rsqrtf(ss / (float)K + fn.eps);
        }
        __syncthreads();
        const int nvec = (k_end - k_begin) / 8;
        for (int idx = tid; idx < MP * nvec; idx += kStThreads) {
            const int m = idx / nvec, i = idx % nvec;
            float v[8], gmm[8];
            Vec16<__half>::load(xn + (size_t)m * xn_ld + i * 8, v);
            Vec16<__half>::load(fn.gamma + k_begin + i * 8, gmm);
            const float inv = inv_rms[m];
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = gmm[e] * v[e] * inv;
            *reinterpret_cast<uint4*>(xn + (size_t)m * xn_ld + i * 8) = Vec16<__half>::pack(v);
        }
        // visibility to the other warps: the barrier at the top of the main loop
    } else {
        // Activations of the stages already on their way: plain loads (they sit in L2, the producer has
        // just written them) stored to shared memory by the thread that will later copy them
        // asynchronously.  Had they joined the ring as one more copy group, the first stage would have
        // to wait for every weight copy issued above.
        constexpr int kMaxPro = 11;  // ring depth is at most 12
        if (x_thread) {
            uint4 xv[kMaxPro];
#pragma unroll
            for (int s = 0; s < kMaxPro; s++) {
                xv[s] = make_uint4(0u, 0u, 0u, 0u);
                if (s < nst - 1 && s < n_stages && k_begin + s * kKC + x_part * 8 < k_end)
                    xv[s] = *reinterpret_cast<const uint4*>(xsrc + (size_t)s * kKC);
            }
#pragma unroll
            for (int s = 0; s < kMaxPro; s++)
                if (s < nst - 1) *reinterpret_cast<uint4*>(smem + (size_t)s * STAGE + xdst) = xv[s];
            xsrc += (size_t)(nst - 1) * kKC;
        }
        x_issued = nst - 1;
        // visible to the other warps through the barrier at the top of the main loop
    }
    uint32_t cons = 0, fill = (uint32_t)((nst - 1) * STAGE);  // byte offsets of the slot consumed / refilled
    const uint32_t ring_bytes = (uint32_t)(nst * STAGE);

    // ldmatrix source of this lane inside a 16-row step: matrix m = lane/8 -> rows (m/2)*8 + lane%8,
    // columns +8 for odd m; this warp owns columns 16*warp .. 16*warp+15 of the tile
    const int lm_row = ((lane >> 4) << 3) + (lane & 7);
    const int lm_c16 = warp * 2 + ((lane >> 3) & 1);
    const uint32_t lm_off0 = lm_row * (kBN * 2) + ((lm_c16 ^ (lm_row & 7)) << 4);          // rows 0..15
    const uint32_t lm_off1 = (16 + lm_row) * (kBN * 2) + ((lm_c16 ^ (lm_row & 7)) << 4);   // rows 16..31
    const uint32_t xb_off = NW * kStageBytes + g * kXRowBytes + 4 * t;

    for (int s = 0; s < n_stages; s++) {
        cp_async_wait_dyn(nst - 2);
        __syncthreads();
        issue_w(smem_base + fill);
        issue_x(smem_base + fill);
        cp_async_commit();
        const uint32_t sbase = smem_base + cons;
        const unsigned char* xs = FUSED ? reinterpret_cast<const unsigned char*>(xn) + (size_t)g * xn_ld * 2 + (size_t)s * kKC * 2 + 4 * t
                                        : smem + cons + xb_off;
        const int x_row_bytes = FUSED ? xn_ld * 2 : kXRowBytes;
        cons = cons + STAGE == ring_bytes ? 0 : cons + STAGE;
        fill = fill + STAGE == ring_bytes ? 0 : fill + STAGE;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            uint32_t xb[MB][2];
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                const unsigned char* p = xs + 8 * mb * x_row_bytes + 32 * kk;
                xb[mb][0] = *reinterpret_cast<const uint32_t*>(p);
                xb[mb][1] = *reinterpret_cast<const uint32_t*>(p + 16);
            }
            if (!FUSED && ep.rms && warp == 0) {
                // lane (g, t) holds x[token 8*mb + g][k = 2t, 2t+1, 2t+8, 2t+9] of this 16-row step
#pragma unroll
                for (int mb = 0; mb < MB; mb++) {
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&xb[mb][0]));
                    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&xb[mb][1]));
                    ssq[mb] = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ssq[mb]))));
                }
            }
#pragma unroll
            for (int w = 0; w < NW; w++) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, sbase + w * kStageBytes + (kk ? lm_off1 : lm_off0));
                // ldmatrix order is (n 0-7, k 0-7), (n 8-15, k 0-7), (n 0-7, k 8-15), (n 8-15, k 8-15)
                // = a0, a1, a2, a3 of the mma "row" operand
#pragma unroll
                for (int mb = 0; mb < MB; mb++) mma16816(acc[w][mb], a, xb[mb][0], xb[mb][1]);
            }
        }
    }
    cp_async_wait<0>();
    if (!ep.early_dependents) pdl_launch_dependents();
    __syncthreads();

    // this block's partial tile, then the cluster-wide sum in rank order
    float* red = reinterpret_cast<float*>(smem);  // [NW][MP][kRedLd]
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int tok = 8 * mb + 2 * t + (e & 1);
                const int c = warp * 16 + g + ((e & 2) ? 8 : 0);
                red[(w * MP + tok) * kRedLd + c] = acc[w][mb][e];
            }
    float* red_ss = red + NW * MP * kRedLd;  // [MP] partial sums of squares
    if (!FUSED && ep.rms && warp == 0) {
#pragma unroll
        for (int mb = 0; mb < MB; mb++) {
            float v = ssq[mb];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) red_ss[8 * mb + g] = v;
        }
    }
    splitk_epilogue<MP, DUAL, FUSED, kStThreads>(red, cluster, y, M, N, K, n0, ep);
    cluster.sync();  // peers may still be reading this block's tile
}

// Resident blocks of `kern` for a cluster size and ring depth (cached).
template <typename Kern>
static int staged_slots(Kern kern, int ks, int nst, size_t smem, int col_blocks)
{
    // one table for every instantiation (they share the function-pointer type): the kernel is
    // part of the key
    static std::map<std::tuple<const void*, int, size_t, int>, int> cache;
    static std::mutex cache_mu;  // the planners of different instantiations reach this table under their own locks
    const auto key = std::make_tuple((const void*)kern, ks, smem, current_device());  // occupancy is a per-device figure
    (void)nst;
    {
        std::lock_guard<std::mutex> lock(cache_mu);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(col_blocks, ks, 1);
    cfg.blockDim = dim3(kStThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
        (void)cudaGetLastError();
        clusters = num_sms() / ks;
    }
    std::lock_guard<std::mutex> lock(cache_mu);
    cache[key] = clusters * ks;
    return clusters * ks;
}

// Launch plan of one projection shape: K split (= cluster size), ring depth, stages per block.
struct StagedPlan {
    int ks, nst, per_block;
    size_t smem;
    cudaError_t status;  // cudaErrorInvalidConfiguration: the tensor-parallel epilogue was asked for and no plan fits one wave
};

// Launch plans found by sweeping (K split, ring depth) with the decoder layer's five kernels as one CUDA graph as the
// objective (batch 8, B200): the Llama-2-7B projections whole and sliced 2, 4 and 8 ways.  The general rule below
// (most bytes in flight with every block resident) is within a few percent on the whole shapes but picks too few,
// too deep blocks for the narrow slices (the 2-way gate/up slice: 129 blocks of 12 stages, 21 us; 215 blocks of
// 4 stages, 10 us less for the layer).
struct TunedPlan {
    int N, K;
    bool dual;
    int ks, nst;
};
static const TunedPlan kTunedPlans[] = {
    {12288, 4096, false, 5, 5}, {4096, 4096, false, 8, 8},  {11008, 4096, true, 3, 6}, {4096, 11008, false, 8, 10},
    {6144, 4096, false, 8, 6},  {4096, 2048, false, 6, 5},  {5504, 4096, true, 5, 4},  {4096, 5504, false, 8, 10},
    {3072, 4096, false, 8, 10}, {4096, 1024, false, 6, 4},  {2752, 4096, true, 8, 5},  {4096, 2752, false, 8, 8},
    {1536, 4096, false, 8, 4},  {4096, 512, false, 4, 4},   {1376, 4096, true, 8, 5},  {4096, 1376, false, 8, 4},
};

// Plans forced from outside (onellm_gemm_plan_override): (N, K, dual) -> (K split, ring depth)
static std::map<std::tuple<int, int, bool>, std::pair<int, int>>& plan_overrides()
{
    static std::map<std::tuple<int, int, bool>, std::pair<int, int>> t;
    return t;
}
static std::mutex g_override_mu;

template <int MB, bool DUAL, bool FUSED>
static StagedPlan plan_staged(int N, int K, bool tp)
{
    auto kern = skinny_kn_staged_kernel<MB, DUAL, FUSED>;
    constexpr int NW = DUAL ? 2 : 1;
    constexpr size_t stage = (size_t)NW * kStageBytes + (FUSED ? 0 : 8 * MB * kXRowBytes);
    constexpr size_t red = ((size_t)NW * 8 * MB * kRedLd + 8 * MB) * sizeof(float);
    constexpr size_t smem_cap = 226 * 1024;
    static DeviceOnce smem_attr;
    StagedPlan plan = {1, 3, 0, 0, cudaSuccess};
    plan.status = smem_attr.run([kern] {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap);
        if (e != cudaSuccess) return e;
        return prefer_max_shared((const void*)kern);
    });
    if (plan.status != cudaSuccess) return plan;
    const int col_blocks = (N + kBN - 1) / kBN;
    const int total_stages = (K + kKC - 1) / kKC;
    {
        std::lock_guard<std::mutex> lock(g_override_mu);
        auto ov = plan_overrides().find(std::make_tuple(N, K, DUAL));
        if (ov != plan_overrides().end() && !tp) {
            plan.ks = std::max(1, std::min(ov->second.first, std::min(8, total_stages)));
            plan.nst = std::max(3, std::min(ov->second.second, 12));  // the prologue holds at most 11 stages of activations in registers
            plan.per_block = (total_stages + plan.ks - 1) / plan.ks;
            const size_t xn = FUSED ? (size_t)8 * MB * (plan.per_block * kKC + 8) * sizeof(__half) : 0;
            plan.smem = std::max(stage * plan.nst, red) + xn;
            if (plan.smem > smem_cap) plan.status = cudaErrorInvalidConfiguration;
            return plan;
        }
    }
    static std::mutex mu;  // the plan and occupancy caches
    std::lock_guard<std::mutex> lock(mu);
    static std::map<std::tuple<int, int, bool, int>, StagedPlan> plans;  // one table per instantiation
    const auto key = std::make_tuple(N, K, tp, current_device());
    auto it = plans.find(key);
    if (it != plans.end()) return it->second;
    // Shapes that were swept on B200 (python -m onellm_b200.tune_plans) take the plan that made the whole decoder layer
    // fastest, as long as its blocks are all resident at once on this device.
    if (MB == 1 && !FUSED) {
        for (const TunedPlan& t : kTunedPlans) {
            if (t.N != N || t.K != K || t.dual != DUAL || t.ks > total_stages) continue;
            const int per = (total_stages + t.ks - 1) / t.ks;
            const size_t smem = std::max(stage * t.nst, red);
            if (smem > smem_cap || per * (t.ks - 1) >= total_stages) break;
            if (staged_slots(kern, t.ks, t.nst, smem, col_blocks) < (long)col_blocks * t.ks) break;
            if (tp && (long)col_blocks * t.ks > kTpMaxBlocks) break;
            plan.ks = t.ks;
            plan.nst = t.nst;
            plan.per_block = per;
            plan.smem = smem;
            plans[key] = plan;
            return plan;
        }
    }
    // The K split (= cluster size, 1..8) and ring depth that keep the most bytes in flight
    // while every block is resident at once (residency asked from the runtime, because clusters
    // do not always pack the SMs of a GPC fully).  A sweep over (split, depth) on B200 for the
    // four projection shapes of the 7B model agrees with this rule within a microsecond.
    int best_ks = 1, best_nst = 3;
    double best_inflight = -1.0;
    for (int ks = 1; ks <= 8; ks++) {
        const int per = (total_stages + ks - 1) / ks;
        if (ks > 1 && per < 4) break;
        const long total = (long)col_blocks * ks;
        const size_t xn_b = FUSED ? (size_t)8 * MB * (per * kKC + 8) * sizeof(__half) : 0;
        for (int nst = std::min(12, std::max(3, per + 1)); nst >= 3; nst--) {
            const size_t smem = std::max(stage * nst, red) + xn_b;
            if (smem > smem_cap) continue;
            if (staged_slots(kern, ks, nst, smem, col_blocks) < total) continue;
            // FUSED: every block redoes the row statistics, so fewer blocks are better there
            const double inflight = (double)total * (nst - 1) * (double)(NW * kStageBytes) / (FUSED ? (double)ks : 1.0);
            if (inflight > best_inflight * 1.02) {
                best_inflight = inflight;
                best_ks = ks;
                best_nst = nst;
            }
            break;  // shallower rings for this split only lose
        }
    }
    if (best_inflight < 0) {  // nothing fits in one wave: smallest blocks, shallow ring
        // (not for the tensor-parallel epilogue: its blocks wait for their peers on other GPUs, which is
        // only free of deadlock when every block of the launch is resident)
        if (tp) plan.status = cudaErrorInvalidConfiguration;
        best_ks = 1;
        best_nst = 3;
    }
    plan.ks = best_ks;
    plan.nst = best_nst;
    plan.per_block = (total_stages + best_ks - 1) / best_ks;
    const size_t xn_final = FUSED ? (size_t)8 * MB * (plan.per_block * kKC + 8) * sizeof(__half) : 0;
    plan.smem = std::max(stage * best_nst, red) + xn_final;
    if (plan.status == cudaSuccess && plan.smem > smem_cap) plan.status = cudaErrorInvalidConfiguration;
    if (plan.status == cudaSuccess && tp && (long)col_blocks * best_ks > kTpMaxBlocks) plan.status = cudaErrorInvalidConfiguration;
    plans[key] = plan;
    return plan;
}

template <int MB, bool DUAL, bool FUSED>
static cudaError_t launch_staged(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K,
                                 const FusedNormArgs& fn, const EpilogueArgs& ep, cudaStream_t st)
{
    auto kern = skinny_kn_staged_kernel<MB, DUAL, FUSED>;
    const StagedPlan plan = plan_staged<MB, DUAL, FUSED>(N, K, ep.tp.world > 1);
    if (plan.status != cudaSuccess) return plan.status;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = plan.ks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((N + kBN - 1) / kBN, plan.ks, 1);
    cfg.blockDim = dim3(kStThreads);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    note_launch();
    return cudaLaunchKernelEx(&cfg, kern, x, W0, W1, y, M, N, K, plan.per_block, plan.nst, fn, ep);
}

template <int MB>
static StagedPlan plan_for(bool dual, int N, int K)
{
    return dual ? plan_staged<MB, true, false>(N, K, false) : plan_staged<MB, false, false>(N, K, false);
}

// The plan a projection of M tokens would be launched with (K split, ring depth, thread blocks).
bool skinny_tc_takes(int M, int N, int K);                                      // skinny_gemm_tc.cu
cudaError_t skinny_tc_plan_query(int N, int K, bool dual, int* ks, int* nst);  // skinny_gemm_tc.cu

cudaError_t staged_plan_query(int M, int N, int K, bool dual, int* ks, int* nst, int* blocks)
{
    if (skinny_tc_takes(M, N, K)) {
        int k = 1, n = 3;
        const cudaError_t e = skinny_tc_plan_query(N, K, dual, &k, &n);
        if (ks) *ks = k;
        if (nst) *nst = n;
        if (blocks) *blocks = k * ((N + kBN - 1) / kBN);
        return e;
    }
    const StagedPlan p = M <= 8 ? plan_for<1>(dual, N, K) : M <= 16 ? plan_for<2>(dual, N, K) : M <= 32 ? plan_for<4>(dual, N, K) : plan_for<8>(dual, N, K);
    if (ks) *ks = p.ks;
    if (nst) *nst = p.nst;
    if (blocks) *blocks = p.ks * ((N + kBN - 1) / kBN);
    return p.status;
}

// The override registered for a shape, if any (also honoured by the tcgen05 kernel's planner).
bool plan_override_lookup(int N, int K, bool dual, int* ks, int* nst)
{
    std::lock_guard<std::mutex> lock(g_override_mu);
    auto ov = plan_overrides().find(std::make_tuple(N, K, dual));
    if (ov == plan_overrides().end()) return false;
    *ks = ov->second.first;
    *nst = ov->second.second;
    return true;
}

void staged_plan_override(int N, int K, bool dual, int ks, int nst)
{
    std::lock_guard<std::mutex> lock(g_override_mu);
    if (ks <= 0)
        plan_overrides().erase(std::make_tuple(N, K, dual));
    else
        plan_overrides()[std::make_tuple(N, K, dual)] = std::make_pair(ks, nst);
}

// skinny_gemm_tc.cu
bool skinny_tc_takes(int M, int N, int K);
cudaError_t skinny_tc_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K, const EpilogueArgs& ep,
                               cudaStream_t st);

// One pass of at most 64 tokens.  Called from skinny_gemm.cu.
cudaError_t skinny_kn_staged_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                      int K, bool dual, cudaStream_t st, const __half* resid, const __half* bias,
                                      float rms_eps, const TpEpilogue* tp)
{
    const FusedNormArgs none = {nullptr, nullptr, nullptr, nullptr, 0.f};
    if (skinny_tc_takes(M, N, K)) {  // more than a few 8-token rows: the tcgen05 kernel (skinny_gemm_tc.cu)
        const EpilogueArgs ep_tc = {resid, resid ? bias : nullptr, rms_eps, rms_eps >= 0.f ? 1 : 0, 1, tp ? *tp : TpEpilogue{}};
        return skinny_tc_dispatch(x, W0, dual ? W1 : nullptr, y, M, N, K, ep_tc, st);
    }
    // the next kernel is released as soon as this one's first weight copies are out: its blocks cannot
    // become resident before blocks of this kernel retire (shared memory), but its launch latency is hidden
    const EpilogueArgs ep = {resid, resid ? bias : nullptr, rms_eps, rms_eps >= 0.f ? 1 : 0, 1, tp ? *tp : TpEpilogue{}};
    if (dual) {
        if (M <= 8) return launch_staged<1, true, false>(x, W0, W1, y, M, N, K, none, ep, st);
        if (M <= 16) return launch_staged<2, true, false>(x, W0, W1, y, M, N, K, none, ep, st);
        if (M <= 32) return launch_staged<4, true, false>(x, W0, W1, y, M, N, K, none, ep, st);
        return launch_staged<8, true, false>(x, W0, W1, y, M, N, K, none, ep, st);
    }
    if (M <= 8) return launch_staged<1, false, false>(x, W0, nullptr, y, M, N, K, none, ep, st);
    if (M <= 16) return launch_staged<2, false, false>(x, W0, nullptr, y, M, N, K, none, ep, st);
    if (M <= 32) return launch_staged<4, false, false>(x, W0, nullptr, y, M, N, K, none, ep, st);
    return launch_staged<8, false, false>(x, W0, nullptr, y, M, N, K, none, ep, st);
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_add_residual_rmsnorm_gemm(int dtype, const void* x, const void* residual, const void* bias,
                                                const void* gamma, float eps, void* residual_out, const void* W,
                                                const void* Wu, void* y, int M, int N, int K, void* stream)
{
    ONELLM_REQUIRE(residual && gamma && W && y, ONELLM_ERR_ARG, "add_residual_rmsnorm_gemm: null pointer");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "add_residual_rmsnorm_gemm: only F16 is implemented");
    ONELLM_REQUIRE(M >= 0 && N > 0 && K > 0, ONELLM_ERR_ARG, "add_residual_rmsnorm_gemm: bad size");
    ONELLM_REQUIRE(M <= 16, ONELLM_ERR_UNSUPPORTED,
                   "add_residual_rmsnorm_gemm: covers M <= 16; use onellm_add_residual_rmsnorm then onellm_gemm");
    ONELLM_REQUIRE(K % 16 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED,
                   "add_residual_rmsnorm_gemm: need K %% 16 == 0 and N %% 8 == 0");
    ONELLM_REQUIRE(!x || residual_out, ONELLM_ERR_ARG, "add_residual_rmsnorm_gemm: residual_out is required when x is given");
    ONELLM_REQUIRE(residual_out != residual, ONELLM_ERR_ARG,
                   "add_residual_rmsnorm_gemm: residual_out must not alias residual");
    ONELLM_REQUIRE(aligned16(residual) && aligned16(gamma) && aligned16(W) && aligned16(y) && (!x || aligned16(x)) &&
                       (!bias || aligned16(bias)) && (!Wu || aligned16(Wu)) && (!residual_out || aligned16(residual_out)),
                   ONELLM_ERR_ARG, "add_residual_rmsnorm_gemm: pointers must be 16-byte aligned");
    if (M == 0) return ONELLM_OK;
    const FusedNormArgs fn = {(const __half*)residual, (const __half*)bias, (const __half*)gamma,
                              x ? (__half*)residual_out : nullptr, eps};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half *xh = (const __half*)x, *w0 = (const __half*)W, *w1 = (const __half*)Wu;
    __half* yh = (__half*)y;
    const EpilogueArgs no_ep = {nullptr, nullptr, 0.f, 0, 0, TpEpilogue{}};
    cudaError_t e;
    if (Wu)
        e = M <= 8 ? launch_staged<1, true, true>(xh, w0, w1, yh, M, N, K, fn, no_ep, st)
                   : launch_staged<2, true, true>(xh, w0, w1, yh, M, N, K, fn, no_ep, st);
    else
        e = M <= 8 ? launch_staged<1, false, true>(xh, w0, nullptr, yh, M, N, K, fn, no_ep, st)
                   : launch_staged<2, false, true>(xh, w0, nullptr, yh, M, N, K, fn, no_ep, st);
    ONELLM_REQUIRE(e == cudaSuccess, ONELLM_ERR_CUDA, "add_residual_rmsnorm_gemm: %s", cudaGetErrorString(e));
    return ONELLM_OK;
}
