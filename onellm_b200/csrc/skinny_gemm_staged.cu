// Decode-time projections with [K, N] weights, shared-memory staged: the main weight-streaming
// kernel of a decode step (QKV, o_proj, gate/up + SwiGLU, down_proj at M <= 64 tokens).
//
// Replaces the cuBLAS GEMM behind launchLinearGemm (src/kernels/qkv_linear.cu:8-65 of the
// reference) for these shapes and the SwiGLU of src/kernels/activation_kernel.cu:10-21.
//
// The weight tile of a block is 128 columns wide; it is brought in by 16-byte cp.async copies,
// 32 rows (8 KB) per stage, through a ring of stages deep enough that the bytes in flight per
// SM are set by shared memory, not by registers or by how many warps are resident.  Every
// warp-wide copy instruction covers two whole 256-byte row segments.  The 16-byte chunks of a
// row are XOR-swizzled with the row number so that ldmatrix reads them back without bank
// conflicts; ldmatrix.trans turns the [k][n] tile into the 16x16 "row" operand of
// mma.m16n8k16 (the WEIGHT is the 16-row operand, the 8 tokens of a batch block the 8-column
// operand, so a batch of 8 wastes nothing).  The four warps of a block split the 128 columns,
// so no cross-warp reduction is needed; K is split across the blocks of a thread-block
// cluster and the partial sums meet in distributed shared memory in a fixed order.
#include <cooperative_groups.h>
#include <math.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace onellm {

constexpr int kStThreads = 128;
constexpr int kBN = 128;                 // columns per block
constexpr int kKC = 32;                  // rows per stage
constexpr int kStageBytes = kKC * kBN * 2;  // 8 KB per weight matrix
constexpr int kRedLd = kBN + 1;
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
// grid = (ceil(N/128), KS), cluster (1, KS, 1); M <= 8*MB; K % 16 == 0; N % 8 == 0.
template <int MB, bool DUAL>
__global__ void __launch_bounds__(kStThreads)
skinny_kn_staged_kernel(const __half* __restrict__ x, const __half* __restrict__ W0, const __half* __restrict__ W1,
                        __half* __restrict__ y, int M, int N, int K, int stages_per_block, int nst)
{
    constexpr int NW = DUAL ? 2 : 1;
    constexpr int MP = 8 * MB;
    constexpr int STAGE = NW * kStageBytes + MP * kXRowBytes;  // weights, then the activations of the same rows
    extern __shared__ __align__(128) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int KS = gridDim.y, rank = blockIdx.y;
    const int n0 = blockIdx.x * kBN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int k_begin = rank * stages_per_block * kKC;
    const int k_end = min(k_begin + stages_per_block * kKC, K);
    const int n_stages = k_end > k_begin ? (k_end - k_begin + kKC - 1) / kKC : 0;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    // copy assignments of this thread: chunk c = tid + 128*i -> row c/16, 16-byte column c%16;
    // `buf` is the ring slot of stage s (s % nst, tracked by the caller)
    auto issue_w = [&](int s, int buf) {
        if (s < n_stages) {
            const int k0 = k_begin + s * kKC;
            const uint32_t sbase = smem_base + (uint32_t)(buf * STAGE);
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const __half* W = w == 0 ? W0 : W1;
#pragma unroll
                for (int i = 0; i < (kKC * kBN / 8) / kStThreads; i++) {
                    const int c = tid + kStThreads * i;
                    const int row = c >> 4, c16 = c & 15;
                    const int k = k0 + row, col = n0 + c16 * 8;
                    const bool ok = k < k_end && col < N;
                    const __half* src = ok ? W + (size_t)k * N + col : W;
                    const uint32_t dst = sbase + w * kStageBytes + row * (kBN * 2) + ((c16 ^ (row & 7)) << 4);
                    cp_async16(dst, src, ok ? 16 : 0);
                }
            }
        }
    };
    // activations x[0..MP)[k0..k0+32): MP rows of four 16-byte chunks
    auto issue_x = [&](int s, int buf) {
        if (s < n_stages) {
            const int k0 = k_begin + s * kKC;
            const uint32_t sbase = smem_base + (uint32_t)(buf * STAGE);
            for (int c = tid; c < MP * 4; c += kStThreads) {
                const int row = c >> 2, part = c & 3;
                const int k = k0 + part * 8;
                const bool ok = k < k_end;
                const __half* src = ok ? x + (size_t)min(row, M - 1) * K + k : x;
                cp_async16(sbase + NW * kStageBytes + row * kXRowBytes + part * 16, src, ok ? 16 : 0);
            }
        }
    };

    float acc[NW][2][MB][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int ng = 0; ng < 2; ng++)
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[w][ng][mb][e] = 0.f;

    // The weights do not depend on the kernel that ran before this one, the activations do:
    // fill the ring with weights first and only then wait for the producer of x (programmatic
    // dependent launch; a no-op for a plain launch).  The next kernel in the stream is released
    // after the main loop, so that its prologue overlaps this kernel's reduction but its blocks
    // do not take shared memory from this kernel's ring.
    for (int s = 0; s < nst - 1; s++) issue_w(s, s);
    pdl_wait();
    for (int s = 0; s < nst - 1; s++) {
        issue_x(s, s);
        cp_async_commit();  // group 0 also carries every weight copy issued above
    }
    int buf = 0, fill = nst - 1;  // slot being consumed, slot being refilled

    // ldmatrix source of this lane inside a 16-row step: matrix m = lane/8 -> rows (m/2)*8 + lane%8,
    // columns +8 for odd m
    const int lm_row = ((lane >> 4) << 3) + (lane & 7);
    const int lm_col16 = (lane >> 3) & 1;

    for (int s = 0; s < n_stages; s++) {
        cp_async_wait_dyn(nst - 2);
        __syncthreads();
        issue_w(s + nst - 1, fill);
        issue_x(s + nst - 1, fill);
        cp_async_commit();
        const uint32_t sbase = smem_base + (uint32_t)(buf * STAGE);
        const unsigned char* xs = smem + buf * STAGE + NW * kStageBytes;
        buf = buf + 1 == nst ? 0 : buf + 1;
        fill = fill + 1 == nst ? 0 : fill + 1;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            uint32_t xb[MB][2];
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                const unsigned char* p = xs + (8 * mb + g) * kXRowBytes + (16 * kk + 2 * t) * 2;
                xb[mb][0] = *reinterpret_cast<const uint32_t*>(p);
                xb[mb][1] = *reinterpret_cast<const uint32_t*>(p + 16);
            }
            const int row = 16 * kk + lm_row;
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
                for (int ng = 0; ng < 2; ng++) {
                    const int c16 = warp * 4 + ng * 2 + lm_col16;
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, sbase + w * kStageBytes + row * (kBN * 2) + ((c16 ^ (row & 7)) << 4));
                    // ldmatrix order is (n 0-7, k 0-7), (n 8-15, k 0-7), (n 0-7, k 8-15), (n 8-15, k 8-15)
                    // = a0, a1, a2, a3 of the mma "row" operand
#pragma unroll
                    for (int mb = 0; mb < MB; mb++) mma16816(acc[w][ng][mb], a, xb[mb][0], xb[mb][1]);
                }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    __syncthreads();

    // this block's partial tile, then the cluster-wide sum in rank order
    float* red = reinterpret_cast<float*>(smem);  // [NW][MP][kRedLd]
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int ng = 0; ng < 2; ng++)
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int tok = 8 * mb + 2 * t + (e & 1);
                    const int c = warp * 32 + ng * 16 + g + ((e & 2) ? 8 : 0);
                    red[(w * MP + tok) * kRedLd + c] = acc[w][ng][mb][e];
                }
    cluster.sync();
    const int per_rank = (MP * kBN + KS - 1) / KS;
    const int e_begin = rank * per_rank, e_end = min(e_begin + per_rank, MP * kBN);
    for (int e = e_begin + tid; e < e_end; e += kStThreads) {
        const int tok = e / kBN, c = e % kBN;
        float s0 = 0.f, s1 = 0.f;
        for (int r = 0; r < KS; r++) {
            const float* peer = cluster.map_shared_rank(red, r);
            s0 += peer[tok * kRedLd + c];
            if (DUAL) s1 += peer[(MP + tok) * kRedLd + c];
        }
        if (tok < M && n0 + c < N) {
            const float v = DUAL ? (s0 / (1.0f + __expf(-s0))) * s1 : s0;
            y[(size_t)tok * N + n0 + c] = __float2half_rn(v);
        }
    }
    cluster.sync();  // peers may still be reading this block's tile
}

// Resident blocks of `kern` for a cluster size and ring depth (cached).
template <typename Kern>
static int staged_slots(Kern kern, int ks, int nst, size_t smem, int col_blocks)
{
    // one table for every instantiation (they share the function-pointer type): the kernel is
    // part of the key
    static std::map<std::tuple<const void*, int, int>, int> cache;
    const auto key = std::make_tuple((const void*)kern, ks, nst);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
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
    cache[key] = clusters * ks;
    return clusters * ks;
}

template <int MB, bool DUAL>
static cudaError_t launch_staged(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N, int K,
                                 cudaStream_t st)
{
    auto kern = skinny_kn_staged_kernel<MB, DUAL>;
    constexpr int NW = DUAL ? 2 : 1;
    constexpr size_t stage = (size_t)NW * kStageBytes + 8 * MB * kXRowBytes;
    constexpr size_t red = (size_t)NW * 8 * MB * kRedLd * sizeof(float);
    constexpr size_t smem_cap = 226 * 1024;
    static bool attr_set = false;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int col_blocks = (N + kBN - 1) / kBN;
    const int total_stages = (K + kKC - 1) / kKC;
    auto smem_for = [&](int nst) { return std::max(stage * nst, red); };
    // Plan.  Measured on B200 with a copy-only version of this tiling: about 1.7 blocks per SM
    // (256 blocks) with a ring of 8 stages already streams at the ceiling of the staged path;
    // more, smaller blocks are slower (each pays its own pipeline fill and reduction), fewer
    // blocks need deeper rings.  So: split K so that the grid lands near 1.75 blocks per SM,
    // keep every block resident (one wave), and give each ring what shared memory allows.
    const int target_blocks = num_sms() * 7 / 4;
    int best_ks = 1;
    {
        double best_d = 1e30;
        for (int ks = 1; ks <= 8; ks++) {
            const int per = (total_stages + ks - 1) / ks;
            if (ks > 1 && per < 4) break;
            const double d = fabs(log((double)col_blocks * ks / (double)target_blocks));
            if (d < best_d) {
                best_d = d;
                best_ks = ks;
            }
        }
    }
    const int per_block = (total_stages + best_ks - 1) / best_ks;
    const long total = (long)col_blocks * best_ks;
    int best_nst = std::min(12, std::max(3, per_block + 1));
    best_nst = std::min<int>(best_nst, (int)(smem_cap / stage));
    while (best_nst > 3 && staged_slots(kern, best_ks, best_nst, smem_for(best_nst), col_blocks) < total) best_nst--;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = best_ks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(col_blocks, best_ks, 1);
    cfg.blockDim = dim3(kStThreads);
    cfg.dynamicSmemBytes = smem_for(best_nst);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kern, x, W0, W1, y, M, N, K, (total_stages + best_ks - 1) / best_ks, best_nst);
}

// One pass of at most 64 tokens.  Called from skinny_gemm.cu.
cudaError_t skinny_kn_staged_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                      int K, bool dual, cudaStream_t st)
{
    if (dual) {
        if (M <= 8) return launch_staged<1, true>(x, W0, W1, y, M, N, K, st);
        if (M <= 16) return launch_staged<2, true>(x, W0, W1, y, M, N, K, st);
        if (M <= 32) return launch_staged<4, true>(x, W0, W1, y, M, N, K, st);
        return launch_staged<8, true>(x, W0, W1, y, M, N, K, st);
    }
    if (M <= 8) return launch_staged<1, false>(x, W0, nullptr, y, M, N, K, st);
    if (M <= 16) return launch_staged<2, false>(x, W0, nullptr, y, M, N, K, st);
    if (M <= 32) return launch_staged<4, false>(x, W0, nullptr, y, M, N, K, st);
    return launch_staged<8, false>(x, W0, nullptr, y, M, N, K, st);
}

}  // namespace onellm
