// Decode-time projections (M <= 64 tokens) for sm_100a: weight-streaming, HBM-bound.
//
// Replaces the cuBLAS calls behind launchLinearGemm (src/kernels/qkv_linear.cu:8-65,
// src/kernels/cublas_wrapper.cc:45-90) for the shapes of a decode step, and fuses the SwiGLU
// of src/kernels/activation_kernel.cu:10-21 into the gate/up projection.
//
// At M <= 64 every weight is used for a handful of FMAs, so the kernel is judged on bytes per
// second.  The weight matrix is read exactly once, straight from global memory into
// registers with 16-byte loads, in the layout it has on disk and in the reference's weight
// structs ([K, N], N contiguous); nothing is staged in shared memory.  The arithmetic runs on
// the tensor cores as mma.m16n8k16 with the WEIGHT as the 16-row operand and the 8 tokens of a
// batch block as the 8-column operand, so a batch of 8 wastes nothing.  Because a sum over k
// does not care about the order of k, each lane may feed the k slots of its fragment from
// whichever rows it loaded: lane (g, t) loads rows kb+4t .. kb+4t+3 at columns n0+8g .. +7 and
// pairs halves of two rows with one byte-permute per register.  The activations are the
// small operand and come through L1 as 8-byte loads.
//
// K is split over the warps of a block and over the blocks of a thread-block cluster; the
// partial sums meet in distributed shared memory (no global scratch, no atomics, a fixed
// summation order, so results are bitwise reproducible).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace onellm {

constexpr int kSkinnyThreads = 128;  // 4 warps
constexpr int kColsPerBlock = 64;
constexpr int kRedStride = 65;       // floats per row of the reduction tile

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// y[M,N] = x[M,K] . W[K,N]            (DUAL = false)
// y[M,N] = silu(x.W0) * (x.W1)        (DUAL = true)
// grid = (ceil(N/64), KS), cluster = (1, KS, 1); M <= 8*MB.
template <int MB, bool DUAL, int UK>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_kn_kernel(const __half* __restrict__ x, const __half* __restrict__ W0, const __half* __restrict__ W1,
                 __half* __restrict__ y, int M, int N, int K, int ksteps_per_block)
{
    constexpr int NW = DUAL ? 2 : 1;
    constexpr int MP = 8 * MB;  // padded token count
    cg::cluster_group cluster = cg::this_cluster();
    const int KS = gridDim.y;
    const int rank = blockIdx.y;
    const int n0 = blockIdx.x * kColsPerBlock;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int col = n0 + 8 * g;
    const bool col_ok = col < N;  // N is a multiple of 8
    const int total_ksteps = K / 16;
    const int ks_begin = rank * ksteps_per_block;
    const int ks_end = min(ks_begin + ksteps_per_block, total_ksteps);

    float acc[NW][MB][4][4];
#pragma unroll
    for (int w = 0; w < NW; w++)
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[w][mb][i][e] = 0.f;

    const __half* xrow[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++) xrow[mb] = x + (size_t)min(8 * mb + g, M - 1) * K + 4 * t;
    const __half* wbase[NW];
    wbase[0] = W0 + (size_t)(4 * t) * N + col;
    if (DUAL) wbase[NW - 1] = W1 + (size_t)(4 * t) * N + col;

    for (int ks = ks_begin + warp; ks < ks_end; ks += 4 * UK) {
        uint4 wr[NW][UK][4];
        uint2 xb[UK][MB];
#pragma unroll
        for (int u = 0; u < UK; u++) {
            const int ksu = ks + 4 * u;
            const bool ok = ksu < ks_end;
            const size_t kb = (size_t)ksu * 16;
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    wr[w][u][j] = (ok && col_ok) ? ld_nc_16(wbase[w] + (kb + j) * N) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
                xb[u][mb] = ok ? __ldg(reinterpret_cast<const uint2*>(xrow[mb] + kb)) : make_uint2(0, 0);
        }
#pragma unroll
        for (int u = 0; u < UK; u++)
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                    const uint32_t lo0 = (i < 2) ? wr[w][u][0].x : wr[w][u][0].y;
                    const uint32_t lo1 = (i < 2) ? wr[w][u][1].x : wr[w][u][1].y;
                    const uint32_t lo2 = (i < 2) ? wr[w][u][2].x : wr[w][u][2].y;
                    const uint32_t lo3 = (i < 2) ? wr[w][u][3].x : wr[w][u][3].y;
                    const uint32_t hi0 = (i < 2) ? wr[w][u][0].z : wr[w][u][0].w;
                    const uint32_t hi1 = (i < 2) ? wr[w][u][1].z : wr[w][u][1].w;
                    const uint32_t hi2 = (i < 2) ? wr[w][u][2].z : wr[w][u][2].w;
                    const uint32_t hi3 = (i < 2) ? wr[w][u][3].z : wr[w][u][3].w;
                    const uint32_t a0 = __byte_perm(lo0, lo1, sel);  // column 8g+i,   k slots 2t, 2t+1
                    const uint32_t a2 = __byte_perm(lo2, lo3, sel);  // column 8g+i,   k slots 2t+8, 2t+9
                    const uint32_t a1 = __byte_perm(hi0, hi1, sel);  // column 8g+4+i, k slots 2t, 2t+1
                    const uint32_t a3 = __byte_perm(hi2, hi3, sel);  // column 8g+4+i, k slots 2t+8, 2t+9
#pragma unroll
                    for (int mb = 0; mb < MB; mb++) mma_16816(acc[w][mb][i], a0, a1, a2, a3, xb[u][mb].x, xb[u][mb].y);
                }
    }

    // reduce the four warps into this block's tile: red[w][token][column]
    extern __shared__ float red[];  // NW * MP * kRedStride floats
    for (int wsel = 0; wsel < 4; wsel++) {
        if (warp == wsel) {
#pragma unroll
            for (int w = 0; w < NW; w++)
#pragma unroll
                for (int mb = 0; mb < MB; mb++)
#pragma unroll
                    for (int i = 0; i < 4; i++)
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int tok = 8 * mb + 2 * t + (e & 1);
                            const int c = 8 * g + i + ((e & 2) ? 4 : 0);
                            float* dst = &red[(w * MP + tok) * kRedStride + c];
                            *dst = (wsel == 0) ? acc[w][mb][i][e] : *dst + acc[w][mb][i][e];
                        }
        }
        __syncthreads();
    }
    cluster.sync();

    // every block of the cluster finishes a slice of the tile, summing ranks in order
    const int per_rank = (MP * kColsPerBlock + KS - 1) / KS;
    const int e_begin = rank * per_rank;
    const int e_end = min(e_begin + per_rank, MP * kColsPerBlock);
    for (int e = e_begin + threadIdx.x; e < e_end; e += kSkinnyThreads) {
        const int tok = e / kColsPerBlock, c = e % kColsPerBlock;
        float s0 = 0.f, s1 = 0.f;
        for (int r = 0; r < KS; r++) {
            const float* peer = cluster.map_shared_rank(red, r);
            s0 += peer[tok * kRedStride + c];
            if (DUAL) s1 += peer[(MP + tok) * kRedStride + c];
        }
        if (tok < M && n0 + c < N) {
            const float v = DUAL ? silu_f(s0) * s1 : s0;
            y[(size_t)tok * N + n0 + c] = __float2half_rn(v);
        }
    }
    cluster.sync();  // peers may still be reading this block's tile
}

// y[M,N] = x[M,K] . W^T with W [N, K] (K contiguous): the LM head.  Each warp owns 16 rows of W
// and streams them contiguously, 64 bytes per row per load instruction; no byte-permutes are
// needed because consecutive k are already adjacent.  grid = (ceil(N/64)), 4 warps x 16 rows.
template <int MB, int UK>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_nk_kernel(const __half* __restrict__ x, const __half* __restrict__ W, __half* __restrict__ y, int M, int N,
                 int K)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 64 + warp * 16;  // first W row of this warp
    if (r0 >= N) return;
    const int ra = min(r0 + g, N - 1), rb = min(r0 + g + 8, N - 1);
    const __half* wa = W + (size_t)ra * K + 8 * t;
    const __half* wb = W + (size_t)rb * K + 8 * t;
    const __half* xrow[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++) xrow[mb] = x + (size_t)min(8 * mb + g, M - 1) * K + 8 * t;

    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[mb][e] = 0.f;

    const int total = K / 32;  // 32 k per step: lane t covers k 8t .. 8t+7
    for (int ks = 0; ks < total; ks += UK) {
        uint4 a[UK], b[UK], xv[UK][MB];
#pragma unroll
        for (int u = 0; u < UK; u++) {
            const bool ok = ks + u < total;
            const size_t kb = (size_t)(ks + u) * 32;
            a[u] = ok ? ld_nc_16(wa + kb) : make_uint4(0, 0, 0, 0);
            b[u] = ok ? ld_nc_16(wb + kb) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
                xv[u][mb] = ok ? __ldg(reinterpret_cast<const uint4*>(xrow[mb] + kb)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UK; u++)
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                mma_16816(acc[mb], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][mb].x, xv[u][mb].y);
                mma_16816(acc[mb], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][mb].z, xv[u][mb].w);
            }
    }
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int tok = 8 * mb + 2 * t + (e & 1);
            const int n = r0 + g + ((e & 2) ? 8 : 0);
            if (tok < M && n < N) y[(size_t)tok * N + n] = __float2half_rn(acc[mb][e]);
        }
}

// Plain fp32 projection for the reference's own dtype: 64x64 tiles, 16x16 threads, 4x4 outputs
// per thread.  Correctness path for fp32 callers, not a tuned kernel.
template <bool W_NK>
__global__ void __launch_bounds__(256)
sgemm_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ y, int M, int N, int K)
{
    __shared__ float xs[16][64 + 1];
    __shared__ float ws[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            const int kk = i & 15, mm = i >> 4;
            xs[kk][mm] = (m0 + mm < M && k0 + kk < K) ? x[(size_t)(m0 + mm) * K + k0 + kk] : 0.f;
        }
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            if (W_NK) {
                const int kk = i & 15, nn = i >> 4;
                ws[kk][nn] = (n0 + nn < N && k0 + kk < K) ? W[(size_t)(n0 + nn) * K + k0 + kk] : 0.f;
            } else {
                const int nn = i & 63, kk = i >> 6;
                ws[kk][nn] = (n0 + nn < N && k0 + kk < K) ? W[(size_t)(k0 + kk) * N + n0 + nn] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) y[(size_t)m * N + n] = acc[i][j];
        }
}

static int pick_ksplit(int N, int K)
{
    const int col_blocks = (N + kColsPerBlock - 1) / kColsPerBlock;
    const int target = num_sms() * 4;
    int ks = 1;
    while (ks < 8 && col_blocks * ks < target && K / (ks * 2) >= 4 * 16 * 2) ks *= 2;
    return ks;
}

template <int MB, bool DUAL, int UK>
static cudaError_t launch_skinny_kn(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                    int K, cudaStream_t st)
{
    const int KS = pick_ksplit(N, K);
    const int total_ksteps = K / 16;
    const int per_block = (total_ksteps + KS - 1) / KS;
    const size_t smem = (size_t)(DUAL ? 2 : 1) * 8 * MB * kRedStride * sizeof(float);
    auto kern = skinny_kn_kernel<MB, DUAL, UK>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + kColsPerBlock - 1) / kColsPerBlock, KS, 1);
    cfg.blockDim = dim3(kSkinnyThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = KS;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, x, W0, W1, y, M, N, K, per_block);
}

// one pass of at most 64 tokens
static cudaError_t skinny_kn_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                      int K, bool dual, cudaStream_t st)
{
    if (dual) {
        if (M <= 8) return launch_skinny_kn<1, true, 2>(x, W0, W1, y, M, N, K, st);
        if (M <= 16) return launch_skinny_kn<2, true, 2>(x, W0, W1, y, M, N, K, st);
        return launch_skinny_kn<4, true, 1>(x, W0, W1, y, M, N, K, st);
    }
    if (M <= 8) return launch_skinny_kn<1, false, 4>(x, W0, nullptr, y, M, N, K, st);
    if (M <= 16) return launch_skinny_kn<2, false, 4>(x, W0, nullptr, y, M, N, K, st);
    if (M <= 32) return launch_skinny_kn<4, false, 2>(x, W0, nullptr, y, M, N, K, st);
    return launch_skinny_kn<8, false, 2>(x, W0, nullptr, y, M, N, K, st);
}

static void skinny_nk_dispatch(const __half* x, const __half* W, __half* y, int M, int N, int K, cudaStream_t st)
{
    const dim3 grid((N + 63) / 64), block(kSkinnyThreads);
    if (M <= 8) skinny_nk_kernel<1, 4><<<grid, block, 0, st>>>(x, W, y, M, N, K);
    else if (M <= 16) skinny_nk_kernel<2, 4><<<grid, block, 0, st>>>(x, W, y, M, N, K);
    else if (M <= 32) skinny_nk_kernel<4, 2><<<grid, block, 0, st>>>(x, W, y, M, N, K);
    else skinny_nk_kernel<8, 2><<<grid, block, 0, st>>>(x, W, y, M, N, K);
}

// Defined in gemm_tc.cu: the tiled tensor-core path for M > 64.
int gemm_f16_large(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout,
                   cudaStream_t st);

int gemm_f16_skinny(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout,
                    cudaStream_t st)
{
    if (w_layout == ONELLM_W_KN) {
        ONELLM_REQUIRE(K % 16 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED,
                       "gemm: [K,N] weights need K %% 16 == 0 and N %% 8 == 0 (K=%d N=%d)", K, N);
        ONELLM_CUDA(skinny_kn_dispatch(x, W, nullptr, y, M, N, K, false, st));
    } else {
        ONELLM_REQUIRE(K % 32 == 0, ONELLM_ERR_UNSUPPORTED, "gemm: [N,K] weights need K %% 32 == 0 (K=%d)", K);
        skinny_nk_dispatch(x, W, y, M, N, K, st);
        ONELLM_CHECK_LAUNCH();
    }
    return ONELLM_OK;
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_gemm(int dtype, const void* x, const void* W, void* y, int M, int N, int K, int w_layout,
                           void* stream)
{
    ONELLM_REQUIRE(x && W && y, ONELLM_ERR_ARG, "gemm: null pointer");
    ONELLM_REQUIRE(M >= 0 && N > 0 && K > 0, ONELLM_ERR_ARG, "gemm: bad size M=%d N=%d K=%d", M, N, K);
    ONELLM_REQUIRE(w_layout == ONELLM_W_KN || w_layout == ONELLM_W_NK, ONELLM_ERR_ARG, "gemm: bad w_layout %d",
                   w_layout);
    if (M == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == ONELLM_F32) {
        const dim3 grid((N + 63) / 64, (M + 63) / 64);
        ONELLM_REQUIRE(grid.y <= 65535, ONELLM_ERR_UNSUPPORTED, "gemm: M too large for the fp32 path");
        if (w_layout == ONELLM_W_NK)
            sgemm_kernel<true><<<grid, 256, 0, st>>>((const float*)x, (const float*)W, (float*)y, M, N, K);
        else
            sgemm_kernel<false><<<grid, 256, 0, st>>>((const float*)x, (const float*)W, (float*)y, M, N, K);
        ONELLM_CHECK_LAUNCH();
        return ONELLM_OK;
    }
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm: dtype %d", dtype);
    ONELLM_REQUIRE(aligned16(x) && aligned16(W) && aligned16(y), ONELLM_ERR_ARG,
                   "gemm: pointers must be 16-byte aligned");
    const __half* xh = (const __half*)x;
    const __half* Wh = (const __half*)W;
    __half* yh = (__half*)y;
    if (M > 64) return gemm_f16_large(xh, Wh, yh, M, N, K, w_layout, st);
    return gemm_f16_skinny(xh, Wh, yh, M, N, K, w_layout, st);
}

extern "C" int onellm_gemm_swiglu(int dtype, const void* x, const void* Wg, const void* Wu, void* out, int M,
                                  int I, int K, void* stream)
{
    ONELLM_REQUIRE(x && Wg && Wu && out, ONELLM_ERR_ARG, "gemm_swiglu: null pointer");
    ONELLM_REQUIRE(M >= 0 && I > 0 && K > 0, ONELLM_ERR_ARG, "gemm_swiglu: bad size");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm_swiglu: only F16 is implemented");
    ONELLM_REQUIRE(M <= 32, ONELLM_ERR_UNSUPPORTED,
                   "gemm_swiglu: fused path covers M <= 32; use two projections and onellm_swiglu");
    ONELLM_REQUIRE(K % 16 == 0 && I % 8 == 0, ONELLM_ERR_UNSUPPORTED, "gemm_swiglu: need K %% 16 == 0, I %% 8 == 0");
    ONELLM_REQUIRE(aligned16(x) && aligned16(Wg) && aligned16(Wu) && aligned16(out), ONELLM_ERR_ARG,
                   "gemm_swiglu: pointers must be 16-byte aligned");
    if (M == 0) return ONELLM_OK;
    ONELLM_CUDA(skinny_kn_dispatch((const __half*)x, (const __half*)Wg, (const __half*)Wu, (__half*)out, M, I, K,
                                   true, reinterpret_cast<cudaStream_t>(stream)));
    return ONELLM_OK;
}
