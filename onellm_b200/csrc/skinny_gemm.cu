// Projection entry points (onellm_gemm, onellm_gemm_swiglu) and two of their kernels:
//   - the LM head at decode time, y = x . W^T with W [N, K] (vocab rows, K contiguous), M <= 64;
//   - a plain fp32 GEMM for callers that keep the reference's fp32 tensors.
// The [K, N] weight-streaming kernel is in skinny_gemm_staged.cu, the tiled kernel for M > 64 in
// gemm_tc.cu.  Replaces launchLinearGemm / cublasWrapper::Gemm (src/kernels/qkv_linear.cu:8-65,
// src/kernels/cublas_wrapper.cc:45-90 of the reference).

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace onellm {

constexpr int kSkinnyThreads = 128;  // 4 warps

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// y[M,N] = x[M,K] . W^T with W [N, K] (K contiguous): the LM head.  Each warp owns 16 rows of W
// and streams them contiguously, 64 bytes per row per load instruction; no byte-permutes are
// needed because consecutive k are already adjacent.  Warps are independent, so the block size
// (1, 2 or 4 warps of 16 rows) is picked per launch to fill whole waves.
template <int MB, int UK>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_nk_kernel(const __half* __restrict__ x, const __half* __restrict__ W, __half* __restrict__ y, int M, int N,
                 int K)
{
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = (blockIdx.x * (blockDim.x >> 5) + warp) * 16;  // first W row of this warp
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
sgemm_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ y, int M, int N, int K, long ldy)
{
    __shared__ float xs[16][64 + 1];
    __shared__ float ws[16][64 + 1];
    pdl_wait();
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
            if (m < M && n < N) y[(size_t)m * ldy + n] = acc[i][j];
        }
}

// skinny_gemm_staged.cu
cudaError_t skinny_kn_staged_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                      int K, bool dual, cudaStream_t st, const __half* resid, const __half* bias,
                                      float rms_eps, const TpEpilogue* tp);

static cudaError_t skinny_kn_dispatch(const __half* x, const __half* W0, const __half* W1, __half* y, int M, int N,
                                      int K, bool dual, cudaStream_t st)
{
    return skinny_kn_staged_dispatch(x, W0, W1, y, M, N, K, dual, st, nullptr, nullptr, -1.f, nullptr);
}

template <int MB, int UK>
static void launch_skinny_nk(const __half* x, const __half* W, __half* y, int M, int N, int K, cudaStream_t st)
{
    auto kern = skinny_nk_kernel<MB, UK>;
    static int best_warps[3] = {0, 0, 0};  // residency per block size, queried once
    static std::mutex mu;
    int per_sm[3];
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < 3; i++) {
            if (best_warps[i] == 0) {
                int n = 0;
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 32 << i, 0) != cudaSuccess || n < 1) {
                    (void)cudaGetLastError();
                    n = 4;
                }
                best_warps[i] = n;
            }
            per_sm[i] = best_warps[i];
        }
    }
    const int tasks = (N + 15) / 16;  // one warp each
    int pick = 2;
    double best = -1.0;
    for (int i = 0; i < 3; i++) {
        const int warps = 1 << i;
        const long blocks = (tasks + warps - 1) / warps;
        const long slots = (long)per_sm[i] * num_sms();
        const long waves = (blocks + slots - 1) / slots;
        const double eff = (double)blocks / (double)(waves * slots) + 0.01 * i;  // ties: larger blocks
        if (eff > best) {
            best = eff;
            pick = i;
        }
    }
    const int warps = 1 << pick;
    (void)launch_pdl(kern, dim3((tasks + warps - 1) / warps), dim3(32 * warps), 0, st, x, W, y, M, N, K);
}

static void skinny_nk_dispatch(const __half* x, const __half* W, __half* y, int M, int N, int K, cudaStream_t st)
{
    if (M <= 8) launch_skinny_nk<1, 4>(x, W, y, M, N, K, st);
    else if (M <= 16) launch_skinny_nk<2, 4>(x, W, y, M, N, K, st);
    else if (M <= 32) launch_skinny_nk<4, 2>(x, W, y, M, N, K, st);
    else launch_skinny_nk<8, 2>(x, W, y, M, N, K, st);
}

// Defined in gemm_tc.cu: the tiled tensor-core path for M > 64.
int gemm_swiglu_f16_large(const __half* x, const __half* Wg, const __half* Wu, __half* out, int M, int I, int K, cudaStream_t st);
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

extern "C" int onellm_gemm_ld(int dtype, const void* x, const void* W, void* y, long ldy, int M, int N, int K, int w_layout,
                              void* stream)
{
    ONELLM_REQUIRE(x && W && y, ONELLM_ERR_ARG, "gemm: null pointer");
    ONELLM_REQUIRE(M >= 0 && N > 0 && K > 0 && ldy >= N, ONELLM_ERR_ARG, "gemm: bad size M=%d N=%d K=%d ldy=%ld", M, N, K, ldy);
    ONELLM_REQUIRE(w_layout == ONELLM_W_KN || w_layout == ONELLM_W_NK, ONELLM_ERR_ARG, "gemm: bad w_layout %d",
                   w_layout);
    if (M == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == ONELLM_F32) {
        const dim3 grid((N + 63) / 64, (M + 63) / 64);
        ONELLM_REQUIRE(grid.y <= 65535, ONELLM_ERR_UNSUPPORTED, "gemm: M too large for the fp32 path");
        note_launch();
        if (w_layout == ONELLM_W_NK)
            sgemm_kernel<true><<<grid, 256, 0, st>>>((const float*)x, (const float*)W, (float*)y, M, N, K, ldy);
        else
            sgemm_kernel<false><<<grid, 256, 0, st>>>((const float*)x, (const float*)W, (float*)y, M, N, K, ldy);
        ONELLM_CHECK_LAUNCH();
        return ONELLM_OK;
    }
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm: dtype %d", dtype);
    ONELLM_REQUIRE(ldy == N, ONELLM_ERR_UNSUPPORTED, "gemm: the F16 kernels write dense rows (ldy must equal N)");
    ONELLM_REQUIRE(aligned16(x) && aligned16(W) && aligned16(y), ONELLM_ERR_ARG,
                   "gemm: pointers must be 16-byte aligned");
    const __half* xh = (const __half*)x;
    const __half* Wh = (const __half*)W;
    __half* yh = (__half*)y;
    if (M > 64) return gemm_f16_large(xh, Wh, yh, M, N, K, w_layout, st);
    return gemm_f16_skinny(xh, Wh, yh, M, N, K, w_layout, st);
}

extern "C" int onellm_gemm(int dtype, const void* x, const void* W, void* y, int M, int N, int K, int w_layout,
                           void* stream)
{
    return onellm_gemm_ld(dtype, x, W, y, N, M, N, K, w_layout, stream);
}

namespace onellm {
cudaError_t staged_plan_query(int M, int N, int K, bool dual, int* ks, int* nst, int* blocks);
void staged_plan_override(int N, int K, bool dual, int ks, int nst);
}  // namespace onellm

extern "C" int onellm_gemm_plan_query(int M, int N, int K, int dual, int* k_split, int* ring_depth, int* blocks)
{
    ONELLM_REQUIRE(M >= 1 && M <= 64 && N > 0 && K > 0 && K % 16 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED,
                   "gemm_plan_query: covers the fp16 projections of at most 64 tokens with [K, N] weights");
    ONELLM_CUDA(staged_plan_query(M, N, K, dual != 0, k_split, ring_depth, blocks));
    return ONELLM_OK;
}

extern "C" int onellm_gemm_plan_override(int N, int K, int dual, int k_split, int ring_depth)
{
    ONELLM_REQUIRE(N > 0 && K > 0 && k_split <= 8 && (k_split <= 0 || ring_depth >= 3), ONELLM_ERR_ARG,
                   "gemm_plan_override: K split in 1..8 (0 removes the override), ring depth >= 3");
    staged_plan_override(N, K, dual != 0, k_split, ring_depth);
    return ONELLM_OK;
}

extern "C" int onellm_gemm_fused(int dtype, const void* x, const void* W, const void* Wu, void* y, int M, int N, int K,
                                 float rms_eps, const void* resid, const void* bias, void* stream)
{
    ONELLM_REQUIRE(x && W && y, ONELLM_ERR_ARG, "gemm_fused: null pointer");
    ONELLM_REQUIRE(M >= 0 && N > 0 && K > 0, ONELLM_ERR_ARG, "gemm_fused: bad size");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm_fused: only F16 is implemented");
    ONELLM_REQUIRE(M <= 64, ONELLM_ERR_UNSUPPORTED, "gemm_fused: covers M <= 64 tokens");
    ONELLM_REQUIRE(K % 16 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED, "gemm_fused: need K %% 16 == 0, N %% 8 == 0");
    ONELLM_REQUIRE(resid || !bias, ONELLM_ERR_ARG, "gemm_fused: bias is added with the residual; pass resid too");
    ONELLM_REQUIRE(aligned16(x) && aligned16(W) && aligned16(y) && (!Wu || aligned16(Wu)), ONELLM_ERR_ARG,
                   "gemm_fused: pointers must be 16-byte aligned");
    ONELLM_REQUIRE(x != y, ONELLM_ERR_ARG, "gemm_fused: y must not alias x");
    if (M == 0) return ONELLM_OK;
    ONELLM_CUDA(skinny_kn_staged_dispatch((const __half*)x, (const __half*)W, (const __half*)Wu, (__half*)y, M, N, K, Wu != nullptr,
                                          reinterpret_cast<cudaStream_t>(stream), (const __half*)resid, (const __half*)bias,
                                          rms_eps, nullptr));
    return ONELLM_OK;
}

namespace onellm {
int gemm_rows_parts(int N, bool dual);  // gemm_tc.cu
int gemm_rows_f16(const __half* x, const __half* W, const __half* W2, __half* y, int M, int N, int K, const float* row_ss, int ss_parts,
                  float eps, const __half* resid, const __half* bias, float* ss_out, cudaStream_t st);
}  // namespace onellm

extern "C" int onellm_gemm_rows_parts(int N, int dual) { return N > 0 ? onellm::gemm_rows_parts(N, dual != 0) : 0; }

extern "C" int onellm_gemm_rows(int dtype, const void* x, const void* W, const void* Wu, void* y, int M, int N, int K, const float* row_ss,
                                int ss_parts, float rms_eps, const void* resid, const void* bias, float* row_ss_out, void* stream)
{
    ONELLM_REQUIRE(x && W && y, ONELLM_ERR_ARG, "gemm_rows: null pointer");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm_rows: only F16 is implemented");
    ONELLM_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 8 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED, "gemm_rows: need K %% 8 == 0 and N %% 8 == 0");
    ONELLM_REQUIRE(!row_ss || ss_parts >= 1, ONELLM_ERR_ARG, "gemm_rows: row_ss needs its number of partial sums per row");
    ONELLM_REQUIRE(resid || !bias, ONELLM_ERR_ARG, "gemm_rows: bias is added with the residual; pass resid too");
    ONELLM_REQUIRE(!(Wu && (resid || row_ss_out)), ONELLM_ERR_UNSUPPORTED, "gemm_rows: the gate/up form takes neither resid nor row_ss_out");
    ONELLM_REQUIRE(aligned16(x) && aligned16(W) && aligned16(y) && (!Wu || aligned16(Wu)) && (!resid || aligned16(resid)) &&
                       (!bias || aligned16(bias)) && x != y,
                   ONELLM_ERR_ARG, "gemm_rows: pointers must be 16-byte aligned and y must not alias x");
    if (M == 0) return ONELLM_OK;
    return onellm::gemm_rows_f16((const __half*)x, (const __half*)W, (const __half*)Wu, (__half*)y, M, N, K, row_ss, ss_parts, rms_eps,
                                 (const __half*)resid, (const __half*)bias, row_ss_out, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int onellm_gemm_swiglu(int dtype, const void* x, const void* Wg, const void* Wu, void* out, int M,
                                  int I, int K, void* stream)
{
    ONELLM_REQUIRE(x && Wg && Wu && out, ONELLM_ERR_ARG, "gemm_swiglu: null pointer");
    ONELLM_REQUIRE(M >= 0 && I > 0 && K > 0, ONELLM_ERR_ARG, "gemm_swiglu: bad size");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "gemm_swiglu: only F16 is implemented");
    ONELLM_REQUIRE(K % 16 == 0 && I % 8 == 0, ONELLM_ERR_UNSUPPORTED, "gemm_swiglu: need K %% 16 == 0, I %% 8 == 0");
    ONELLM_REQUIRE(aligned16(x) && aligned16(Wg) && aligned16(Wu) && aligned16(out), ONELLM_ERR_ARG,
                   "gemm_swiglu: pointers must be 16-byte aligned");
    if (M == 0) return ONELLM_OK;
    if (M > 64)  // tensor-core tiles, SwiGLU in the epilogue
        return gemm_swiglu_f16_large((const __half*)x, (const __half*)Wg, (const __half*)Wu, (__half*)out, M, I, K,
                                     reinterpret_cast<cudaStream_t>(stream));
    ONELLM_CUDA(skinny_kn_dispatch((const __half*)x, (const __half*)Wg, (const __half*)Wu, (__half*)out, M, I, K,
                                   true, reinterpret_cast<cudaStream_t>(stream)));
    return ONELLM_OK;
}
