// RMSNorm and fused add-bias-residual RMSNorm for sm_100a: HBM-bound, one pass over the data.
//
// Replaces RMSNorm (src/kernels/rmsnorm_kernel.cu:47-83) and FusedAddBiasResidualRMSNorm
// (src/kernels/fused_addresidual_norm.cu:51-107) of the reference.
//
// One thread block per token row, a fixed 256 threads whatever the hidden size (the
// reference sizes the block as hidden/4, which stops launching beyond hidden 4096).  Each
// thread owns up to kMaxVec 16-byte vectors of the row and keeps them in registers between
// the sum-of-squares reduction and the scaling, so a row is read once and written once.
// Rows too long for the register budget are re-read from L2 in the second phase.
#include "common.cuh"

namespace onellm {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;

__device__ __forceinline__ float block_sum_256(float v)
{
    __shared__ float part[kNormThreads / 32];
    __shared__ float total;
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < kNormThreads / 32 ? part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) total = t;
    }
    __syncthreads();
    return total;
}

// FUSED = false: x <- gamma * x * rsqrt(mean(x^2)+eps)
// FUSED = true : r <- x + r + bias; x <- gamma * r * rsqrt(mean(r^2)+eps)
template <typename T, bool FUSED, bool IN_REGS>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ bias,
               const T* __restrict__ gamma, float eps, int hidden)
{
    constexpr int VEC = Vec16<T>::N;
    const int nvec = hidden / VEC;
    pdl_launch_dependents();
    pdl_wait();
    T* xr = x + (size_t)blockIdx.x * hidden;
    T* rr = FUSED ? residual + (size_t)blockIdx.x * hidden : nullptr;

    float keep[IN_REGS ? kMaxVec : 1][VEC];
    float ss = 0.f;
    // loads vector i of the row (adding residual and bias and storing the sum when FUSED)
    auto fetch = [&](int i, float (&f)[VEC]) {
        Vec16<T>::load(xr + (size_t)i * VEC, f);
        if (FUSED) {
            float r[VEC];
            Vec16<T>::load(rr + (size_t)i * VEC, r);
#pragma unroll
            for (int e = 0; e < VEC; e++) f[e] += r[e];
            if (bias) {
                float bb[VEC];
                Vec16<T>::load(bias + (size_t)i * VEC, bb);
#pragma unroll
                for (int e = 0; e < VEC; e++) f[e] += bb[e];
            }
            *reinterpret_cast<uint4*>(rr + (size_t)i * VEC) = Vec16<T>::pack(f);
        }
#pragma unroll
        for (int e = 0; e < VEC; e++) ss = fmaf(f[e], f[e], ss);
    };
    if (IN_REGS) {
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * kNormThreads;
            if (i < nvec) fetch(i, keep[j]);
        }
    } else {
        for (int i = threadIdx.x; i < nvec; i += kNormThreads) {
            float f[VEC];
            fetch(i, f);
        }
    }
    const float inv = rsqrtf(block_sum_256(ss) / (float)hidden + eps);

    if (IN_REGS) {
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * kNormThreads;
            if (i < nvec) {
                float g[VEC], o[VEC];
                Vec16<T>::load(gamma + (size_t)i * VEC, g);
#pragma unroll
                for (int e = 0; e < VEC; e++) o[e] = g[e] * keep[j][e] * inv;
                *reinterpret_cast<uint4*>(xr + (size_t)i * VEC) = Vec16<T>::pack(o);
            }
        }
    } else {
        // long rows: the summed row was just written (FUSED) or is still in L2
        const T* src = FUSED ? rr : xr;
        for (int i = threadIdx.x; i < nvec; i += kNormThreads) {
            float f[VEC], g[VEC], o[VEC];
            Vec16<T>::load(src + (size_t)i * VEC, f);
            Vec16<T>::load(gamma + (size_t)i * VEC, g);
#pragma unroll
            for (int e = 0; e < VEC; e++) o[e] = g[e] * f[e] * inv;
            *reinterpret_cast<uint4*>(xr + (size_t)i * VEC) = Vec16<T>::pack(o);
        }
    }
}

template <typename T, bool FUSED>
static void launch_norm(void* x, void* residual, const void* bias, const void* gamma, float eps,
                        int num_tokens, int hidden, cudaStream_t st)
{
    const int nvec = hidden / Vec16<T>::N;
    if (nvec <= kNormThreads * kMaxVec)
        (void)launch_pdl(rmsnorm_kernel<T, FUSED, true>, dim3(num_tokens), dim3(kNormThreads), 0, st, (T*)x, (T*)residual,
                         (const T*)bias, (const T*)gamma, eps, hidden);
    else
        (void)launch_pdl(rmsnorm_kernel<T, FUSED, false>, dim3(num_tokens), dim3(kNormThreads), 0, st, (T*)x,
                         (T*)residual, (const T*)bias, (const T*)gamma, eps, hidden);
}

static int check_norm_args(const char* who, int dtype, const void* x, const void* gamma, int num_tokens,
                           int hidden)
{
    ONELLM_REQUIRE(x && gamma, ONELLM_ERR_ARG, "%s: null pointer", who);
    ONELLM_REQUIRE(num_tokens >= 0 && hidden > 0, ONELLM_ERR_ARG, "%s: bad size", who);
    const size_t es = dtype_size(dtype);
    ONELLM_REQUIRE(es != 0, ONELLM_ERR_UNSUPPORTED, "%s: dtype %d", who, dtype);
    ONELLM_REQUIRE(((size_t)hidden * es) % 16 == 0, ONELLM_ERR_UNSUPPORTED,
                   "%s: hidden=%d rows are not a multiple of 16 bytes", who, hidden);
    ONELLM_REQUIRE(aligned16(x) && aligned16(gamma), ONELLM_ERR_ARG, "%s: pointers must be 16-byte aligned",
                   who);
    return ONELLM_OK;
}

}  // namespace onellm

using namespace onellm;

namespace onellm {
// out[row] = sum of squares of the fp16 row: the row statistics the norm-free context-phase projections take as an
// input (one warp per row)
__global__ void __launch_bounds__(256) row_sumsq_kernel(const __half* __restrict__ x, float* __restrict__ out, int rows, int cols)
{
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const __half* xr = x + (size_t)row * cols;
    float s = 0.f;
    for (int i = lane; i < cols / 8; i += 32) {
        float v[8];
        Vec16<__half>::load(xr + (size_t)i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; e++) s = fmaf(v[e], v[e], s);
    }
    s = warp_sum(s);
    if (lane == 0) out[row] = s;
}
}  // namespace onellm

extern "C" int onellm_row_sumsq(int dtype, const void* x, int rows, int cols, float* out, void* stream)
{
    ONELLM_REQUIRE(x && out, ONELLM_ERR_ARG, "row_sumsq: null pointer");
    ONELLM_REQUIRE(dtype == ONELLM_F16, ONELLM_ERR_UNSUPPORTED, "row_sumsq: only F16 is implemented");
    ONELLM_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && aligned16(x), ONELLM_ERR_ARG, "row_sumsq: rows of whole 16-byte vectors");
    if (rows == 0) return ONELLM_OK;
    ONELLM_CUDA(launch_pdl(onellm::row_sumsq_kernel, dim3((rows + 7) / 8), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                           (const __half*)x, out, rows, cols));
    return ONELLM_OK;
}

extern "C" int onellm_rmsnorm(int dtype, void* x, const void* gamma, float eps, int num_tokens, int hidden,
                              void* stream)
{
    const int rc = check_norm_args("rmsnorm", dtype, x, gamma, num_tokens, hidden);
    if (rc) return rc;
    if (num_tokens == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == ONELLM_F16)
        launch_norm<__half, false>(x, nullptr, nullptr, gamma, eps, num_tokens, hidden, st);
    else
        launch_norm<float, false>(x, nullptr, nullptr, gamma, eps, num_tokens, hidden, st);
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

extern "C" int onellm_add_residual_rmsnorm(int dtype, void* residual, void* decoder_out, const void* bias,
                                           const void* gamma, float eps, int num_tokens, int hidden,
                                           void* stream)
{
    const int rc = check_norm_args("add_residual_rmsnorm", dtype, decoder_out, gamma, num_tokens, hidden);
    if (rc) return rc;
    ONELLM_REQUIRE(residual && aligned16(residual) && (!bias || aligned16(bias)), ONELLM_ERR_ARG,
                   "add_residual_rmsnorm: residual missing or misaligned pointer");
    if (num_tokens == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == ONELLM_F16)
        launch_norm<__half, true>(decoder_out, residual, bias, gamma, eps, num_tokens, hidden, st);
    else
        launch_norm<float, true>(decoder_out, residual, bias, gamma, eps, num_tokens, hidden, st);
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}
