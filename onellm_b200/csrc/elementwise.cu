// Small HBM-bound kernels: SwiGLU on a packed [tokens, 2, I] buffer and the embedding gather.
//
// Replace silu_and_mul_kernel (src/kernels/activation_kernel.cu:10-21) and embeddingFunctor
// (src/kernels/input_embedding.cu:7-20) of the reference with 16-byte vectorised versions.
#include "common.cuh"

namespace onellm {

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, int inter)
{
    constexpr int VEC = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const T* gate = in + (size_t)blockIdx.y * 2 * inter;
    const T* up = gate + inter;
    T* o = out + (size_t)blockIdx.y * inter;
    const int nvec = inter / VEC;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gridDim.x * blockDim.x) {
        float g[VEC], u[VEC], r[VEC];
        Vec16<T>::load(gate + (size_t)i * VEC, g);
        Vec16<T>::load(up + (size_t)i * VEC, u);
#pragma unroll
        for (int e = 0; e < VEC; e++) r[e] = (g[e] / (1.0f + expf(-g[e]))) * u[e];
        *reinterpret_cast<uint4*>(o + (size_t)i * VEC) = Vec16<T>::pack(r);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
embedding_kernel(const int* __restrict__ ids, T* __restrict__ out, T* __restrict__ out2, const T* __restrict__ table,
                 int hidden, int vocab, int* __restrict__ bad_id_flag)
{
    constexpr int VEC = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && bad_id_flag && threadIdx.x == 0) atomicExch(bad_id_flag, 1);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * hidden);
    uint4* dst2 = out2 ? reinterpret_cast<uint4*>(out2 + (size_t)t * hidden) : nullptr;
    for (int i = threadIdx.x; i < hidden / VEC; i += blockDim.x) {
        const uint4 v = ok ? src[i] : make_uint4(0, 0, 0, 0);
        dst[i] = v;
        if (dst2) dst2[i] = v;
    }
}

}  // namespace onellm

using namespace onellm;

extern "C" int onellm_swiglu(int dtype, const void* input, void* out, int tokens, int inter, void* stream)
{
    ONELLM_REQUIRE(input && out, ONELLM_ERR_ARG, "swiglu: null pointer");
    ONELLM_REQUIRE(tokens >= 0 && inter > 0, ONELLM_ERR_ARG, "swiglu: bad size");
    const size_t es = dtype_size(dtype);
    ONELLM_REQUIRE(es != 0, ONELLM_ERR_UNSUPPORTED, "swiglu: dtype %d", dtype);
    ONELLM_REQUIRE(((size_t)inter * es) % 16 == 0 && aligned16(input) && aligned16(out), ONELLM_ERR_ARG,
                   "swiglu: rows must be 16-byte aligned");
    ONELLM_REQUIRE(tokens <= 65535, ONELLM_ERR_UNSUPPORTED, "swiglu: more than 65535 tokens per call");
    if (tokens == 0) return ONELLM_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int nvec = inter / (int)(16 / es);
    const dim3 grid((nvec + 255) / 256, tokens);
    note_launch();
    if (dtype == ONELLM_F16)
        swiglu_kernel<__half><<<grid, 256, 0, st>>>((const __half*)input, (__half*)out, inter);
    else
        swiglu_kernel<float><<<grid, 256, 0, st>>>((const float*)input, (float*)out, inter);
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}

namespace onellm {
// Shared by the C entry point and the model driver; out2 (may be NULL) receives a second copy
// of the rows (the residual stream).  `pdl` = false launches with a full stream dependency.
int embedding_launch(int dtype, const int* ids, void* out, void* out2, const void* table, int n_tokens, int hidden,
                     int vocab, int* bad_id_flag, bool pdl, cudaStream_t st)
{
    ONELLM_REQUIRE(ids && out && table, ONELLM_ERR_ARG, "embedding: null pointer");
    ONELLM_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, ONELLM_ERR_ARG, "embedding: bad size");
    const size_t es = dtype_size(dtype);
    ONELLM_REQUIRE(es != 0, ONELLM_ERR_UNSUPPORTED, "embedding: dtype %d", dtype);
    ONELLM_REQUIRE(((size_t)hidden * es) % 16 == 0 && aligned16(out) && aligned16(table) && (!out2 || aligned16(out2)),
                   ONELLM_ERR_ARG, "embedding: rows must be 16-byte aligned");
    if (n_tokens == 0) return ONELLM_OK;
    if (!pdl) note_launch();  // launch_pdl counts its own
    if (dtype == ONELLM_F16) {
        if (pdl)
            ONELLM_CUDA(launch_pdl(embedding_kernel<__half>, dim3(n_tokens), dim3(256), 0, st, ids, (__half*)out,
                                   (__half*)out2, (const __half*)table, hidden, vocab, bad_id_flag));
        else
            embedding_kernel<__half><<<n_tokens, 256, 0, st>>>(ids, (__half*)out, (__half*)out2, (const __half*)table,
                                                               hidden, vocab, bad_id_flag);
    } else {
        if (pdl)
            ONELLM_CUDA(launch_pdl(embedding_kernel<float>, dim3(n_tokens), dim3(256), 0, st, ids, (float*)out,
                                   (float*)out2, (const float*)table, hidden, vocab, bad_id_flag));
        else
            embedding_kernel<float><<<n_tokens, 256, 0, st>>>(ids, (float*)out, (float*)out2, (const float*)table, hidden,
                                                              vocab, bad_id_flag);
    }
    ONELLM_CHECK_LAUNCH();
    return ONELLM_OK;
}
}  // namespace onellm

extern "C" int onellm_embedding(int dtype, const int* ids, void* out, const void* table, int n_tokens, int hidden,
                                int vocab, int* bad_id_flag, void* stream)
{
    return embedding_launch(dtype, ids, out, nullptr, table, n_tokens, hidden, vocab, bad_id_flag, true,
                            reinterpret_cast<cudaStream_t>(stream));
}
