// Tiled tensor-core projection for M > 64 (context phase).
#include "common.cuh"

namespace onellm {

int gemm_f16_skinny(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout,
                    cudaStream_t st);

int gemm_f16_large(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout,
                   cudaStream_t st)
{
    // TEMPORARY: 64-token passes of the weight-streaming kernel until the tiled kernel lands.
    for (int m0 = 0; m0 < M; m0 += 64) {
        const int mm = M - m0 < 64 ? M - m0 : 64;
        const int rc = gemm_f16_skinny(x + (size_t)m0 * K, W, y + (size_t)m0 * N, mm, N, K, w_layout, st);
        if (rc) return rc;
    }
    return ONELLM_OK;
}

}  // namespace onellm
