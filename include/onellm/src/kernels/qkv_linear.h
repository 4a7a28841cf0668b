// Drop-in for src/kernels/qkv_linear.h of oneLLM: launchLinearGemm (:9-14, qkv_linear.cu:8-65) and
// launchLinearStridedBatchGemm (:16-20, qkv_linear.cu:67-120) on the onellm_b200 kernels.
// Both compute what the layers need from them, with row-major operands read from the tensors:
//   launchLinearGemm:  output[T, N] = input[T, K] . W, W = weight.data [K, N] ([N, K] if trans_b).
//     T = (elements of input) / K, so a 3-D input [a, b, c] against a weight with b*c rows is
//     [a, b*c].  N and K come from weight.shape (the reference reads N from output->shape[1], which
//     is wrong for 3-D outputs).  No handle is created per call (the reference creates a cuBLAS
//     handle in every call and never destroys it).
//     An output of shape {2, T, N} is the FFN's gate/up buffer (src/layers/ffn/ffn.cpp:25,62-66): it
//     is filled as [T, 2, N], the layout launchAct reads; shared_out_buf selects the second half.
//   launchLinearStridedBatchGemm: out[b,h] = in1[b,h] . in2[b,h] (in2 transposed if trans_b) over the
//     two leading extents; used for Q.K^T and P.V of the context phase.
#pragma once
#include "src/kernels/cublas_wrapper.h"
#include "src/utils/tensor.h"
#include "src/weights/base_weights.h"

inline void launchLinearGemm(Tensor* input, BaseWeight& weight, Tensor* output, bool trans_a = false, bool trans_b = false,
                             bool shared_out_buf = false)
{
    ONELLM_CHECK_WITH_INFO(!trans_a, "launchLinearGemm: a transposed input is not supported");
    ONELLM_CHECK_WITH_INFO(weight.shape.size() == 2 && weight.data, "launchLinearGemm: weight needs a 2-D shape and data");
    const int K = trans_b ? weight.shape[1] : weight.shape[0];
    const int N = trans_b ? weight.shape[0] : weight.shape[1];
    const long in_elems = input->size();
    ONELLM_CHECK_WITH_INFO(in_elems > 0 && in_elems % K == 0, "launchLinearGemm: input extent does not match the weight");
    const int T = static_cast<int>(in_elems / K);
    const size_t esz = getTypeSize(output->dtype);
    char* y = static_cast<char*>(output->data);
    long ldy = N;
    if (output->shape.size() == 3 && output->shape[0] == 2 && output->shape[1] == T && output->shape[2] == N) {
        ldy = 2L * N;
        if (shared_out_buf) y += static_cast<size_t>(N) * esz;
    } else {
        ONELLM_CHECK_WITH_INFO(!shared_out_buf, "launchLinearGemm: shared_out_buf needs an output of shape {2, tokens, N}");
    }
    ONELLM_B200_CALL(onellm_gemm_ld(onellmDtype(input->dtype), input->data, weight.data, y, ldy, T, N, K,
                                    trans_b ? ONELLM_W_NK : ONELLM_W_KN, nullptr));
}

inline void launchLinearStridedBatchGemm(Tensor* input1, Tensor* input2, Tensor* output, bool trans_a = false, bool trans_b = false)
{
    ONELLM_CHECK_WITH_INFO(input1->shape.size() == 4 && input2->shape.size() == 4, "launchLinearStridedBatchGemm: 4-D tensors expected");
    const int batch = input1->shape[0] * input1->shape[1];
    const int m = trans_a ? input1->shape[3] : input1->shape[2];
    const int k = trans_a ? input1->shape[2] : input1->shape[3];
    const int n = trans_b ? input2->shape[2] : input2->shape[3];
    ONELLM_CHECK_WITH_INFO((trans_b ? input2->shape[3] : input2->shape[2]) == k, "launchLinearStridedBatchGemm: inner extents differ");
    ONELLM_B200_CALL(onellm_batched_gemm(onellmDtype(input1->dtype), input1->data, input2->data, output->data, batch, m, n, k, trans_a,
                                         trans_b, nullptr));
}
