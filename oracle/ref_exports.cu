// C entry points over the REFERENCE's own code, for oracle/_ref/libonellm_ref.so.
// TEST INFRASTRUCTURE ONLY.  Nothing here restates arithmetic: every function forwards to a function
// or kernel of the reference tree (found through -I<reference root>), compiled where it lies.
//   ref_cpu_*  : the scalar CPU helpers of tests/unittests/*.cu (exact only where noted in the oracle)
//   ref_gpu_*  : the reference's launch* functions on raw device pointers (fp32), for use as a second
//                opinion on the GPU box.  Only launchers whose indexing was checked by reading are exported,
//                and each wrapper documents the argument ranges for which that check holds.
#include "src/utils/tensor.h"
#include "src/weights/llama/norm_weights.h"
#include "src/weights/base_weights.h"
#include "src/models/llama/llama_params.h"
#include "src/kernels/rmsnorm_kernel.h"
#include "src/kernels/activation_kernel.h"
#include "src/kernels/input_embedding.h"
#include "src/kernels/qkv_bias_and_RoPE.h"
#include "src/kernels/append_to_kvcache.h"
#include "src/kernels/transpose_kernel.h"
#include "src/kernels/fused_transpose_reshape_remv_pad.h"
#include "src/kernels/build_casual_mask.h"
// the decode kernel is included as source so that it can be launched with its parameters in the order its
// own signature declares (the shipped launcher passes two of them swapped)
#include "src/kernels/decoder_masked_attn.cu"

#define REF_API extern "C" __attribute__((visibility("default")))

// CPU helpers, defined in the reference's unit-test sources (compiled with main renamed)
void CPUfusedresidandRMSNorm(float*, float*, float*, float*, float, int, int);
void CPUSwiGLU(float*, float*, int, int);
void CPUlinear(float*, float*, float*, int, int, int);
void cpuEmbedding(const int*, float*, float*, const int, const int, const int);
void CPUbuildCasualMask(float*, const int*, const int*, int, int, int);
void CPUfunc(float*, float*, float*, float*, const float*, const int*, const int*, const int*, const int, const int, const int,
             const int, const int, const int, const int, float);

REF_API void ref_cpu_fused_resid_rmsnorm(float* residual, float* decoder_out, float* bias, float* scale, float eps, int hidden, int tokens)
{
    CPUfusedresidandRMSNorm(residual, decoder_out, bias, scale, eps, hidden, tokens);
}
REF_API void ref_cpu_swiglu(float* in, float* out, int batch, int inter) { CPUSwiGLU(in, out, batch, inter); }
// output[m,n] += weight[m,k] . input[k,n]  (tests/unittests/test_linear.cu:30-39)
REF_API void ref_cpu_linear(float* input, float* weight, float* output, int m, int k, int n) { CPUlinear(input, weight, output, m, k, n); }
REF_API void ref_cpu_embedding(const int* ids, float* out, float* table, int n, int hidden, int vocab) { cpuEmbedding(ids, out, table, n, hidden, vocab); }
REF_API void ref_cpu_causal_mask(float* mask, const int* q_lens, const int* k_lens, int max_q, int max_k, int batch)
{
    CPUbuildCasualMask(mask, q_lens, k_lens, max_q, max_k, batch);
}
REF_API void ref_cpu_qkv_bias_rope(float* q, float* k, float* v, float* QKV, const float* bias, const int* padding_offset,
                                   const int* history, const int* input_len, int batch, int seq_len, int tokens, int H, int Hkv,
                                   int D, int rot_dim, float base)
{
    CPUfunc(q, k, v, QKV, bias, padding_offset, history, input_len, batch, seq_len, tokens, H, Hkv, D, rot_dim, base);
}

static Tensor dev_f(std::vector<int> shape, void* p) { return Tensor(Device::GPU, DataType::FP32, shape, p); }
static Tensor dev_i(std::vector<int> shape, void* p) { return Tensor(Device::GPU, DataType::INT32, shape, p); }

// hidden must be a multiple of 4 and at most 4096 (the block is hidden/4 threads)
REF_API int ref_gpu_rmsnorm(float* x, float* gamma, float eps, int tokens, int hidden)
{
    if (hidden % 4 || hidden > 4096 || hidden < 4) return -1;
    Tensor t = dev_f({tokens, hidden}, x);
    LayerNormWeight w{gamma};
    launchRMSNorm(&t, w, eps);
    return (int)cudaDeviceSynchronize();
}
REF_API int ref_gpu_swiglu(const float* in, float* out, int batch, int inter)
{
    launchAct<float>(in, out, batch, inter);
    return (int)cudaDeviceSynchronize();
}
// ids must lie in [0, vocab)
REF_API int ref_gpu_embedding(int* ids, float* out, float* table, int batch, int seq, int hidden, int vocab)
{
    Tensor a = dev_i({batch, seq}, ids), o = dev_f({batch, seq, hidden}, out), t = dev_f({vocab, hidden}, table);
    launchInputEmbedding(&a, &o, &t);
    return (int)cudaDeviceSynchronize();
}
// D must be a multiple of 4; padding_offset[t] + t < batch*seq_len for every token; bias must be non-null
REF_API int ref_gpu_qkv_bias_rope(float* q, float* k, float* v, float* QKV, float* bias, int* padding_offset, int* history,
                                  int* input_len, int batch, int seq_len, int tokens, int H, int Hkv, int D, int rot_dim, float base)
{
    if (D % 4 || !bias) return -1;
    Tensor tq = dev_f({batch, H, seq_len, D}, q), tk = dev_f({batch, Hkv, seq_len, D}, k), tv = dev_f({batch, Hkv, seq_len, D}, v);
    Tensor tQKV = dev_f({tokens, H + 2 * Hkv, D}, QKV);
    Tensor po = dev_i({tokens}, padding_offset), hl = dev_i({batch}, history), il = dev_i({batch}, input_len);
    BaseWeight w;
    w.data = nullptr;
    w.bias = bias;
    w.type = WeightType::FP32_W;
    LLaMAAttentionStaticParams sp{rot_dim, base, 2048, false};
    launchAddFusedQKVBiasTransposeAndRoPE(&tq, &tk, &tv, &tQKV, w, &po, &hl, &il, sp);
    return (int)cudaDeviceSynchronize();
}
// history[b] + cur_len[b] <= max_seq_len for every sequence
REF_API int ref_gpu_append_kv(float* k_src, float* v_src, int* cur_len, int* history, float* k_dst, float* v_dst, int batch,
                              int Hkv, int max_q_len, int max_seq_len, int D)
{
    Tensor ks = dev_f({batch, Hkv, max_q_len, D}, k_src), vs = dev_f({batch, Hkv, max_q_len, D}, v_src);
    Tensor kd = dev_f({batch, Hkv, max_seq_len, D}, k_dst), vd = dev_f({batch, Hkv, max_seq_len, D}, v_dst);
    int layer = 0;
    Tensor lid(Device::CPU, DataType::INT32, {1}, &layer);
    Tensor cl = dev_i({batch}, cur_len), hl = dev_i({batch}, history);
    launchAppendKVCache(&ks, &vs, &lid, &cl, &hl, &kd, &vd);
    return (int)cudaDeviceSynchronize();
}
// context_len[b] <= max_k_len <= max_seq_len
REF_API int ref_gpu_repeat_kv(float* k_src, float* v_src, int* context_len, float* k_dst, float* v_dst, int batch, int H,
                              int Hkv, int max_seq_len, int max_k_len, int D)
{
    Tensor ks = dev_f({batch, Hkv, max_seq_len, D}, k_src), vs = dev_f({batch, Hkv, max_seq_len, D}, v_src);
    Tensor kd = dev_f({batch, H, max_k_len, D}, k_dst), vd = dev_f({batch, H, max_k_len, D}, v_dst);
    int layer = 0;
    Tensor lid(Device::CPU, DataType::INT32, {1}, &layer);
    Tensor cl = dev_i({batch}, context_len);
    launchTransposeKVCache(&ks, &vs, &cl, &lid, &kd, &vd);
    return (int)cudaDeviceSynchronize();
}
// padding_offset[t] + t < batch*seq_len for every token
REF_API int ref_gpu_transpose_remove_padding(float* src, int* padding_offset, float* dst, int batch, int H, int seq_len, int D,
                                             int tokens)
{
    Tensor s = dev_f({batch, H, seq_len, D}, src), d = dev_f({tokens, H, D}, dst), po = dev_i({tokens}, padding_offset);
    launchTransposeOutRemovePadding(&s, &po, &d);
    return (int)cudaDeviceSynchronize();
}
REF_API int ref_gpu_causal_mask(float* mask, const int* q_lens, const int* k_lens, int max_q, int max_k, int batch)
{
    launchBuildCausalMasks<float>(mask, q_lens, k_lens, max_q, max_k, batch);
    return (int)cudaDeviceSynchronize();
}
// The decode kernel, launched with its parameters in declaration order.  Valid only for
// Hkv == H (its KV head mapping), step <= D <= 1024 (softmax covers the first blockDim logits), D % 4 == 0,
// separate q/k/v [B,H,D] buffers and caches laid out [S, B, H, D] with S >= step.
REF_API int ref_gpu_masked_mha(const float* q, const float* k, const float* v, float* bias, float* k_cache, float* v_cache,
                               float* out, int B, int H, int D, int step, int rot_dim, float base)
{
    if (step > D || D % 4 || D > 1024 || step < 1 || !bias) return -1;
    masked_MHA_kernel<<<B * H, D, (3 * D + step) * sizeof(float)>>>(q, k, v, bias, k_cache, v_cache, out, B, H, H, D, step,
                                                                    rsqrtf((float)D), rot_dim, base);
    return (int)cudaDeviceSynchronize();
}
