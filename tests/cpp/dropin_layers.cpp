// Drives the reference's own attention layer classes (LLaMAContextAttentionLayer, LLaMASelfAttentionLayer, compiled
// unchanged from the oneLLM tree) and the launch* entry points through the drop-in headers, on seeded
// inputs, and writes every result as a raw float file into the directory given as argv[1].  The pytest
// side regenerates the same inputs and checks the files against the CPU oracle.  (The FFN layer and the two
// decoder classes are driven by dropin_self_decoder.cpp and dropin_context_decoder.cpp: the reference's layer
// headers carry no include guards, so the two decoders cannot share a translation unit.)
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "src/kernels/activation_kernel.h"
#include "src/kernels/build_casual_mask.h"
#include "src/kernels/cal_paddingoffset.h"
#include "src/kernels/beamsearch_topK.h"
#include "src/kernels/fused_addresidual_norm.h"
#include "src/kernels/input_embedding.h"
#include "src/kernels/rmsnorm_kernel.h"
#include "src/kernels/topK_sampling.h"
#include "src/layers/attention/context_attention.h"
#include "src/layers/attention/masked_self_attention.h"
#include "src/memory/allocator/cuda_allocator.h"
#include "src/weights/llama/llama_weights.h"

#include "dropin_common.h"

int main(int argc, char** argv)
{
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <output directory>\n", argv[0]);
        return 2;
    }
    g_dir = argv[1];
    const int B = 2, H = 4, Hkv = 2, D = 32, hidden = H * D, QH = H + 2 * Hkv, S = 24, L = 2, inter = 192;
    const DataType f32 = getTensorType<float>(), i32 = getTensorType<int>();
    LLaMAAttentionStaticParams sp{D, 10000.0f, 2048, false};
    CudaAllocator allocator;
    cublasWrapper wrapper(nullptr, nullptr);

    // weights shared by both attention layers
    LLaMAattentionWeights aw;
    aw.qkv.shape = {hidden, QH * D};
    aw.qkv.data = to_dev(randv((size_t)hidden * QH * D, 0.2f));
    aw.qkv.bias = to_dev(randv((size_t)QH * D, 0.2f));
    aw.output.shape = {hidden, hidden};
    aw.output.data = to_dev(randv((size_t)hidden * hidden, 0.2f));

    // ---------------------------------------------------------------- context phase, layer 1 of 2
    {
        const std::vector<int> lens = {5, 3}, hist = {2, 0}, ctx = {7, 3};
        const int T = 8, max_q = 5, max_k = 7;
        float* d_x = to_dev(randv((size_t)T * hidden, 2.0f));
        float* d_kc = to_dev(randv((size_t)L * B * Hkv * S * D, 2.0f));
        float* d_vc = to_dev(randv((size_t)L * B * Hkv * S * D, 2.0f));
        int *d_lens = to_dev(lens), *d_hist = to_dev(hist), *d_ctx = to_dev(ctx);
        int *d_po = nullptr, *d_cum = nullptr;
        float *d_mask = nullptr, *d_out = nullptr;
        CHECK(cudaMalloc((void**)&d_po, sizeof(int) * B * max_q));
        CHECK(cudaMalloc((void**)&d_cum, sizeof(int) * (B + 1)));
        CHECK(cudaMalloc((void**)&d_mask, sizeof(float) * B * max_q * max_k));
        CHECK(cudaMalloc((void**)&d_out, sizeof(float) * T * hidden));
        int pinned = 0, token_num = 0;
        launchCalPaddingoffset(&pinned, &token_num, d_po, d_cum, d_lens, B, max_q);
        launchBuildCausalMasks(d_mask, d_lens, d_ctx, max_q, max_k, B);
        if (token_num != T) return 3;
        int layer = 1;
        LLaMAAttentionDynParams dyn{B, T, max_q, max_k, L};
        TensorMap in{{"attention_input", Tensor(GPU, f32, {T, hidden}, d_x)},
                     {"padding_offset", Tensor(GPU, i32, {T}, d_po)},
                     {"history_length", Tensor(GPU, i32, {B}, d_hist)},
                     {"input_length", Tensor(GPU, i32, {B}, d_lens)},
                     {"context_length", Tensor(GPU, i32, {B}, d_ctx)},
                     {"attention_mask", Tensor(GPU, f32, {B, max_q, max_k}, d_mask)},
                     {"layer_id", Tensor(GPU, i32, {1}, &layer)}};  // tagged GPU, host pointer: as context_decoder.cpp does
        TensorMap out{{"attention_output", Tensor(GPU, f32, {T, hidden}, d_out)},
                      {"all_k_cache", Tensor(GPU, f32, {L, B, Hkv, S, D}, d_kc)},
                      {"all_v_cache", Tensor(GPU, f32, {L, B, Hkv, S, D}, d_vc)}};
        LLaMAContextAttentionLayer layer_obj(H, Hkv, D, sp, nullptr, &wrapper, &allocator, true);
        layer_obj.forward(in, out, aw, dyn, sp);
        DeviceSyncAndCheckCudaError();
        dump("ctx_out", d_out, (size_t)T * hidden);
        dump("ctx_k_cache", d_kc, (size_t)L * B * Hkv * S * D);
        dump("ctx_v_cache", d_vc, (size_t)L * B * Hkv * S * D);
        dump("ctx_mask", d_mask, (size_t)B * max_q * max_k);
    }

    // ---------------------------------------------------------------- decode step
    {
        int step = 6, layer = 0;
        float* d_x = to_dev(randv((size_t)B * hidden, 2.0f));
        float* d_kc = to_dev(randv((size_t)L * B * Hkv * S * D, 2.0f));
        float* d_vc = to_dev(randv((size_t)L * B * Hkv * S * D, 2.0f));
        std::vector<unsigned char> fin(B, 0);
        unsigned char* d_fin = to_dev(fin);
        float* d_out = nullptr;
        CHECK(cudaMalloc((void**)&d_out, sizeof(float) * B * hidden));
        LLaMAAttentionDynParams dyn{B, B, 1, step, L};
        TensorMap in{{"attention_input", Tensor(GPU, f32, {B, hidden}, d_x)},
                     {"finished", Tensor(GPU, getTensorType<bool>(), {B}, d_fin)},
                     {"step", Tensor(CPU, i32, {1}, &step)},
                     {"layer_id", Tensor(CPU, i32, {1}, &layer)}};
        TensorMap out{{"attention_output", Tensor(GPU, f32, {B, hidden}, d_out)},
                      {"all_k_cache", Tensor(GPU, f32, {L, B, Hkv, S, D}, d_kc)},
                      {"all_v_cache", Tensor(GPU, f32, {L, B, Hkv, S, D}, d_vc)}};
        LLaMASelfAttentionLayer layer_obj(H, Hkv, D, sp, nullptr, &wrapper, &allocator, true);
        layer_obj.forward(in, out, aw, dyn);
        DeviceSyncAndCheckCudaError();
        dump("dec_out", d_out, (size_t)B * hidden);
        dump("dec_k_cache", d_kc, (size_t)B * Hkv * S * D);  // layer 0 is what the launcher touches
        dump("dec_v_cache", d_vc, (size_t)B * Hkv * S * D);
    }

    // ---------------------------------------------------------------- FFN sequence of src/layers/ffn/ffn.cpp:62-68
    {
        const int T = 3;
        float* d_x = to_dev(randv((size_t)T * hidden, 2.0f));
        BaseWeight gate, up, down;
        gate.shape = up.shape = {hidden, inter};
        down.shape = {inter, hidden};
        gate.data = to_dev(randv((size_t)hidden * inter, 0.2f));
        up.data = to_dev(randv((size_t)hidden * inter, 0.2f));
        down.data = to_dev(randv((size_t)inter * hidden, 0.2f));
        Tensor x(GPU, f32, {T, hidden}, d_x);
        Tensor gu(GPU, f32, {2, T, inter}), act(GPU, f32, {T, inter}), y(GPU, f32, {T, hidden});
        gu.data = allocator.Malloc(gu.data, sizeof(float) * 2 * T * inter, false);
        act.data = allocator.Malloc(act.data, sizeof(float) * T * inter, false);
        y.data = allocator.Malloc(y.data, sizeof(float) * T * hidden, false);
        launchLinearGemm(&x, gate, &gu);
        launchLinearGemm(&x, up, &gu, false, false, true);
        launchAct((float*)gu.data, (float*)act.data, T, inter);
        launchLinearGemm(&act, down, &y);
        DeviceSyncAndCheckCudaError();
        dump("ffn_out", y.data, (size_t)T * hidden);
        // norms on the same activations
        LayerNormWeight gamma;
        gamma.gamma = to_dev(randv(hidden, 1.0f));
        float* d_res = to_dev(randv((size_t)T * hidden, 2.0f));
        launchFusedAddBiasResidualRMSNorm(d_res, (float*)y.data, (const float*)nullptr, (const float*)gamma.gamma, 1e-5f, T, hidden);
        launchRMSNorm(&x, gamma, 1e-5f);
        DeviceSyncAndCheckCudaError();
        dump("norm_residual", d_res, (size_t)T * hidden);
        dump("norm_fused", y.data, (size_t)T * hidden);
        dump("norm_plain", d_x, (size_t)T * hidden);
        void* first = act.data;
        allocator.deviceFree(act.data);
        void* again = allocator.deviceMalloc(nullptr, sizeof(float) * T * inter, false);
        if (again != first) return 4;  // a freed block is handed out again instead of a new cudaMalloc
    }

    // ---------------------------------------------------------------- embedding, top-K, sampling
    {
        const int V = 1000, hid = 64, rows = 2;
        std::vector<int> ids = {7, 999, 0, 512};
        float* d_table = to_dev(randv((size_t)V * hid, 2.0f));
        int* d_ids = to_dev(ids);
        float* d_emb = nullptr;
        CHECK(cudaMalloc((void**)&d_emb, sizeof(float) * 4 * hid));
        Tensor t_ids(GPU, i32, {2, 2}, d_ids), t_emb(GPU, f32, {2, 2, hid}, d_emb), t_table(GPU, f32, {V, hid}, d_table);
        launchInputEmbedding(&t_ids, &t_emb, &t_table);
        dump("emb_out", d_emb, 4 * hid);
        // beam-search top-K over [rows * 2, V] scores, then one sampled token per row
        float* d_probs = to_dev(randv((size_t)rows * 2 * V, 20.0f));
        float* d_ws = nullptr;
        const size_t ws_floats = 2 * (size_t)rows * 2 + 2 * (size_t)rows * 2 * 8 * 2;
        CHECK(cudaMalloc((void**)&d_ws, sizeof(float) * ws_floats));
        launchTopKforBeamSearch(d_probs, rows, V, d_ws);
        float* final_vals = d_ws + 2 * (size_t)rows * 2 * 8 * 2;
        int* final_ids = (int*)(final_vals + rows * 2);
        dump("topk_vals", final_vals, rows * 2);
        dump("topk_ids_as_float_bits", final_ids, rows * 2);
        std::vector<int> seqlen = {10, 20}, outid(rows, -1);
        int* d_seqlen = to_dev(seqlen);
        int* d_outid = to_dev(outid);
        std::vector<unsigned char> fin(rows, 0);
        unsigned char* d_fin = to_dev(fin);
        Tensor t_id(GPU, i32, {rows, 2}, final_ids), t_val(GPU, f32, {rows, 2}, final_vals), t_seq(GPU, i32, {rows}, d_seqlen),
            t_fin(GPU, getTensorType<bool>(), {rows}, d_fin), t_out(GPU, i32, {rows}, d_outid);
        IntDict params{{"vocab_size", V}, {"step", 5}, {"end_id", 2}};
        launchSampling(&t_id, &t_val, &t_seq, &t_fin, &t_out, params);
        DeviceSyncAndCheckCudaError();
        dump("sample_ids_as_float_bits", d_outid, rows);
        dump("sample_seqlen_as_float_bits", d_seqlen, rows);
    }

    // ---------------------------------------------------------------- weight classes
    {
        LlamaWeight w(H, Hkv, D, inter, 100, 2, /*attn_bias=*/true, WeightType::FP32_W);
        if (w.layers().size() != 2 || w.layers()[0]->self_attn_weight.qkv.shape[1] != QH * D || !w.layers()[1]->ffn_weight.down.data) return 5;
    }
    std::printf("dropin_layers ok\n");
    return 0;
}
