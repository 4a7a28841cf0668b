// Drives the reference's LlamaSelfDecoder (src/layers/decoder/self_decoder.cpp:15-78, compiled unchanged from the
// oneLLM tree with its LLaMASelfAttentionLayer and LLaMAFFNLayer) for one decode step of a one-layer model through
// the drop-in headers; results go to the directory given as argv[1] as raw float files, which
// tests/test_dropin_gpu.py checks against the CPU oracle's run of the same sequence.
#include "src/layers/decoder/self_decoder.h"
#include "src/memory/allocator/cuda_allocator.h"

#include "dropin_common.h"

int main(int argc, char** argv)
{
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <output directory>\n", argv[0]);
        return 2;
    }
    g_dir = argv[1];
    const int B = 2, H = 4, Hkv = 2, D = 32, hidden = H * D, QH = H + 2 * Hkv, S = 24, inter = 192;
    const DataType f32 = getTensorType<float>(), i32 = getTensorType<int>();
    LLaMAAttentionStaticParams sp{D, 10000.0f, 2048, false};
    CudaAllocator allocator;
    cublasWrapper wrapper(nullptr, nullptr);
    // ---------------------------------------------------------------- the two decoder classes, one layer each
    {
        LlamaLayerWeight lw(H, Hkv, D, inter, WeightType::FP32_W, /*attn_bias=*/true);
        auto put = [&](void* dst, size_t n, float scale) {
            const std::vector<float> h = randv(n, scale);
            CHECK(cudaMemcpy(dst, h.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        };
        put(lw.attn_norm_weight.gamma, hidden, 1.0f);
        put(lw.ffn_norm_weight.gamma, hidden, 1.0f);
        put(lw.self_attn_weight.qkv.data, (size_t)hidden * QH * D, 0.2f);
        put(lw.self_attn_weight.qkv.bias, (size_t)QH * D, 0.2f);
        put(lw.self_attn_weight.output.data, (size_t)hidden * hidden, 0.2f);
        put(lw.self_attn_weight.output.bias, hidden, 0.2f);
        put(lw.ffn_weight.gate.data, (size_t)hidden * inter, 0.2f);
        put(lw.ffn_weight.up.data, (size_t)hidden * inter, 0.2f);
        put(lw.ffn_weight.down.data, (size_t)inter * hidden, 0.2f);
        float* d_out_norm = to_dev(randv(hidden, 1.0f));
        std::vector<LlamaLayerWeight*> lws{&lw};

        // LlamaSelfDecoder::forward (src/layers/decoder/self_decoder.cpp:15-78): one decode step at step 4
        {
            int step = 4;
            float* d_x = to_dev(randv((size_t)B * hidden, 2.0f));
            float* d_kc = to_dev(randv((size_t)B * Hkv * S * D, 2.0f));
            float* d_vc = to_dev(randv((size_t)B * Hkv * S * D, 2.0f));
            std::vector<unsigned char> fin(B, 0);
            unsigned char* d_fin = to_dev(fin);
            float* d_out = nullptr;
            CHECK(cudaMalloc((void**)&d_out, sizeof(float) * B * hidden));
            LLaMAAttentionDynParams dyn{B, B, 1, step, 1};
            TensorMap in{{"decoder_input", Tensor(GPU, f32, {B, hidden}, d_x)},
                         {"step", Tensor(CPU, i32, {1}, &step)},
                         {"finished", Tensor(GPU, getTensorType<bool>(), {B}, d_fin)},
                         {"output_norm_weight", Tensor(GPU, f32, {hidden}, d_out_norm)}};
            TensorMap out{{"decoder_output", Tensor(GPU, f32, {B, hidden}, d_out)},
                          {"all_k_cache", Tensor(GPU, f32, {1, B, Hkv, S, D}, d_kc)},
                          {"all_v_cache", Tensor(GPU, f32, {1, B, Hkv, S, D}, d_vc)}};
            LlamaSelfDecoder dec(H, Hkv, D, inter, 1, sp, 1e-5f, nullptr, &wrapper, &allocator, true);
            dec.forward(in, lws, out, dyn);
            DeviceSyncAndCheckCudaError();
            dump("sdec_out", d_out, (size_t)B * hidden);
            dump("sdec_residual", d_x, (size_t)B * hidden);
            dump("sdec_k_cache", d_kc, (size_t)B * Hkv * S * D);
            dump("sdec_v_cache", d_vc, (size_t)B * Hkv * S * D);
        }
    }
    std::printf("dropin_self_decoder ok\n");
    return 0;
}
