// Drives the reference's LLaMAFFNLayer (src/layers/ffn/ffn.cpp:53-73) and LlamaContextDecoder
// (src/layers/decoder/context_decoder.cpp:32-134), compiled unchanged from the oneLLM tree, through the drop-in
// headers: one FFN call and the context phase of a one-layer model; results go to the directory given as argv[1]
// as raw float files, which tests/test_dropin_gpu.py checks against the CPU oracle's run of the same sequences.
#include "src/layers/decoder/context_decoder.h"
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
    // ---------------------------------------------------------------- LLaMAFFNLayer::forward (src/layers/ffn/ffn.cpp:53-73)
    // The layer never writes its "ffn_output" tensor: the down projection lands in a buffer of its own.  The allocator
    // below remembers what it handed out, in order (gate/up buffer, SwiGLU output, down-projection output).
    struct RecordingAllocator : BaseAllocator {
        CudaAllocator inner;
        std::vector<void*> got;
        void* deviceMalloc(void* ptr, size_t size, bool is_host = false) override
        {
            void* p = inner.deviceMalloc(ptr, size, is_host);
            got.push_back(p);
            return p;
        }
        void deviceFree(void* ptr, bool is_host = false) override { inner.deviceFree(ptr, is_host); }
    };
    {
        const int T = 3;
        RecordingAllocator rec;
        float* d_x = to_dev(randv((size_t)T * hidden, 2.0f));
        LLaMAFFNWeights fw;
        fw.gate.shape = fw.up.shape = {hidden, inter};
        fw.down.shape = {inter, hidden};
        fw.gate.data = to_dev(randv((size_t)hidden * inter, 0.2f));
        fw.up.data = to_dev(randv((size_t)hidden * inter, 0.2f));
        fw.down.data = to_dev(randv((size_t)inter * hidden, 0.2f));
        float* d_y = nullptr;
        CHECK(cudaMalloc((void**)&d_y, sizeof(float) * T * hidden));
        LLaMAAttentionDynParams dyn{T, T, 1, 1, 1};  // launchAct takes its row count from batch_size (ffn.cpp:66)
        TensorMap in{{"ffn_input", Tensor(GPU, f32, {T, hidden}, d_x)}};
        TensorMap out{{"ffn_output", Tensor(GPU, f32, {T, hidden}, d_y)}};
        LLaMAFFNLayer ffn(H, D, inter, nullptr, &wrapper, &rec, false);
        ffn.forward(in, out, fw, dyn);
        DeviceSyncAndCheckCudaError();
        if (rec.got.size() != 3) return 6;
        dump("ffn_class_down_out", rec.got[2], (size_t)T * hidden);
    }

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

        // LlamaContextDecoder::forward (src/layers/decoder/context_decoder.cpp:32-134): two prompts of 5 and 3 tokens,
        // the first behind a history of 2
        {
            const std::vector<int> lens = {5, 3}, hist = {2, 0}, ctx = {7, 3};
            const int T = 8, max_q = 5, max_k = 7;
            float* d_x = to_dev(randv((size_t)T * hidden, 2.0f));
            float* d_kc = to_dev(randv((size_t)B * Hkv * S * D, 2.0f));
            float* d_vc = to_dev(randv((size_t)B * Hkv * S * D, 2.0f));
            int *d_lens = to_dev(lens), *d_hist = to_dev(hist), *d_ctx = to_dev(ctx);
            int* d_po = nullptr;
            float *d_mask = nullptr, *d_out = nullptr;
            CHECK(cudaMalloc((void**)&d_po, sizeof(int) * B * max_q));
            CHECK(cudaMalloc((void**)&d_mask, sizeof(float) * B * max_q * max_k));
            CHECK(cudaMalloc((void**)&d_out, sizeof(float) * T * hidden));
            LLaMAAttentionDynParams dyn{B, T, max_q, max_k, 1};
            TensorMap in{{"decoder_input", Tensor(GPU, f32, {T, hidden}, d_x)},
                         {"padding_offset", Tensor(GPU, i32, {B * max_q}, d_po)},
                         {"history_length", Tensor(GPU, i32, {B}, d_hist)},
                         {"input_length", Tensor(GPU, i32, {B}, d_lens)},
                         {"context_length", Tensor(GPU, i32, {B}, d_ctx)},
                         {"attention_mask", Tensor(GPU, f32, {B, max_q, max_k}, d_mask)},
                         {"output_norm_weight", Tensor(GPU, f32, {hidden}, d_out_norm)}};
            TensorMap out{{"decoder_output", Tensor(GPU, f32, {T, hidden}, d_out)},
                          {"all_k_cache", Tensor(GPU, f32, {1, B, Hkv, S, D}, d_kc)},
                          {"all_v_cache", Tensor(GPU, f32, {1, B, Hkv, S, D}, d_vc)}};
            LlamaContextDecoder dec(H, Hkv, D, inter, 1, sp, 1e-5f, nullptr, &wrapper, &allocator, true);
            dec.forward(in, lws, out, dyn);
            DeviceSyncAndCheckCudaError();
            dump("cdec_out", d_out, (size_t)T * hidden);
            dump("cdec_residual", d_x, (size_t)T * hidden);
            dump("cdec_k_cache", d_kc, (size_t)B * Hkv * S * D);
            dump("cdec_v_cache", d_vc, (size_t)B * Hkv * S * D);
        }
    }
    std::printf("dropin_context_decoder ok\n");
    return 0;
}
