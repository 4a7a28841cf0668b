// Drop-in for src/weights/llama/layer_weights.h + layer_weights.cc of oneLLM: one decoder layer's
// weights (constructor allocates :2-39, loadWeights from files :42-56 or from caller-owned device
// pointers :58-82, destructor frees :96-107).  Header-only; fp32 or fp16 storage by weight_type.
// File names (no separator between weight_path and the suffix): .attention_norm.weight,
// .ffn_norm.weight, .attention.w_qkv.weight, .attention.wo.weight, .feed_forward.w1.weight (gate),
// .feed_forward.w3.weight (up), .feed_forward.w2.weight (down), .attention.w_qkv.bias, .attention.wo.bias.
#pragma once
#include <stdexcept>
#include <string>

#include "src/utils/cuda_utils.h"
#include "src/weights/llama/attention_weights.h"
#include "src/weights/llama/ffn_weights.h"
#include "src/weights/llama/norm_weights.h"

struct LlamaLayerWeight {
private:
    int head_num;
    int kv_head_num;
    int head_size;
    int hidden_units;
    int inter_size;
    WeightType weight_type;
    int bit_size;
    bool attn_bias;
    bool owns_ = true;  // false once loadWeights(T*...) has re-pointed the members to caller memory

    size_t elem() const { return static_cast<size_t>(bit_size / 8); }
    void* devAlloc(size_t count)
    {
        void* p = nullptr;
        CHECK(cudaMalloc(&p, count * elem()));
        return p;
    }
    void describe(BaseWeight& w, int rows, int cols, bool with_bias)
    {
        w.type = weight_type;
        w.shape = {rows, cols};
        w.data = devAlloc(static_cast<size_t>(rows) * cols);
        w.bias = with_bias ? devAlloc(cols) : nullptr;
    }
    template <typename T>
    void readAll(const std::string& p)
    {
        const size_t h = hidden_units, qkv = static_cast<size_t>(head_num + 2 * kv_head_num) * head_size, I = inter_size;
        int bad = 0;
        bad |= loadWeightFromBin<T, T>((T*)attn_norm_weight.gamma, {h}, p + ".attention_norm.weight");
        bad |= loadWeightFromBin<T, T>((T*)ffn_norm_weight.gamma, {h}, p + ".ffn_norm.weight");
        bad |= loadWeightFromBin<T, T>((T*)self_attn_weight.qkv.data, {h, qkv}, p + ".attention.w_qkv.weight");
        bad |= loadWeightFromBin<T, T>((T*)self_attn_weight.output.data, {h, h}, p + ".attention.wo.weight");
        bad |= loadWeightFromBin<T, T>((T*)ffn_weight.gate.data, {h, I}, p + ".feed_forward.w1.weight");
        bad |= loadWeightFromBin<T, T>((T*)ffn_weight.up.data, {h, I}, p + ".feed_forward.w3.weight");
        bad |= loadWeightFromBin<T, T>((T*)ffn_weight.down.data, {I, h}, p + ".feed_forward.w2.weight");
        if (attn_bias) {
            bad |= loadWeightFromBin<T, T>((T*)self_attn_weight.qkv.bias, {qkv}, p + ".attention.w_qkv.bias");
            bad |= loadWeightFromBin<T, T>((T*)self_attn_weight.output.bias, {h}, p + ".attention.wo.bias");
        }
        if (bad) throw std::runtime_error("[oneLLM][ERROR] weights under " + p + " are missing or of the wrong size");
    }
    void release()
    {
        if (!owns_) return;
        cudaFree(attn_norm_weight.gamma);
        cudaFree(ffn_norm_weight.gamma);
        for (BaseWeight* w : {&self_attn_weight.qkv, &self_attn_weight.output, &ffn_weight.gate, &ffn_weight.up, &ffn_weight.down}) {
            cudaFree(w->data);
            if (w->bias) cudaFree(w->bias);
            w->data = w->bias = nullptr;
        }
        attn_norm_weight.gamma = ffn_norm_weight.gamma = nullptr;
    }

public:
    LlamaLayerWeight() = delete;
    LlamaLayerWeight(const LlamaLayerWeight&) = delete;
    LlamaLayerWeight& operator=(const LlamaLayerWeight&) = delete;

    LlamaLayerWeight(int head_num, int kv_head_num, int head_size, int inter_size, WeightType weight_type, bool attn_bias)
        : head_num(head_num), kv_head_num(kv_head_num), head_size(head_size), hidden_units(head_num * head_size),
          inter_size(inter_size), weight_type(weight_type), bit_size(getBitNum(weight_type)), attn_bias(attn_bias)
    {
        if (weight_type != WeightType::FP32_W && weight_type != WeightType::FP16_W)
            throw std::runtime_error("[oneLLM][ERROR] layer weights are FP32_W or FP16_W");
        attn_norm_weight.gamma = static_cast<float*>(devAlloc(hidden_units));
        ffn_norm_weight.gamma = static_cast<float*>(devAlloc(hidden_units));
        describe(self_attn_weight.qkv, hidden_units, (head_num + 2 * kv_head_num) * head_size, attn_bias);
        describe(self_attn_weight.output, hidden_units, hidden_units, attn_bias);
        describe(ffn_weight.gate, hidden_units, inter_size, false);
        describe(ffn_weight.up, hidden_units, inter_size, false);
        describe(ffn_weight.down, inter_size, hidden_units, false);
    }
    ~LlamaLayerWeight() { release(); }

    // weight_path: everything in front of ".attention_norm.weight" etc.; files hold the storage type
    void loadWeights(std::string weight_path, WeightType /*file_type*/)
    {
        if (weight_type == WeightType::FP16_W) readAll<half>(weight_path);
        else readAll<float>(weight_path);
    }

    // adopt caller-owned device arrays; what the constructor allocated is returned to the driver
    template <typename T>
    void loadWeights(T* d_attn_norm_weight, T* d_ffn_norm_weight, T* d_qkv_weights, T* d_qkv_bias, T* d_output_weights,
                     T* d_out_bias, T* d_ffn_down, T* d_ffn_down_bias, T* d_ffn_gate, T* d_ffn_up)
    {
        release();
        owns_ = false;
        attn_norm_weight.gamma = reinterpret_cast<float*>(d_attn_norm_weight);
        ffn_norm_weight.gamma = reinterpret_cast<float*>(d_ffn_norm_weight);
        self_attn_weight.qkv.data = d_qkv_weights;
        self_attn_weight.qkv.bias = d_qkv_bias;
        self_attn_weight.output.data = d_output_weights;
        self_attn_weight.output.bias = d_out_bias;
        ffn_weight.gate.data = d_ffn_gate;
        ffn_weight.up.data = d_ffn_up;
        ffn_weight.down.data = d_ffn_down;
        ffn_weight.down.bias = d_ffn_down_bias;
    }

    LayerNormWeight attn_norm_weight;
    LayerNormWeight ffn_norm_weight;
    LLaMAattentionWeights self_attn_weight;
    LLaMAFFNWeights ffn_weight;
};
