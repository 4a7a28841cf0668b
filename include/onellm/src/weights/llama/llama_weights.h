// Drop-in for src/weights/llama/llama_weights.h + llama_weights.cc of oneLLM (:8-35; constructor
// :3-34, loadWeights :36-46, destructor :48-57): all layers plus final norm, token embedding and LM
// head.  Files: <p>.norm.weight [h], <p>.tok_embeddings.weight [V,h], <p>.output.weight [V,h],
// <p>layers.<l>.* per layer.  The reference loads tok_embeddings into the POST-decoder table and
// output.weight into the PRE-decoder table (:40-41); here each goes where its name says.
// Additions: accessors for what the reference keeps private and never exposes.
#pragma once
#include <string>
#include <vector>

#include "src/weights/base_weights.h"
#include "src/weights/llama/embedding_weights.h"
#include "src/weights/llama/layer_weights.h"
#include "src/weights/weight.h"

struct LlamaWeight : public Weight {
private:
    int hidden_units = 0;
    int inter_size = 0;
    int vocab_size = 0;
    int vocab_size_padded = 0;
    int num_layer = 0;
    WeightType weight_type = WeightType::FP32_W;
    std::vector<LlamaLayerWeight*> llama_layer_weight;
    LayerNormWeight out_rmsnorm_weight;
    EmbeddingWeight post_decoder_embedding_weight;
    EmbeddingWeight pre_decoder_embedding_weight;

    float* devAlloc(size_t count)
    {
        void* p = nullptr;
        CHECK(cudaMalloc(&p, count * (getBitNum(weight_type) / 8)));
        return static_cast<float*>(p);
    }
    template <typename T>
    void readTop(const std::string& p)
    {
        const size_t h = hidden_units, V = vocab_size;
        int bad = 0;
        bad |= loadWeightFromBin<T, T>((T*)out_rmsnorm_weight.gamma, {h}, p + ".norm.weight");
        bad |= loadWeightFromBin<T, T>((T*)pre_decoder_embedding_weight.emb_table, {V, h}, p + ".tok_embeddings.weight");
        bad |= loadWeightFromBin<T, T>((T*)post_decoder_embedding_weight.emb_table, {V, h}, p + ".output.weight");
        if (bad) throw std::runtime_error("[oneLLM][ERROR] weights under " + p + " are missing or of the wrong size");
    }

public:
    LlamaWeight() = default;
    LlamaWeight(const LlamaWeight&) = delete;
    LlamaWeight& operator=(const LlamaWeight&) = delete;

    LlamaWeight(int head_num, int kv_head_num, int head_size, int inter_size, int vocab_size, int num_layer, bool attn_bias,
                WeightType weight_type)
        : hidden_units(head_num * head_size), inter_size(inter_size), vocab_size(vocab_size), vocab_size_padded(vocab_size),
          num_layer(num_layer), weight_type(weight_type)
    {
        llama_layer_weight.reserve(num_layer);
        for (int l = 0; l < num_layer; ++l)
            llama_layer_weight.push_back(new LlamaLayerWeight(head_num, kv_head_num, head_size, inter_size, weight_type, attn_bias));
        out_rmsnorm_weight.gamma = devAlloc(hidden_units);
        post_decoder_embedding_weight.emb_table = devAlloc(static_cast<size_t>(vocab_size) * hidden_units);
        pre_decoder_embedding_weight.emb_table = devAlloc(static_cast<size_t>(vocab_size) * hidden_units);
    }

    ~LlamaWeight() override
    {
        cudaFree(pre_decoder_embedding_weight.emb_table);
        cudaFree(post_decoder_embedding_weight.emb_table);
        cudaFree(out_rmsnorm_weight.gamma);
        for (LlamaLayerWeight* p : llama_layer_weight) delete p;
    }

    void loadWeights(std::string weight_path) override
    {
        if (weight_type == WeightType::FP16_W) readTop<half>(weight_path);
        else readTop<float>(weight_path);
        for (int l = 0; l < num_layer; ++l) llama_layer_weight[l]->loadWeights(weight_path + "layers." + std::to_string(l), weight_type);
    }

    // additions
    const std::vector<LlamaLayerWeight*>& layers() const { return llama_layer_weight; }
    LayerNormWeight& outputNorm() { return out_rmsnorm_weight; }
    EmbeddingWeight& tokenEmbedding() { return pre_decoder_embedding_weight; }
    EmbeddingWeight& lmHead() { return post_decoder_embedding_weight; }
};
