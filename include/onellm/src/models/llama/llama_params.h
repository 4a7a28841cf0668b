// Drop-in for src/models/llama/llama_params.h of oneLLM (:2-15).
#pragma once

// fixed per model
struct LLaMAAttentionStaticParams {
    int rotary_embedding_dim;
    float rotary_embedding_base;
    int max_position_embeddings;
    bool use_dynamic_ntk;
};

// per forward call
struct LLaMAAttentionDynParams {
    int batch_size;
    int num_tokens;
    int max_q_len;
    int max_k_len;
    int num_layers;
};
