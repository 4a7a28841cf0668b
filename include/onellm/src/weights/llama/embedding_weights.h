// Drop-in for src/weights/llama/embedding_weights.h of oneLLM (:1-3): [vocab, hidden] table.
#pragma once
struct EmbeddingWeight {
    float* emb_table = nullptr;
};
