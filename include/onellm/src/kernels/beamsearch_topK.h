// Drop-in for src/kernels/beamsearch_topK.h of oneLLM (:35-38, beamsearch_topK.cu:85-119): for each of
// batch_size items, the 2 largest of its 2 * vocab_size candidates (beam width 2), ids as offsets
// into probs.  The workspace keeps the reference's plan (:91-99):
//   float vals[B*2*8*2] | int ids[B*2*8*2] | float final_vals[B*2] | int final_ids[B*2]
// of which only the two final blocks are written here (one pass, no intermediate candidates).
#pragma once
#include "src/utils/macro.h"

inline void launchTopKforBeamSearch(const float* probs, const int batch_size, const int vocab_size, float* topk_workspace)
{
    constexpr int kBeam = 2, kBlocksPerBeam = 8;
    const size_t stage = (size_t)batch_size * kBeam * kBlocksPerBeam * kBeam;
    float* final_vals = topk_workspace + 2 * stage;
    int* final_ids = reinterpret_cast<int*>(final_vals + (size_t)batch_size * kBeam);
    ONELLM_B200_CALL(onellm_topk(ONELLM_F32, probs, batch_size, kBeam * vocab_size, kBeam, final_vals, final_ids, /*global_ids=*/1, nullptr));
}
