// Drop-in for src/kernels/cal_paddingoffset.h of oneLLM (:5-10, cal_paddingoffset.cu:9-46).
// *h_token_num is valid on return (the reference copies it out before its kernel has finished).
#pragma once
#include "src/utils/macro.h"

inline void launchCalPaddingoffset(int* h_pinned_token_num, int* h_token_num, int* padding_offset, int* cum_seqlens,
                                   const int* seq_lens, const int batch_size, const int max_q_len)
{
    int total = 0;
    ONELLM_B200_CALL(onellm_cal_padding_offset(padding_offset, cum_seqlens, seq_lens, batch_size, max_q_len, &total, nullptr));
    if (h_pinned_token_num) *h_pinned_token_num = total;
    if (h_token_num) *h_token_num = total;
}
