/*
 * onellm_b200 — C ABI of the sm_100a kernels that replace oneLLM's kernel layer.
 *
 * Every entry point takes raw DEVICE pointers, explicit sizes and strides (in elements),
 * a dtype tag and a CUDA stream (passed as void*, 0 = legacy default stream), launches
 * asynchronously on that stream and returns an int status: 0 on success, negative on
 * failure.  Nothing throws or exits across this boundary; onellm_last_error() returns the
 * text of the calling thread's last failure.  Execution errors surface at the caller's
 * next synchronisation, as they do behind the reference's launch* functions.
 *
 * Each declaration names the reference interface it replaces (path:line inside the
 * oneLLM tree).  The C++ headers under include/onellm/ restate those interfaces with the
 * reference's own signatures on top of this ABI.
 *
 * There is no CPU fallback: without a CUDA device these functions fail with
 * ONELLM_ERR_CUDA.
 */
#ifndef ONELLM_B200_H
#define ONELLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ONELLM_API __attribute__((visibility("default")))

enum onellm_dtype { ONELLM_F32 = 0, ONELLM_F16 = 1 };

enum onellm_status {
    ONELLM_OK = 0,
    ONELLM_ERR_ARG = -1,         /* null pointer, bad size, misaligned pointer or stride */
    ONELLM_ERR_UNSUPPORTED = -2, /* shape or dtype outside what the kernels cover */
    ONELLM_ERR_CUDA = -3,        /* CUDA runtime error (message has the text) */
    ONELLM_ERR_WORKSPACE = -4,   /* caller's scratch buffer is missing or too small */
    ONELLM_ERR_IO = -5,          /* weight file missing or of the wrong size */
    ONELLM_ERR_STATE = -6,       /* call made in the wrong order (e.g. decode before prefill) */
    ONELLM_ERR_COMM = -7         /* NCCL failure or time-out */
};

/* Layout of a projection weight. */
enum onellm_wlayout {
    ONELLM_W_KN = 0, /* [K_in, N_out] row-major: the reference's layer weights */
    ONELLM_W_NK = 1  /* [N_out, K_in] row-major: tok_embeddings / output.weight ([vocab, hidden]) */
};

ONELLM_API const char* onellm_last_error(void);
ONELLM_API int onellm_abi_version(void);

/* ---------------------------------------------------------------------------------------
 * Decode-step fused masked self-attention with RoPE.
 * Replaces launchDecoderMaskedMHA / masked_MHA_kernel
 * (src/kernels/decoder_masked_attn.h:7-14, src/kernels/decoder_masked_attn.cu:136-327).
 *
 *   q [B,H,D], k and v [B,Hkv,D]: the new token's projections; *_stride_b is the element
 *     stride between batches (so the three may be views of one fused [B,H+2Hkv,D] buffer).
 *   bias_q [H*D], bias_k [Hkv*D], bias_v [Hkv*D]: may be NULL.
 *   k_cache, v_cache: ONE layer's cache; element (b, kv_head, row, d) lives at
 *     b*cs_b + kv_head*cs_h + row*cs_s + d.  The reference kernel's [S,B,Hkv,D] order and the
 *     layers' [B,Hkv,S,D] order are both expressible.
 *   step: number of rows attended, the new one included.  q and k get bias then RoPE at
 *     position rope_pos; k and v (+bias) are stored in row step-1; the output is
 *     softmax(scale * q.K^T) V over rows 0..step-1.  Query head h reads KV head h / (H/Hkv).
 *   step_dev: optional DEVICE int.  When non-NULL the kernel reads the step from it at run
 *     time (so a captured CUDA graph can be replayed as the sequence grows); `step` must
 *     then be an upper bound of that value, and the position used is
 *     *step_dev + (rope_pos - step).  The kernel reads the counter as soon as its blocks start,
 *     which under programmatic dependent launch can be while the kernel enqueued just before it
 *     is still running: the counter must have been written by work that was COMPLETE before that
 *     preceding kernel began (the model advances it in the first kernel of a step, launched with a
 *     full stream dependency).  A counter updated by the kernel directly in front of this call
 *     may be read at its old value.
 *   rot_dim, rope_base: rotary dimension and base, pairs (2i, 2i+1), angle
 *     rope_pos / rope_base^(2i/rot_dim).
 *   out [B,H,D] with batch stride out_stride_b.
 *   workspace: device scratch of at least onellm_decode_attn_workspace_bytes(B,H,D,step)
 *     bytes, 16-byte aligned; used when the rows are split across thread blocks.
 *
 * dtype F32 or F16 (F16 storage, fp32 arithmetic).  D*sizeof(T) must be one of
 * 64, 128, 256, 512 bytes.  All pointers and strides must keep rows 16-byte aligned.
 * ------------------------------------------------------------------------------------- */
ONELLM_API size_t onellm_decode_attn_workspace_bytes(int B, int H, int D, int max_step);

ONELLM_API int onellm_decode_attn(int dtype, const void* q, const void* k, const void* v,
                                  long q_stride_b, long k_stride_b, long v_stride_b,
                                  const void* bias_q, const void* bias_k, const void* bias_v,
                                  void* k_cache, void* v_cache, long cs_b, long cs_h, long cs_s,
                                  int B, int H, int Hkv, int D, int step, const int* step_dev,
                                  int rope_pos, int rot_dim, float rope_base, float scale, void* out,
                                  long out_stride_b, void* workspace, size_t workspace_bytes,
                                  void* stream);

/* onellm_decode_attn for a batch whose sequences have different lengths (what padding_offset /
 * history_length / input_length carry through the reference's context phase,
 * src/kernels/cal_paddingoffset.cu:9-32, src/kernels/qkv_bias_and_RoPE.cu:138-143, and its decode
 * kernel then drops: masked_MHA_kernel has one `step` for the whole batch,
 * src/kernels/decoder_masked_attn.cu:294).  step_offset: DEVICE int [B], values <= 0, may be NULL;
 * sequence b attends step + step_offset[b] rows, stores its new row at step + step_offset[b] - 1 and
 * rotates at rope_pos + step_offset[b].  Everything else as onellm_decode_attn; `step` (and
 * *step_dev) describe the longest sequence. */
ONELLM_API int onellm_decode_attn_ragged(int dtype, const void* q, const void* k, const void* v,
                                         long q_stride_b, long k_stride_b, long v_stride_b,
                                         const void* bias_q, const void* bias_k, const void* bias_v,
                                         void* k_cache, void* v_cache, long cs_b, long cs_h, long cs_s,
                                         int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         const int* step_offset, int rope_pos, int rot_dim,
                                         float rope_base, float scale, void* out, long out_stride_b,
                                         void* workspace, size_t workspace_bytes, void* stream);

/* onellm_decode_attn_ragged with the split-KV partials merged inside the attention kernel: one launch whatever
 * the plan (the other entry points launch a small merge kernel behind a split launch).  tickets: B * H ints of
 * device memory, zero before the first call; every call leaves them zero.  The last block of a (sequence, head
 * group) to finish merges the partials of all its splits; no block waits for another.  Same plan, bit-identical
 * results.  Measured on B200 it is no faster than the two-launch form (slower once a split launch runs several
 * waves of blocks: every block ends with a fence and an atomic), so onellm_llama_* does not use it; it is here
 * for hosts where a kernel launch costs more.  Calls that share a ticket array or a workspace must not overlap
 * on the GPU. */
ONELLM_API int onellm_decode_attn_merged(int dtype, const void* q, const void* k, const void* v,
                                         long q_stride_b, long k_stride_b, long v_stride_b,
                                         const void* bias_q, const void* bias_k, const void* bias_v,
                                         void* k_cache, void* v_cache, long cs_b, long cs_h, long cs_s,
                                         int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         const int* step_offset, int rope_pos, int rot_dim,
                                         float rope_base, float scale, void* out, long out_stride_b,
                                         void* workspace, size_t workspace_bytes, int* tickets, void* stream);

/* ---------------------------------------------------------------------------------------
 * onellm_decode_attn for callers that cannot allocate device memory.
 * No counterpart in the reference (its layers allocate scratch through BaseAllocator).
 *
 * Same arguments and results as onellm_decode_attn, without the workspace: the split-KV partials
 * go to a fixed 8 MiB array inside the library image (onellm_decode_attn_static_scratch_bytes()),
 * which every GPU that loads the library holds until the process exits.  Meant for hosts that own
 * all device memory themselves and must not, or cannot, call cudaMalloc on behalf of a kernel
 * (a server with a pool pinned at start-up, a plugin inside another framework's allocator).
 * The call performs no CUDA allocation or free of any kind.
 *
 * Limits: a shape is accepted only if its worst case, onellm_decode_attn_workspace_bytes(B, H, D,
 * step), fits the array; otherwise the call fails with ONELLM_ERR_WORKSPACE and a message naming
 * both sizes.  Llama-2-7B decode at batch 8 and 2048 rows needs 4.3 MiB by that bound.
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 * that device current): make that call before any stream capture.  All calls share the array:
 * calls that overlap on the GPU (other streams or host threads) race and must be serialised.
 * ------------------------------------------------------------------------------------- */
ONELLM_API size_t onellm_decode_attn_static_scratch_bytes(void);

ONELLM_API int onellm_decode_attn_static(int dtype, const void* q, const void* k, const void* v,
                                         long q_stride_b, long k_stride_b, long v_stride_b,
                                         const void* bias_q, const void* bias_k, const void* bias_v,
                                         void* k_cache, void* v_cache, long cs_b, long cs_h, long cs_s,
                                         int B, int H, int Hkv, int D, int step, const int* step_dev,
                                         int rope_pos, int rot_dim, float rope_base, float scale,
                                         void* out, long out_stride_b, void* stream);

/* ---------------------------------------------------------------------------------------
 * RMSNorm in place: x <- gamma * x * rsqrt(mean(x^2) + eps), x [num_tokens, hidden].
 * Replaces launchRMSNorm (src/kernels/rmsnorm_kernel.h:6-9, rmsnorm_kernel.cu:47-103).
 * gamma has the dtype of x.  hidden*sizeof(T) must be a multiple of 16.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_rmsnorm(int dtype, void* x, const void* gamma, float eps, int num_tokens,
                              int hidden, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused add-bias-residual + RMSNorm:
 *     residual    <- decoder_out + residual + bias          (bias may be NULL)
 *     decoder_out <- gamma * residual * rsqrt(mean(residual^2) + eps)
 * Replaces launchFusedAddBiasResidualRMSNorm<T>
 * (src/kernels/fused_addresidual_norm.h:4-12, fused_addresidual_norm.cu:51-141), with the
 * two outputs the decoder code expects from it (src/layers/decoder/self_decoder.cpp:50-73).
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_add_residual_rmsnorm(int dtype, void* residual, void* decoder_out,
                                           const void* bias, const void* gamma, float eps,
                                           int num_tokens, int hidden, void* stream);

/* ---------------------------------------------------------------------------------------
 * A decoder sub-block without norm kernels (F16, M <= 64, [K,N] weights).  No single counterpart
 * in the reference: it is launchFusedAddBiasResidualRMSNorm + launchLinearGemm (+ launchAct)
 * of src/layers/decoder/self_decoder.cpp:47-73 regrouped around the projections:
 *
 *   t = x . W                         (Wu == NULL)      t = silu(x . W) * (x . Wu)   (Wu != NULL)
 *   rms_eps >= 0:  both products are scaled per token by rsqrt(mean_K(x^2) + rms_eps) first, which
 *                  makes them the projection of RMSNorm(x) if the norm's gamma[k] has been multiplied
 *                  into row k of W (and Wu) beforehand; rms_eps < 0: no scaling
 *   y = t                             (resid == NULL)   y = resid + bias + t         (bias may be NULL)
 *
 * resid may be y itself (residual stream updated in place); y must not alias x.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_gemm_fused(int dtype, const void* x, const void* W, const void* Wu, void* y, int M, int N,
                                 int K, float rms_eps, const void* resid, const void* bias, void* stream);

/* ---------------------------------------------------------------------------------------
 * Projection y[M,N] = x[M,K] . W  (fp32 accumulation, no bias).
 * Replaces launchLinearGemm + cublasWrapper::Gemm
 * (src/kernels/qkv_linear.h:9-14, qkv_linear.cu:8-65, cublas_wrapper.cc:45-90).
 * w_layout selects [K,N] (layer weights) or [N,K] (LM head).  F16: tensor cores; M <= 64
 * takes the weight-streaming path, larger M the tiled path.  F32: plain fp32 arithmetic.
 * F16 constraints: [K,N] weights need K % 16 == 0 and N % 8 == 0; [N,K] weights K % 32 == 0.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_gemm(int dtype, const void* x, const void* W, void* y, int M, int N, int K,
                           int w_layout, void* stream);
/* The same with an output row stride: row t of y starts at y + t*ldy (ldy >= N).  Lets the gate and
 * the up projection of the reference's FFN (src/layers/ffn/ffn.cpp:62-64, the shared_out_buf switch
 * of qkv_linear.cu:37-40) write the two halves of one [T, 2, I] buffer.  F32 only; F16 needs ldy = N. */
ONELLM_API int onellm_gemm_ld(int dtype, const void* x, const void* W, void* y, long ldy, int M, int N, int K,
                              int w_layout, void* stream);

/* 1 if a block of the tensor-core GEMM gave up a bounded wait since the last call (the flag is cleared),
 * 0 otherwise, -1 if it cannot be read.  Such a block skips its stores: the output is then incomplete. */
/* Context-phase form of onellm_gemm_fused (any M; tcgen05 tiles): a decoder layer without norm kernels over
 * all prompt tokens at once, replacing launchLinearGemm + launchFusedAddBiasResidualRMSNorm of
 * src/layers/decoder/context_decoder.cpp:95-131 once the norm's gamma is multiplied into the weight rows.
 *   row_ss [M, ss_parts] (or NULL): partial sums whose total is the sum of squares of row m of x; the result
 *     rows are scaled by rsqrt(total / K + rms_eps), i.e. the projection of RMSNorm(x).
 *   resid [M, N] (or NULL, may be y): y = resid + bias + result.  Wu: the gate/up form, y = silu(x.W) * (x.Wu).
 *   row_ss_out [M, onellm_gemm_rows_parts(N, 0)] (or NULL): per column tile, the sum of squares of the values
 *     stored in y -- the row_ss of the projection that reads y next; every entry is written exactly once.
 * onellm_row_sumsq: out[m] = sum of squares of row m (the row_ss, with one part, of a tensor that no projection
 * produced, e.g. the embedding output). */
ONELLM_API int onellm_gemm_rows(int dtype, const void* x, const void* W, const void* Wu, void* y, int M, int N, int K,
                                const float* row_ss, int ss_parts, float rms_eps, const void* resid, const void* bias,
                                float* row_ss_out, void* stream);
ONELLM_API int onellm_gemm_rows_parts(int N, int dual);
ONELLM_API int onellm_row_sumsq(int dtype, const void* x, int rows, int cols, float* out, void* stream);
ONELLM_API int onellm_gemm_timeout_flag(void);

/* Tuning aids for the weight-streaming projections (at most 64 tokens, [K, N] weights; no counterpart in the
 * reference, whose GEMMs go to cuBLAS, src/kernels/qkv_linear.cu:8-65).  A launch is planned once per shape:
 * the K range is split over the blocks of a thread-block cluster (k_split, 1..8) and every block streams its
 * rows through a shared-memory ring of ring_depth stages.  onellm_gemm_plan_query reports the plan a shape
 * gets (dual != 0: gate/up with two weight matrices) and the thread blocks it launches;
 * onellm_gemm_plan_override forces one for every later launch of that shape in this process (k_split 0
 * removes it).  A forced plan that does not fit shared memory makes those launches fail with ONELLM_ERR_CUDA;
 * the tensor-parallel kernel onellm_p2p_gemm_allreduce_add ignores overrides. */
ONELLM_API int onellm_gemm_plan_query(int M, int N, int K, int dual, int* k_split, int* ring_depth, int* blocks);
ONELLM_API int onellm_gemm_plan_override(int N, int K, int dual, int k_split, int ring_depth);
/* Projections of [min_tokens, 64] tokens with [K, N] weights run on the tcgen05 weight-streaming kernel, fewer
 * tokens on the mma.sync one (default 33).  Sets the threshold (min_tokens >= 1; 65 or more: never) and returns
 * the value it had; min_tokens <= 0 only queries.  A tuning aid like the two calls above. */
ONELLM_API int onellm_gemm_tc_min_tokens(int min_tokens);

/* Tuning aid: whether the tcgen05 weight-streaming kernel may give a block 256 output columns instead of 128
 * (single weight, no tensor-parallel exchange, at least 512 columns; the activation tile of a stage then serves twice
 * the weight bytes).  Default 1; 0: never; 2: also for the shapes that have a tuned plan of the 128-column form
 * (for sweeps).  Returns the previous value; a negative argument only reads it. */
ONELLM_API int onellm_gemm_tc_wide(int enabled);

/* The same kind of aid for the fp16 decode attention (head size 64 / 128): forces the thread blocks per SM (1..3,
 * which fixes the depth of the per-warp rings) and / or the number of row ranges a (sequence, head) pair is split
 * into (1..16) for every later launch in this process; 0 leaves the choice to the planner. */
ONELLM_API int onellm_decode_attn_plan_override(int blocks_per_sm, int splits);


/* Gate and up projections with SwiGLU applied on the way out:
 *     out[M,I] = silu(x.Wg) * (x.Wu),   Wg, Wu [K,I]
 * Replaces the gate GEMM, up GEMM and launchAct of LLaMAFFNLayer::forward
 * (src/layers/ffn/ffn.cpp:62-66, src/kernels/activation_kernel.cu:10-32).  F16 only.  M <= 64: the
 * weight-streaming kernel with both matrices in one ring; M > 64: tensor-core tiles whose 256 accumulator
 * columns hold 128 gate columns beside the same 128 up columns, SwiGLU in the epilogue. */
ONELLM_API int onellm_gemm_swiglu(int dtype, const void* x, const void* Wg, const void* Wu, void* out,
                                  int M, int I, int K, void* stream);

/* Fused add-bias-residual RMSNorm in front of a projection (fp16, M <= 16, [K,N] weights):
 *     r = x + residual (+ bias);   residual_out = r;
 *     xn = gamma * r * rsqrt(mean(r^2) + eps);   y = xn . W      (Wu == NULL)
 *                                                y = silu(xn . W) * (xn . Wu)
 * x == NULL: r = residual (a plain RMSNorm in front of the projection; residual_out is ignored).
 * residual_out must not alias residual.  One launch replaces launchFusedAddBiasResidualRMSNorm
 * followed by launchLinearGemm(s) (and launchAct), the order of
 * src/layers/decoder/self_decoder.cpp:50-62 and src/layers/ffn/ffn.cpp:62-66. */
ONELLM_API int onellm_add_residual_rmsnorm_gemm(int dtype, const void* x, const void* residual, const void* bias,
                                                const void* gamma, float eps, void* residual_out,
                                                const void* W, const void* Wu, void* y, int M, int N, int K,
                                                void* stream);

/* Standalone SwiGLU on input [tokens, 2, I] -> out [tokens, I].
 * Replaces launchAct<T> (src/kernels/activation_kernel.h:2-3, activation_kernel.cu:10-32). */
ONELLM_API int onellm_swiglu(int dtype, const void* input, void* out, int tokens, int inter,
                             void* stream);

/* Embedding gather: out[t,:] = table[ids[t],:], ids int32 [n_tokens], table [vocab, hidden].
 * Replaces launchInputEmbedding (src/kernels/input_embedding.h:5-7, input_embedding.cu:7-40).
 * Ids outside [0, vocab) produce a zero row and set *bad_id_flag (device int, may be NULL). */
ONELLM_API int onellm_embedding(int dtype, const int* ids, void* out, const void* table, int n_tokens,
                                int hidden, int vocab, int* bad_id_flag, void* stream);

/* ---------------------------------------------------------------------------------------
 * Context phase, step 1: bias + RoPE on the packed QKV of `num_tokens` prompt tokens, K/V written
 * straight into one layer's cache.
 * Replaces launchAddFusedQKVBiasTransposeAndRoPE (src/kernels/qkv_bias_and_RoPE.h:6-14,
 * qkv_bias_and_RoPE.cu:74-207) and launchAppendKVCache (src/kernels/append_to_kvcache.h:20-26,
 * append_to_kvcache.cu:8-114) without the padded, transposed copies.
 *   qkv [num_tokens, H+2Hkv, D] packed (no padding); q heads are rotated IN PLACE; bias [(H+2Hkv)*D] or NULL.
 *   cu_seqlens [B+1] device ints: token offsets of the sequences (what launchCalPaddingoffset calls
 *     cum_seqlens, src/kernels/cal_paddingoffset.cu:9-32); history_length [B] device ints.
 *   Token i of sequence b has position history_length[b] + i (qkv_bias_and_RoPE.cu:138-143); its k
 *   (rotated) and v go to cache row (b, kv_head, position) with the strides of onellm_decode_attn.
 *   A position >= max_seq_len is not written and sets *overflow_flag (device int, may be NULL).
 * F16 or F32.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_qkv_bias_rope_kvcache(int dtype, void* qkv, const void* bias, const int* cu_seqlens,
                                            const int* history_length, void* k_cache, void* v_cache,
                                            long cs_b, long cs_h, long cs_s, int num_tokens, int B, int H,
                                            int Hkv, int D, int rot_dim, float rope_base, int max_seq_len,
                                            int* overflow_flag, void* stream);

/* ---------------------------------------------------------------------------------------
 * Context phase, step 2: causal attention of the prompt tokens over the cache.
 * Replaces launchTransposeKVCache, launchLinearStridedBatchGemm (Q.K^T and P.V),
 * launchBuildCausalMasks, launchScaleMaskAndSoftmax and launchTransposeOutRemovePadding as chained in
 * LLaMAContextAttentionLayer::forward (src/layers/attention/context_attention.cpp:134-148); no score
 * matrix and no repeated KV are materialised.
 *   q: rotated queries, token t / head h at q + t*q_ld + h*D (q_ld = (H+2Hkv)*D reads them in place
 *   from the QKV buffer); out [num_tokens, H*D].  Token i of sequence b attends cache rows
 *   0 .. history_length[b] + i of KV head h / (H/Hkv).  max_q_len = longest sequence of this call.
 * F16, D = 64 or 128.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_context_attn(int dtype, const void* q, long q_ld, const void* k_cache, const void* v_cache,
                                   long cs_b, long cs_h, long cs_s, const int* cu_seqlens,
                                   const int* history_length, int B, int max_q_len, int H, int Hkv, int D,
                                   float scale, void* out, void* stream);

/* ---------------------------------------------------------------------------------------
 * One-to-one replacements for the nine launchers of the reference's context-attention layer
 * (src/layers/attention/context_attention.cpp:101-158), for a host that keeps that sequence
 * as it is.  dtype F32 or F16; all pointers device memory unless named host_*.  New code uses
 * onellm_qkv_bias_rope_kvcache + onellm_context_attn, which need none of the buffers below.
 * ------------------------------------------------------------------------------------- */
/* launchCalPaddingoffset (src/kernels/cal_paddingoffset.h:5-10, cal_paddingoffset.cu:9-46):
 * cum_seqlens [B+1] exclusive prefix sums of seq_lens [B]; padding_offset [sum] = number of pad
 * slots in front of each real token in the [B, max_q_len] layout.  host_token_num (may be NULL)
 * receives the token count; when given, the call synchronises the stream.  1 <= B <= 64. */
ONELLM_API int onellm_cal_padding_offset(int* padding_offset, int* cum_seqlens, const int* seq_lens, int B,
                                         int max_q_len, int* host_token_num, void* stream);
/* launchBuildCausalMasks (src/kernels/build_casual_mask.h:4-9, build_casual_mask.cu:27-60):
 * mask [B, max_q_len, max_k_len] of 1/0.  attend_history = 0 reproduces the shipped predicate
 * (build_casual_mask.cu:40-43), which also zeroes the history columns; 1 keeps them. */
ONELLM_API int onellm_build_causal_mask(int dtype, void* mask, const int* q_lens, const int* k_lens, int max_q_len,
                                        int max_k_len, int B, int attend_history, void* stream);
/* launchAddFusedQKVBiasTransposeAndRoPE (src/kernels/qkv_bias_and_RoPE.h:6-14,
 * qkv_bias_and_RoPE.cu:74-207): packed QKV [num_tokens, H+2*Hkv, D] (+ bias [H+2*Hkv, D], may be
 * NULL) -> q_buf [B, H, seq_len, D], k_buf / v_buf [B, Hkv, seq_len, D]; interleaved-pair rotation
 * of q and k at position history_length[b] + local index.  Pad rows are left untouched. */
ONELLM_API int onellm_qkv_bias_rope_transpose(int dtype, void* q_buf, void* k_buf, void* v_buf, const void* QKV,
                                              const void* bias, const int* padding_offset,
                                              const int* history_length, int B, int seq_len, int num_tokens, int H,
                                              int Hkv, int D, int rotary_dim, float rope_base, void* stream);
/* launchAppendKVCache (src/kernels/append_to_kvcache.h:20-26, append_to_kvcache.cu:8-114), one
 * layer, one of K or V: src [B, Hkv, max_q_len, D] -> dst [B, Hkv, max_seq_len, D] at rows
 * history_length[b] + [0, cur_query_length[b]).  Rows beyond max_seq_len are dropped and
 * *overflow_flag (device int, may be NULL) is set to 1; the reference writes out of bounds. */
ONELLM_API int onellm_append_kv_cache(int dtype, void* dst, const void* src, const int* cur_query_length,
                                      const int* history_length, int B, int Hkv, int max_q_len, int max_seq_len,
                                      int D, int* overflow_flag, void* stream);
/* launchTransposeKVCache (src/kernels/transpose_kernel.h:5-11, transpose_kernel.cu:7-88), one
 * layer: src [B, Hkv, max_seq_len, D] -> dst [B, H, max_k_len, D], query head h reads KV head
 * h / (H/Hkv), rows [0, context_length[b]); the rest of dst is left untouched. */
ONELLM_API int onellm_repeat_kv(int dtype, void* dst, const void* src, const int* context_length, int B, int H,
                                int Hkv, int max_k_len, int max_seq_len, int D, void* stream);
/* launchLinearStridedBatchGemm (src/kernels/qkv_linear.h:16-20, qkv_linear.cu:67-120):
 * C[b] = op(A[b]) . op(B[b]) over `batch` row-major matrices, A [m,k] ([k,m] when trans_a),
 * B [k,n] ([n,k] when trans_b), fp32 accumulation.  A plain tiled kernel: the context phase of
 * this library never materialises these products. */
ONELLM_API int onellm_batched_gemm(int dtype, const void* A, const void* Bm, void* Cm, int batch, int m, int n, int k,
                                   int trans_a, int trans_b, void* stream);
/* cublasWrapper::Gemm / cublasWrapper::stridedBatchedGemm (src/kernels/cublas_wrapper.h:34-66,
 * cublas_wrapper.cc:45-147) with the BLAS convention those take: column-major operands,
 * C[b] (m x n, ldc) = alpha * op(A[b]) . op(B[b]) + beta * C[b], element strides between batches.
 * batch = 1 is the plain Gemm.  A plain tiled kernel for hosts that call the wrapper directly. */
ONELLM_API int onellm_gemm_strided_batched(int dtype, int trans_a, int trans_b, int m, int n, int k, const void* A,
                                           int lda, long stride_a, const void* Bm, int ldb, long stride_b, void* Cm,
                                           int ldc, long stride_c, int batch, float alpha, float beta, void* stream);
/* launchScaleMaskAndSoftmax (src/kernels/attn_softmax_kernel.h:5-8, attn_softmax_kernel.cu:45-176):
 * attn_score [B, H, q_len, k_len] = softmax over the columns where mask [B, q_len, k_len] != 0 of
 * scale * qk; masked columns and fully masked rows give 0. */
ONELLM_API int onellm_scale_mask_softmax(int dtype, void* attn_score, const void* qk, const void* mask, int B, int H,
                                         int q_len, int k_len, float scale, void* stream);
/* launchTransposeOutRemovePadding (src/kernels/fused_transpose_reshape_remv_pad.h:5-6,
 * fused_transpose_reshape_remv_pad.cu:5-51): src [B, H, S, D] -> dst [num_tokens, H*D]. */
ONELLM_API int onellm_transpose_remove_padding(int dtype, void* dst, const void* src, const int* padding_offset,
                                               int num_tokens, int B, int S, int H, int D, void* stream);

/* ---------------------------------------------------------------------------------------
 * Row-wise top-K of logits [rows, vocab] (F32 or F16), values sorted descending, ties to
 * the lower column.  out_val float [rows,K], out_id int32 [rows,K] (column index, or
 * row*vocab + column when global_ids != 0 as the reference's beam-search kernel emits).
 * Generalises launchTopKforBeamSearch (src/kernels/beamsearch_topK.h:35-38,
 * beamsearch_topK.cu:20-119), whose K is fixed at 2.  1 <= K <= 64.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_topk(int dtype, const void* logits, int rows, int vocab, int K, float* out_val,
                           int* out_id, int global_ids, void* stream);

/* ---------------------------------------------------------------------------------------
 * Top-K sampling from sorted candidates.
 * Replaces launchSampling / SamplingKernel (src/kernels/topK_sampling.h:9-14,
 * topK_sampling.cu:6-70): w_i = exp((val_i - val_0)/temperature); u = curand_uniform of an
 * XORWOW state initialised with (seed = rng_step, subsequence = row, offset = 0); walk the
 * candidates subtracting w_i from u*sum(w) until it goes negative; id = topk_id % vocab_size;
 * seqlen[b] += !finished[b]; finished[b] = (id == end_id).
 * literal_walk != 0 reproduces the shipped walk (subtracts w_0 every time).
 * topk_val is NOT modified (the reference overwrites it with the weights).
 * seqlen / finished (bool bytes) may be NULL.  u_out (float [B], may be NULL) receives the
 * uniform draws.  rng_step_dev: optional DEVICE int read at run time in place of rng_step
 * (for replay inside a captured CUDA graph); like step_dev of onellm_decode_attn it is read when
 * the kernel starts, so it must not be written by the kernel enqueued directly before this call.
 * ------------------------------------------------------------------------------------- */
ONELLM_API int onellm_topk_sample(const int* topk_id, const float* topk_val, int B, int K,
                                  float temperature, int rng_step, const int* rng_step_dev,
                                  int vocab_size, int end_id, int literal_walk, int* output_id,
                                  int* seqlen, unsigned char* finished, float* u_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * One-shot all-reduce over peer memory fused with the residual add, for tensor-parallel decode:
 *
 *     resid[i] <- resid[i] + bias[i % row_len] + sum over ranks of partial_r[i]          (F16)
 *
 * replacing ncclAllReduce + the add of launchFusedAddBiasResidualRMSNorm after o_proj and down_proj
 * when the reference's decoder (src/layers/decoder/self_decoder.cpp:47-73) runs tensor parallel.
 * One process per GPU on one node.  Every rank creates a communicator (which allocates its two send
 * buffers and its flags), the 64-byte handles are exchanged by the host (any transport) and passed,
 * in rank order, to onellm_p2p_connect.  Per call every rank first lets a kernel write its partial
 * into onellm_p2p_send_buffer(which) on `stream`, then calls onellm_p2p_allreduce_add with the same
 * `which`, n_elems and row_len on every rank; the two buffers must be used alternately (0, 1, 0, 1, ...),
 * which keeps a rank from overwriting data a slower peer is still reading.  Sums are taken in rank
 * order: every rank computes bit-identical results.  Waits for peers are bounded (about a second);
 * onellm_p2p_error returns 1 once one has run out (the data of that call is then undefined).
 * ------------------------------------------------------------------------------------- */
#define ONELLM_P2P_HANDLE_BYTES 64
typedef struct onellm_p2p onellm_p2p;
ONELLM_API int onellm_p2p_create(int rank, int world, size_t max_elems, onellm_p2p** out);
ONELLM_API int onellm_p2p_handle(onellm_p2p* comm, void* handle64);
ONELLM_API int onellm_p2p_connect(onellm_p2p* comm, const void* handles /* world * 64 bytes, rank order */);
ONELLM_API void* onellm_p2p_send_buffer(onellm_p2p* comm, int which);
ONELLM_API int onellm_p2p_allreduce_add(onellm_p2p* comm, int dtype, int which, void* resid, const void* bias,
                                        int n_elems, int row_len, void* stream);
/* Projection and all-reduce in ONE kernel (F16, 1 <= M <= 64, [K,N] weights):
 *     resid[M,N] <- resid + bias + sum over ranks of (x[M,K] . W_r),   W_r = this rank's rows of the weight.
 * The block that has finished two output elements pushes them to every peer at once and gathers the peers'
 * values of the same elements, so the link latency hides behind the rest of the projection.  Same rules as
 * above: identical calls on every rank, receive buffers 0 and 1 alternately, bounded waits.  Must not be
 * mixed with a concurrent onellm_p2p_allreduce_add on the same `which`. */
ONELLM_API int onellm_p2p_gemm_allreduce_add(onellm_p2p* comm, int dtype, int which, const void* x, const void* W,
                                             void* resid, const void* bias, int M, int N, int K, void* stream);

/* The exchange inside onellm_p2p_gemm_allreduce_add has two forms with the same arithmetic and the same bits.
 * One-shot: every rank sends its partial of an element to every peer and adds what it receives (one hop, world - 1
 * copies of the message per rank on the wire).  Two-shot: token row t belongs to rank t % world; partials go to
 * the owner only, which adds them, the residual and the bias and sends the finished value to everybody (two hops,
 * 2 (world - 1) / world of one message per rank).  The two-shot form is taken when the one-shot form would put
 * at least `bytes` on the wire per rank, (world - 1) * M * N * 4, and there are more than two ranks (default
 * 3 MiB: the 64-token messages of a 13B model on 4 or 8 ranks, not a batch of 8).  Returns the previous threshold;
 * a negative argument only reads it; 0 = always two-shot, on two ranks too.  Process-wide; every rank must use the
 * same value. */
ONELLM_API long long onellm_p2p_two_shot_bytes(long long bytes);

ONELLM_API int onellm_p2p_error(onellm_p2p* comm);
ONELLM_API void onellm_p2p_destroy(onellm_p2p* comm);

/* ---------------------------------------------------------------------------------------
 * LLaMA model: weights, KV cache and the generation loop (host side in C++).
 * Fills in the model class the reference leaves empty (src/models/llama/llama.h, outline in
 * src/models/llama/llama.cpp:1-50) with the kernel order of LlamaSelfDecoder::forward
 * (src/layers/decoder/self_decoder.cpp:15-78).  fp16 weights and activations.
 * ------------------------------------------------------------------------------------- */
typedef struct onellm_llama onellm_llama;

typedef struct onellm_llama_config {
    int num_layers, hidden, head_num, kv_head_num, head_size, inter_size, vocab_size;
    int max_seq_len, max_batch; /* KV cache is [L, max_batch, kv_head_num/tp, max_seq_len, head_size] */
    float rope_base;            /* <= 0: 10000 */
    int rot_dim;                /* <= 0: head_size */
    float rms_eps;              /* <= 0: 1e-5 */
    int bos_id, eos_id;
    int attn_bias;              /* qkv / o biases present (src/weights/llama/layer_weights.cc:26-29) */
    int tp_rank, tp_size;       /* tensor parallel slice held by this process */
} onellm_llama_config;

ONELLM_API int onellm_llama_create(const onellm_llama_config* cfg, onellm_llama** out);
/* The configuration from the config.ini the reference's converter writes next to the weight files
 * (tools/FT_convert_weight_to_bin_final.py:43-64, section [llama]: head_num, kv_head_num, hidden_size, head_size,
 * inter_size, num_layer, vocab_size, bos_token_id, eos_token_id, weight_data_type, max_position_embeddings,
 * rope_theta, rms_norm_eps, attention_bias, top_k).  onellm_llama_config_from_ini fills the fields the file names
 * and leaves max_batch, tp_rank and tp_size as the caller set them (max_seq_len too unless it is <= 0, in which
 * case it becomes max_position_embeddings); *top_k (may be NULL) receives the file's top_k.  No GPU is touched.
 * onellm_llama_create_from_ini does that, creates the model and sets its sampling to the file's top_k.
 * Missing file, section or required key, or a malformed value: ONELLM_ERR_IO with the key in the message. */
ONELLM_API int onellm_llama_config_from_ini(const char* path, onellm_llama_config* cfg, int* top_k);
ONELLM_API int onellm_llama_create_from_ini(const char* path, int max_batch, int max_seq_len, int tp_rank, int tp_size,
                                            onellm_llama** out);
ONELLM_API void onellm_llama_destroy(onellm_llama* m);
ONELLM_API size_t onellm_llama_device_bytes(const onellm_llama* m);
ONELLM_API void* onellm_llama_stream(onellm_llama* m);

/* Weights from the reference's .bin files: `weight_path` is the prefix the reference's
 * LlamaWeight::loadWeights takes (src/weights/llama/llama_weights.cc:36-46): files
 * <p>.norm.weight, <p>.tok_embeddings.weight, <p>.output.weight,
 * <p>layers.<l>.{attention_norm,ffn_norm}.weight, .attention.w_qkv.weight, .attention.wo.weight,
 * .feed_forward.{w1,w3,w2}.weight (+ .attention.w_qkv.bias / .attention.wo.bias).  fp32 or fp16
 * files; each rank keeps its tensor-parallel slice.  Missing / wrongly sized file: ONELLM_ERR_IO. */
ONELLM_API int onellm_llama_load_weights(onellm_llama* m, const char* weight_path);
/* Random weights ~N(0, std), gammas 1, generated on the device; identical for every tp_size. */
ONELLM_API int onellm_llama_init_random(onellm_llama* m, uint64_t seed, float std);

/* Tensor parallel: rank 0 creates the id, every rank passes the same 128 bytes. */
ONELLM_API int onellm_nccl_unique_id(void* id128);
ONELLM_API int onellm_llama_init_comm(onellm_llama* m, const void* id128);

ONELLM_API int onellm_llama_set_sampling(onellm_llama* m, int top_k, float temperature, int literal_walk);
ONELLM_API int onellm_llama_set_graphs(onellm_llama* m, int enabled);
/* Tensor parallel over peer memory instead of NCCL for the decode step (batch * hidden small): every rank
 * calls onellm_llama_p2p_handle, the host exchanges the handles, every rank calls onellm_llama_p2p_connect
 * with all of them in rank order.  The context phase keeps using NCCL (onellm_llama_init_comm). */
ONELLM_API int onellm_llama_p2p_handle(onellm_llama* m, void* handle64);
ONELLM_API int onellm_llama_p2p_connect(onellm_llama* m, const void* handles);
ONELLM_API int onellm_llama_p2p_error(onellm_llama* m);
/* Tensor parallel with peer memory connected: which exchange the decode step uses.  peer_memory != 0 (the
 * default after onellm_llama_p2p_connect): the projections reduce over peer memory in their own epilogue;
 * 0: ncclAllReduce on the model's stream, as the context phase does.  Both compute the sum the tensor-parallel
 * run of src/layers/decoder/self_decoder.cpp:47-73 needs behind o_proj and down_proj; the switch lets a caller
 * (the benchmark's result check) run the same steps both ways.  Every rank must choose the same. */
ONELLM_API int onellm_llama_set_tp_exchange(onellm_llama* m, int peer_memory);
/* The uniform draws of the last sampling launch (host_u: max_batch floats) and the step counter they were
 * seeded with: row b drew curand_uniform of curand_init(step, b, 0), the generator of src/kernels/topK_sampling.cu:29-30.
 * The engine takes the skip-ahead to sub-sequence b from a table built (and checked against curand_init) when the
 * model was created; *table_in_use (may be NULL) says whether that table passed its check.  host_step may be
 * NULL.  Waits for the model's stream. */
ONELLM_API int onellm_llama_last_draws(onellm_llama* m, float* host_u, int* host_step, int* table_in_use);
/* 1: run the context phase one position at a time through the decode kernels (cross-check path);
 * 0 (default): all prompt tokens at once through the context-phase kernels; 2: the same with the norm kernels
 * kept between the projections on one GPU too (what tensor-parallel runs always do; comparison). */
ONELLM_API int onellm_llama_set_prefill_by_decode(onellm_llama* m, int enabled);

/* Context phase for `batch` prompts of equal length (host ids [batch, prompt_len]); resets the
 * sequence state.  host_first_ids (may be NULL) receives the first generated token per prompt. */
ONELLM_API int onellm_llama_prefill(onellm_llama* m, const int* host_ids, int batch, int prompt_len,
                                    int* host_first_ids);
/* Prompts of different lengths (the ragged batch of src/layers/decoder/context_decoder.cpp:36-134:
 * padding_offset / input_length): host_ids holds the prompts packed one after the other, lens[b]
 * tokens each.  Decoding then continues with onellm_llama_decode_step as after onellm_llama_prefill;
 * every sequence keeps its own length and positions.  onellm_llama_get_state reports the longest. */
ONELLM_API int onellm_llama_prefill_ragged(onellm_llama* m, const int* host_ids, const int* lens, int batch,
                                           int* host_first_ids);
/* A further turn of the same `batch` sequences: n_new more tokens each (host ids [batch, n_new]) behind
 * the positions already in the KV cache, through the context-phase kernels with history_length =
 * the current length (the multi-turn case of src/layers/decoder/context_decoder.cpp:36-134).
 * host_first_ids (may be NULL) receives the next generated token per sequence. */
ONELLM_API int onellm_llama_extend(onellm_llama* m, const int* host_ids, int n_new, int* host_first_ids);
/* Declares cur_len positions of `batch` sequences as already present in the KV cache and host_ids
 * [batch] as the next input tokens (resume on a cache filled elsewhere; profiling without prefill). */
ONELLM_API int onellm_llama_seek(onellm_llama* m, int batch, int cur_len, const int* host_ids);
/* One generated token per sequence.  host_in_ids (may be NULL: use the previous step's samples)
 * are the tokens to feed; host_out_ids (may be NULL: stay asynchronous) receives the samples. */
ONELLM_API int onellm_llama_decode_step(onellm_llama* m, const int* host_in_ids, int* host_out_ids);
ONELLM_API int onellm_llama_sync(onellm_llama* m);
/* prefill + n_new - 1 decode steps; host_out [batch, n_new]. */
ONELLM_API int onellm_llama_generate(onellm_llama* m, const int* host_prompt, int batch, int prompt_len,
                                     int n_new, int* host_out);
/* Logits of the last step as float [batch, vocab_size] on the host. */
ONELLM_API int onellm_llama_get_logits(onellm_llama* m, float* host_logits);
ONELLM_API int onellm_llama_get_state(onellm_llama* m, int* cur_len, long* kernel_launches, int* host_seqlen,
                                      unsigned char* host_finished);
ONELLM_API int onellm_llama_kv_cache(onellm_llama* m, int layer, void** k_cache, void** v_cache);

#ifdef __cplusplus
}
#endif
#endif /* ONELLM_B200_H */
