"""onellm_b200: sm_100a kernels and a LLaMA decode engine behind oneLLM's kernel interface.

This module is a thin ctypes binding of ``libonellm_b200.so`` (see ``include/onellm_b200.h``)
for the tests and the benchmark.  It does no arithmetic itself and has no fallback: if the
library is missing, or a call fails, it raises.  Device buffers are passed as integer
addresses (``torch.Tensor.data_ptr()``); the caller owns them.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libonellm_b200.so")

F32, F16 = 0, 1
W_KN, W_NK = 0, 1

_lib = None


class OnellmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"onellm_b200 status {status}: {message}")
        self.status = status


class LlamaConfig(C.Structure):
    _fields_ = [
        ("num_layers", C.c_int), ("hidden", C.c_int), ("head_num", C.c_int), ("kv_head_num", C.c_int),
        ("head_size", C.c_int), ("inter_size", C.c_int), ("vocab_size", C.c_int),
        ("max_seq_len", C.c_int), ("max_batch", C.c_int),
        ("rope_base", C.c_float), ("rot_dim", C.c_int), ("rms_eps", C.c_float),
        ("bos_id", C.c_int), ("eos_id", C.c_int), ("attn_bias", C.c_int),
        ("tp_rank", C.c_int), ("tp_size", C.c_int),
    ]


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OnellmError(-100, f"{LIB_PATH} is missing: run `python -m onellm_b200.build` "
                                    "(there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        l.onellm_last_error.restype = C.c_char_p
        l.onellm_decode_attn_workspace_bytes.restype = C.c_size_t
        l.onellm_decode_attn_static_scratch_bytes.restype = C.c_size_t
        l.onellm_llama_device_bytes.restype = C.c_size_t
        l.onellm_llama_stream.restype = C.c_void_p
        l.onellm_llama_destroy.restype = None
        _lib = l
    return _lib


def _check(rc):
    if rc != 0:
        raise OnellmError(rc, lib().onellm_last_error().decode())


def _p(x):
    """Device/host address -> c_void_p (None -> NULL)."""
    if x is None:
        return C.c_void_p(0)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))


def _stream(stream):
    if stream is None:
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return C.c_void_p(int(stream))


def decode_attn_workspace_bytes(B, H, D, max_step):
    return int(lib().onellm_decode_attn_workspace_bytes(C.c_int(B), C.c_int(H), C.c_int(D), C.c_int(max_step)))


def decode_attn(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache,
                cs_b, cs_h, cs_s, B, H, Hkv, D, step, rope_pos, rot_dim, rope_base, scale, out, out_stride_b,
                workspace, workspace_bytes, step_dev=None, stream=None):
    _check(lib().onellm_decode_attn(
        C.c_int(dtype), _p(q), _p(k), _p(v), C.c_long(q_stride_b), C.c_long(k_stride_b), C.c_long(v_stride_b),
        _p(bias_q), _p(bias_k), _p(bias_v), _p(k_cache), _p(v_cache), C.c_long(cs_b), C.c_long(cs_h),
        C.c_long(cs_s), C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(step), _p(step_dev),
        C.c_int(rope_pos), C.c_int(rot_dim), C.c_float(rope_base), C.c_float(scale), _p(out),
        C.c_long(out_stride_b), _p(workspace), C.c_size_t(workspace_bytes), _stream(stream)))


def decode_attn_ragged(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache,
                       cs_b, cs_h, cs_s, B, H, Hkv, D, step, step_offset, rope_pos, rot_dim, rope_base, scale, out,
                       out_stride_b, workspace, workspace_bytes, step_dev=None, stream=None):
    """decode_attn with a device int [B] of per-sequence offsets (<= 0) to `step`."""
    _check(lib().onellm_decode_attn_ragged(
        C.c_int(dtype), _p(q), _p(k), _p(v), C.c_long(q_stride_b), C.c_long(k_stride_b), C.c_long(v_stride_b),
        _p(bias_q), _p(bias_k), _p(bias_v), _p(k_cache), _p(v_cache), C.c_long(cs_b), C.c_long(cs_h),
        C.c_long(cs_s), C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(step), _p(step_dev),
        _p(step_offset), C.c_int(rope_pos), C.c_int(rot_dim), C.c_float(rope_base), C.c_float(scale), _p(out),
        C.c_long(out_stride_b), _p(workspace), C.c_size_t(workspace_bytes), _stream(stream)))


def decode_attn_merged(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache,
                       cs_b, cs_h, cs_s, B, H, Hkv, D, step, step_offset, rope_pos, rot_dim, rope_base, scale, out,
                       out_stride_b, workspace, workspace_bytes, tickets, step_dev=None, stream=None):
    """decode_attn_ragged in one launch: the last block of each (sequence, head group) merges the splits.
    `tickets`: device int [B * H], zero before the first call (every call leaves it zero)."""
    _check(lib().onellm_decode_attn_merged(
        C.c_int(dtype), _p(q), _p(k), _p(v), C.c_long(q_stride_b), C.c_long(k_stride_b), C.c_long(v_stride_b),
        _p(bias_q), _p(bias_k), _p(bias_v), _p(k_cache), _p(v_cache), C.c_long(cs_b), C.c_long(cs_h),
        C.c_long(cs_s), C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(step), _p(step_dev),
        _p(step_offset), C.c_int(rope_pos), C.c_int(rot_dim), C.c_float(rope_base), C.c_float(scale), _p(out),
        C.c_long(out_stride_b), _p(workspace), C.c_size_t(workspace_bytes), _p(tickets), _stream(stream)))


def gemm_tc_wide(enabled=-1):
    """Tuning aid: 256-column blocks in the tcgen05 weight-streaming kernel (default on); returns the previous setting."""
    return int(lib().onellm_gemm_tc_wide(C.c_int(int(enabled))))


def decode_attn_plan_override(blocks_per_sm=0, splits=0):
    """Tuning aid: fixes the tensor-core decode attention's blocks per SM (1..3) and split count (1..16); 0 = planner."""
    _check(lib().onellm_decode_attn_plan_override(C.c_int(blocks_per_sm), C.c_int(splits)))


def decode_attn_static(dtype, q, k, v, q_stride_b, k_stride_b, v_stride_b, bias_q, bias_k, bias_v, k_cache, v_cache,
                       cs_b, cs_h, cs_s, B, H, Hkv, D, step, rope_pos, rot_dim, rope_base, scale, out, out_stride_b,
                       step_dev=None, stream=None):
    """decode_attn with the split-KV scratch taken from the library's built-in array: for hosts that
    cannot allocate device memory.  Calls sharing the GPU must not overlap (one shared array)."""
    _check(lib().onellm_decode_attn_static(
        C.c_int(dtype), _p(q), _p(k), _p(v), C.c_long(q_stride_b), C.c_long(k_stride_b), C.c_long(v_stride_b),
        _p(bias_q), _p(bias_k), _p(bias_v), _p(k_cache), _p(v_cache), C.c_long(cs_b), C.c_long(cs_h),
        C.c_long(cs_s), C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(step), _p(step_dev),
        C.c_int(rope_pos), C.c_int(rot_dim), C.c_float(rope_base), C.c_float(scale), _p(out),
        C.c_long(out_stride_b), _stream(stream)))


def rmsnorm(dtype, x, gamma, eps, num_tokens, hidden, stream=None):
    _check(lib().onellm_rmsnorm(C.c_int(dtype), _p(x), _p(gamma), C.c_float(eps), C.c_int(num_tokens),
                                C.c_int(hidden), _stream(stream)))


def add_residual_rmsnorm(dtype, residual, decoder_out, bias, gamma, eps, num_tokens, hidden, stream=None):
    _check(lib().onellm_add_residual_rmsnorm(C.c_int(dtype), _p(residual), _p(decoder_out), _p(bias), _p(gamma),
                                             C.c_float(eps), C.c_int(num_tokens), C.c_int(hidden),
                                             _stream(stream)))


def gemm(dtype, x, W, y, M, N, K, w_layout=W_KN, stream=None):
    _check(lib().onellm_gemm(C.c_int(dtype), _p(x), _p(W), _p(y), C.c_int(M), C.c_int(N), C.c_int(K),
                             C.c_int(w_layout), _stream(stream)))


def gemm_fused(dtype, x, W, Wu, y, M, N, K, rms_eps=-1.0, resid=None, bias=None, stream=None):
    _check(lib().onellm_gemm_fused(C.c_int(dtype), _p(x), _p(W), _p(Wu), _p(y), C.c_int(M), C.c_int(N), C.c_int(K),
                                   C.c_float(rms_eps), _p(resid), _p(bias), _stream(stream)))


def gemm_swiglu(dtype, x, Wg, Wu, out, M, I, K, stream=None):
    _check(lib().onellm_gemm_swiglu(C.c_int(dtype), _p(x), _p(Wg), _p(Wu), _p(out), C.c_int(M), C.c_int(I),
                                    C.c_int(K), _stream(stream)))


def add_residual_rmsnorm_gemm(dtype, x, residual, bias, gamma, eps, residual_out, W, Wu, y, M, N, K, stream=None):
    _check(lib().onellm_add_residual_rmsnorm_gemm(C.c_int(dtype), _p(x), _p(residual), _p(bias), _p(gamma),
                                                  C.c_float(eps), _p(residual_out), _p(W), _p(Wu), _p(y), C.c_int(M),
                                                  C.c_int(N), C.c_int(K), _stream(stream)))


def gemm_plan_query(M, N, K, dual=False):
    """(k_split, ring_depth, blocks) of the launch plan of a weight-streaming projection."""
    ks, nst, blocks = C.c_int(0), C.c_int(0), C.c_int(0)
    _check(lib().onellm_gemm_plan_query(C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(1 if dual else 0), C.byref(ks),
                                        C.byref(nst), C.byref(blocks)))
    return ks.value, nst.value, blocks.value


def gemm_plan_override(N, K, dual, k_split, ring_depth=12):
    """Forces the launch plan of a projection shape (k_split 0 removes the override)."""
    _check(lib().onellm_gemm_plan_override(C.c_int(N), C.c_int(K), C.c_int(1 if dual else 0), C.c_int(k_split),
                                           C.c_int(ring_depth)))


def gemm_tc_min_tokens(min_tokens=0):
    """Sets (min_tokens >= 1) or queries the token count from which projections use the tcgen05 kernel."""
    return int(lib().onellm_gemm_tc_min_tokens(C.c_int(min_tokens)))


def gemm_rows(dtype, x, W, Wu, y, M, N, K, row_ss=None, ss_parts=0, rms_eps=1e-5, resid=None, bias=None, row_ss_out=None, stream=None):
    _check(lib().onellm_gemm_rows(C.c_int(dtype), _p(x), _p(W), _p(Wu), _p(y), C.c_int(M), C.c_int(N), C.c_int(K), _p(row_ss),
                                  C.c_int(ss_parts), C.c_float(rms_eps), _p(resid), _p(bias), _p(row_ss_out), _stream(stream)))


def gemm_rows_parts(N, dual=False):
    return int(lib().onellm_gemm_rows_parts(C.c_int(N), C.c_int(1 if dual else 0)))


def row_sumsq(dtype, x, rows, cols, out, stream=None):
    _check(lib().onellm_row_sumsq(C.c_int(dtype), _p(x), C.c_int(rows), C.c_int(cols), _p(out), _stream(stream)))


def swiglu(dtype, inp, out, tokens, inter, stream=None):
    _check(lib().onellm_swiglu(C.c_int(dtype), _p(inp), _p(out), C.c_int(tokens), C.c_int(inter),
                               _stream(stream)))


def embedding(dtype, ids, out, table, n_tokens, hidden, vocab, bad_id_flag=None, stream=None):
    _check(lib().onellm_embedding(C.c_int(dtype), _p(ids), _p(out), _p(table), C.c_int(n_tokens),
                                  C.c_int(hidden), C.c_int(vocab), _p(bad_id_flag), _stream(stream)))


def qkv_bias_rope_kvcache(dtype, qkv, bias, cu_seqlens, history_length, k_cache, v_cache, cs_b, cs_h, cs_s, num_tokens,
                          B, H, Hkv, D, rot_dim, rope_base, max_seq_len, overflow_flag=None, stream=None):
    _check(lib().onellm_qkv_bias_rope_kvcache(C.c_int(dtype), _p(qkv), _p(bias), _p(cu_seqlens), _p(history_length),
                                              _p(k_cache), _p(v_cache), C.c_long(cs_b), C.c_long(cs_h), C.c_long(cs_s),
                                              C.c_int(num_tokens), C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D),
                                              C.c_int(rot_dim), C.c_float(rope_base), C.c_int(max_seq_len),
                                              _p(overflow_flag), _stream(stream)))


def context_attn(dtype, q, q_ld, k_cache, v_cache, cs_b, cs_h, cs_s, cu_seqlens, history_length, B, max_q_len, H, Hkv, D,
                 scale, out, stream=None):
    _check(lib().onellm_context_attn(C.c_int(dtype), _p(q), C.c_long(q_ld), _p(k_cache), _p(v_cache), C.c_long(cs_b),
                                     C.c_long(cs_h), C.c_long(cs_s), _p(cu_seqlens), _p(history_length), C.c_int(B),
                                     C.c_int(max_q_len), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_float(scale), _p(out),
                                     _stream(stream)))


def cal_padding_offset(padding_offset, cum_seqlens, seq_lens, B, max_q_len, want_token_num=True, stream=None):
    n = C.c_int(0)
    _check(lib().onellm_cal_padding_offset(_p(padding_offset), _p(cum_seqlens), _p(seq_lens), C.c_int(B), C.c_int(max_q_len),
                                           C.byref(n) if want_token_num else None, _stream(stream)))
    return n.value if want_token_num else None


def build_causal_mask(dtype, mask, q_lens, k_lens, max_q_len, max_k_len, B, attend_history=False, stream=None):
    _check(lib().onellm_build_causal_mask(C.c_int(dtype), _p(mask), _p(q_lens), _p(k_lens), C.c_int(max_q_len),
                                          C.c_int(max_k_len), C.c_int(B), C.c_int(1 if attend_history else 0), _stream(stream)))


def qkv_bias_rope_transpose(dtype, q_buf, k_buf, v_buf, QKV, bias, padding_offset, history_length, B, seq_len, num_tokens,
                            H, Hkv, D, rot_dim, rope_base, stream=None):
    _check(lib().onellm_qkv_bias_rope_transpose(C.c_int(dtype), _p(q_buf), _p(k_buf), _p(v_buf), _p(QKV), _p(bias),
                                                _p(padding_offset), _p(history_length), C.c_int(B), C.c_int(seq_len),
                                                C.c_int(num_tokens), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(rot_dim),
                                                C.c_float(rope_base), _stream(stream)))


def append_kv_cache(dtype, dst, src, cur_query_length, history_length, B, Hkv, max_q_len, max_seq_len, D,
                    overflow_flag=None, stream=None):
    _check(lib().onellm_append_kv_cache(C.c_int(dtype), _p(dst), _p(src), _p(cur_query_length), _p(history_length),
                                        C.c_int(B), C.c_int(Hkv), C.c_int(max_q_len), C.c_int(max_seq_len), C.c_int(D),
                                        _p(overflow_flag), _stream(stream)))


def repeat_kv(dtype, dst, src, context_length, B, H, Hkv, max_k_len, max_seq_len, D, stream=None):
    _check(lib().onellm_repeat_kv(C.c_int(dtype), _p(dst), _p(src), _p(context_length), C.c_int(B), C.c_int(H),
                                  C.c_int(Hkv), C.c_int(max_k_len), C.c_int(max_seq_len), C.c_int(D), _stream(stream)))


def batched_gemm(dtype, A, Bm, Cm, batch, m, n, k, trans_a=False, trans_b=False, stream=None):
    _check(lib().onellm_batched_gemm(C.c_int(dtype), _p(A), _p(Bm), _p(Cm), C.c_int(batch), C.c_int(m), C.c_int(n),
                                     C.c_int(k), C.c_int(1 if trans_a else 0), C.c_int(1 if trans_b else 0), _stream(stream)))


def scale_mask_softmax(dtype, attn_score, qk, mask, B, H, q_len, k_len, scale, stream=None):
    _check(lib().onellm_scale_mask_softmax(C.c_int(dtype), _p(attn_score), _p(qk), _p(mask), C.c_int(B), C.c_int(H),
                                           C.c_int(q_len), C.c_int(k_len), C.c_float(scale), _stream(stream)))


def transpose_remove_padding(dtype, dst, src, padding_offset, num_tokens, B, S, H, D, stream=None):
    _check(lib().onellm_transpose_remove_padding(C.c_int(dtype), _p(dst), _p(src), _p(padding_offset), C.c_int(num_tokens),
                                                 C.c_int(B), C.c_int(S), C.c_int(H), C.c_int(D), _stream(stream)))


def topk(dtype, logits, rows, vocab, K, out_val, out_id, global_ids=False, stream=None):
    _check(lib().onellm_topk(C.c_int(dtype), _p(logits), C.c_int(rows), C.c_int(vocab), C.c_int(K),
                             _p(out_val), _p(out_id), C.c_int(1 if global_ids else 0), _stream(stream)))


def topk_sample(topk_id, topk_val, B, K, temperature, rng_step, vocab_size, end_id, output_id, seqlen=None,
                finished=None, u_out=None, literal_walk=False, rng_step_dev=None, stream=None):
    _check(lib().onellm_topk_sample(_p(topk_id), _p(topk_val), C.c_int(B), C.c_int(K), C.c_float(temperature),
                                    C.c_int(rng_step), _p(rng_step_dev), C.c_int(vocab_size), C.c_int(end_id),
                                    C.c_int(1 if literal_walk else 0), _p(output_id), _p(seqlen), _p(finished),
                                    _p(u_out), _stream(stream)))


def p2p_two_shot_bytes(nbytes=-1):
    """Threshold (one-shot wire bytes per rank) from which the projections' exchange goes two-shot; returns the previous one."""
    f = lib().onellm_p2p_two_shot_bytes
    f.restype = C.c_longlong
    return int(f(C.c_longlong(nbytes)))


class P2p:
    """The peer-memory all-reduce on its own (one object per process / GPU)."""

    def __init__(self, rank, world, max_elems):
        self._h = C.c_void_p()
        _check(lib().onellm_p2p_create(C.c_int(rank), C.c_int(world), C.c_size_t(max_elems), C.byref(self._h)))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(lib().onellm_p2p_handle(self._h, buf))
        return buf.raw

    def connect(self, handles):
        _check(lib().onellm_p2p_connect(self._h, C.c_char_p(b"".join(handles))))

    def send_buffer(self, which) -> int:
        f = lib().onellm_p2p_send_buffer
        f.restype = C.c_void_p
        return int(f(self._h, C.c_int(which)))

    def allreduce_add(self, which, resid, bias, n_elems, row_len, stream=None):
        _check(lib().onellm_p2p_allreduce_add(self._h, C.c_int(F16), C.c_int(which), _p(resid), _p(bias), C.c_int(n_elems),
                                              C.c_int(row_len), _stream(stream)))

    def gemm_allreduce_add(self, which, x, W, resid, bias, M, N, K, stream=None):
        _check(lib().onellm_p2p_gemm_allreduce_add(self._h, C.c_int(F16), C.c_int(which), _p(x), _p(W), _p(resid), _p(bias),
                                                   C.c_int(M), C.c_int(N), C.c_int(K), _stream(stream)))

    def error(self) -> int:
        return int(lib().onellm_p2p_error(self._h))

    def close(self):
        if self._h:
            lib().onellm_p2p_destroy(self._h)
            self._h = C.c_void_p()


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _check(lib().onellm_nccl_unique_id(buf))
    return buf.raw


def llama_config_from_ini(path, max_batch=1, max_seq_len=0, tp_rank=0, tp_size=1):
    """(LlamaConfig, top_k) from the reference converter's config.ini; touches no GPU."""
    cfg = LlamaConfig()
    cfg.max_batch, cfg.max_seq_len, cfg.tp_rank, cfg.tp_size, cfg.bos_id, cfg.eos_id = max_batch, max_seq_len, tp_rank, tp_size, 1, 2
    top_k = C.c_int(0)
    _check(lib().onellm_llama_config_from_ini(str(path).encode(), C.byref(cfg), C.byref(top_k)))
    return cfg, top_k.value


class Llama:
    """Host-side handle of the C++ model (weights, KV cache, generation loop)."""

    @classmethod
    def from_ini(cls, path, max_batch, max_seq_len, tp_rank=0, tp_size=1):
        """The model described by the reference converter's config.ini (sampling set to the file's top_k)."""
        self = cls.__new__(cls)
        self.cfg, _ = llama_config_from_ini(path, max_batch, max_seq_len, tp_rank, tp_size)
        self._h = C.c_void_p(0)
        _check(lib().onellm_llama_create_from_ini(str(path).encode(), C.c_int(max_batch), C.c_int(max_seq_len), C.c_int(tp_rank),
                                                  C.c_int(tp_size), C.byref(self._h)))
        return self

    def __init__(self, *, num_layers, hidden, head_num, kv_head_num, head_size, inter_size, vocab_size,
                 max_seq_len, max_batch, rope_base=10000.0, rot_dim=0, rms_eps=1e-5, bos_id=1, eos_id=2,
                 attn_bias=False, tp_rank=0, tp_size=1):
        self.cfg = LlamaConfig(num_layers, hidden, head_num, kv_head_num, head_size, inter_size, vocab_size,
                               max_seq_len, max_batch, rope_base, rot_dim, rms_eps, bos_id, eos_id,
                               1 if attn_bias else 0, tp_rank, tp_size)
        self._h = C.c_void_p(0)
        _check(lib().onellm_llama_create(C.byref(self.cfg), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().onellm_llama_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def device_bytes(self):
        return int(lib().onellm_llama_device_bytes(self._h))

    @property
    def stream(self):
        return int(lib().onellm_llama_stream(self._h) or 0)

    def load_weights(self, prefix: str):
        _check(lib().onellm_llama_load_weights(self._h, prefix.encode()))

    def init_random(self, seed: int, std: float = 0.02):
        _check(lib().onellm_llama_init_random(self._h, C.c_uint64(seed), C.c_float(std)))

    def init_comm(self, unique_id: bytes):
        _check(lib().onellm_llama_init_comm(self._h, C.c_char_p(unique_id)))

    def p2p_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(lib().onellm_llama_p2p_handle(self._h, buf))
        return buf.raw

    def p2p_connect(self, handles):
        """handles: the 64-byte handles of all ranks, in rank order."""
        blob = b"".join(handles)
        _check(lib().onellm_llama_p2p_connect(self._h, C.c_char_p(blob)))

    def p2p_error(self) -> int:
        return int(lib().onellm_llama_p2p_error(self._h))

    def last_draws(self):
        """(u, step, table_in_use): the uniform draws of the last sampling launch (numpy float32 [max_batch]), the step
        counter that seeded them and whether the engine's skip-ahead table is in use."""
        import numpy as np
        u = np.zeros(self.cfg.max_batch, np.float32)
        step, used = C.c_int(0), C.c_int(0)
        _check(lib().onellm_llama_last_draws(self._h, u.ctypes.data_as(C.c_void_p), C.byref(step), C.byref(used)))
        return u, step.value, bool(used.value)

    def set_sampling(self, top_k=1, temperature=1.0, literal_walk=False):
        _check(lib().onellm_llama_set_sampling(self._h, C.c_int(top_k), C.c_float(temperature),
                                               C.c_int(1 if literal_walk else 0)))

    def set_tp_exchange(self, peer_memory: bool):
        _check(lib().onellm_llama_set_tp_exchange(self._h, C.c_int(1 if peer_memory else 0)))

    def set_graphs(self, enabled: bool):
        _check(lib().onellm_llama_set_graphs(self._h, C.c_int(1 if enabled else 0)))

    def set_prefill_by_decode(self, enabled):
        """False / 0: context-phase kernels; True / 1: position by position; 2: context-phase kernels with norm kernels."""
        _check(lib().onellm_llama_set_prefill_by_decode(self._h, C.c_int(int(enabled))))

    def prefill(self, ids):
        """ids: int32 numpy [batch, prompt_len]; returns the first sampled id per sequence."""
        import numpy as np
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.zeros(ids.shape[0], np.int32)
        _check(lib().onellm_llama_prefill(self._h, ids.ctypes.data_as(C.c_void_p), C.c_int(ids.shape[0]),
                                          C.c_int(ids.shape[1]), out.ctypes.data_as(C.c_void_p)))
        return out

    def prefill_ragged(self, prompts):
        """prompts: a list of int32 arrays of different lengths; returns the first sampled id per sequence."""
        import numpy as np
        lens = np.array([len(p) for p in prompts], np.int32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p, np.int32) for p in prompts]))
        out = np.zeros(len(prompts), np.int32)
        _check(lib().onellm_llama_prefill_ragged(self._h, ids.ctypes.data_as(C.c_void_p), lens.ctypes.data_as(C.c_void_p),
                                                 C.c_int(len(prompts)), out.ctypes.data_as(C.c_void_p)))
        return out

    def extend(self, ids):
        """ids [batch, n_new]: a further turn behind the cached positions; returns the next token per sequence."""
        import numpy as np
        ids = np.ascontiguousarray(ids, np.int32)
        first = np.zeros(ids.shape[0], np.int32)
        _check(lib().onellm_llama_extend(self._h, ids.ctypes.data_as(C.c_void_p), C.c_int(ids.shape[1]),
                                         first.ctypes.data_as(C.c_void_p)))
        return first

    def seek(self, batch, cur_len, ids):
        import numpy as np
        ids = np.ascontiguousarray(ids, np.int32)
        _check(lib().onellm_llama_seek(self._h, C.c_int(batch), C.c_int(cur_len), ids.ctypes.data_as(C.c_void_p)))

    def decode_step(self, in_ids=None, out_ids=None):
        """in_ids / out_ids: int32 numpy [batch] or None (see onellm_llama_decode_step)."""
        _check(lib().onellm_llama_decode_step(
            self._h, None if in_ids is None else in_ids.ctypes.data_as(C.c_void_p),
            None if out_ids is None else out_ids.ctypes.data_as(C.c_void_p)))

    def decode_step_raw(self, in_ptr: int, out_ptr: int):
        """Same with raw host addresses (e.g. pinned torch tensors)."""
        _check(lib().onellm_llama_decode_step(self._h, C.c_void_p(in_ptr), C.c_void_p(out_ptr)))

    def sync(self):
        _check(lib().onellm_llama_sync(self._h))

    def generate(self, prompt, n_new):
        import numpy as np
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros((prompt.shape[0], n_new), np.int32)
        _check(lib().onellm_llama_generate(self._h, prompt.ctypes.data_as(C.c_void_p), C.c_int(prompt.shape[0]),
                                           C.c_int(prompt.shape[1]), C.c_int(n_new),
                                           out.ctypes.data_as(C.c_void_p)))
        return out

    def logits(self, batch):
        import numpy as np
        out = np.zeros((batch, self.cfg.vocab_size), np.float32)
        _check(lib().onellm_llama_get_logits(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def state(self):
        cur = C.c_int(0)
        launches = C.c_long(0)
        _check(lib().onellm_llama_get_state(self._h, C.byref(cur), C.byref(launches), None, None))
        return cur.value, launches.value

    def kv_cache_ptrs(self, layer):
        k, v = C.c_void_p(0), C.c_void_p(0)
        _check(lib().onellm_llama_kv_cache(self._h, C.c_int(layer), C.byref(k), C.byref(v)))
        return k.value, v.value
