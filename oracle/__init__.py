"""numpy front end of the CPU oracle (``onellm_oracle.c``).

TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's CPU-baseline leg
import this module to check or to time the reference arithmetic on the host.  Nothing in
the ``onellm_b200`` package imports it.

Every function takes and returns float32 / int32 numpy arrays and forwards to the C
function of the same name, which cites the reference lines it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libonellm_oracle.so")
_lib = None

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)
_u8p = C.POINTER(C.c_ubyte)


def build(force: bool = False) -> str:
    """Compile the C oracle if it is missing or older than its source."""
    src = os.path.join(_HERE, "onellm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "all"])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _pf(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _pi(a):
    return None if a is None else a.ctypes.data_as(_i32p)


def _chk(rc, name):
    if rc < 0:
        raise ValueError(f"oracle {name} failed with status {rc}")
    return rc


def rope(x, head_size, rot_dim, base, pos):
    """Rotate ``x`` ([n, head_size]) at positions ``pos`` ([n]); returns a new array."""
    x = _f(x).copy()
    pos = _f(pos)
    _chk(lib().orc_rope(_pf(x), C.c_int(x.size // head_size), C.c_int(head_size), C.c_int(rot_dim),
                        C.c_float(base), _pf(pos)), "rope")
    return x


def decode_attn(q, k, v, k_cache, v_cache, step, *, rope_pos=None, rot_dim=None, rope_base=10000.0,
                scale=None, bias_q=None, bias_k=None, bias_v=None, cache_layout="bhsd", acc64=True):
    """Decode-step attention.  q [B,H,D]; k, v [B,Hkv,D]; caches are modified in place.

    cache_layout "bhsd": [B,Hkv,S,D];  "sbhd": [S,B,Hkv,D] (the order the reference kernel indexes).
    Returns out [B,H,D].
    """
    q, k, v = _f(q), _f(k), _f(v)
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
    assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
    B, H, D = q.shape
    Hkv = k.shape[1]
    if cache_layout == "bhsd":
        S = k_cache.shape[2]
        cs_b, cs_h, cs_s = Hkv * S * D, S * D, D
    elif cache_layout == "sbhd":
        cs_s, cs_b, cs_h = B * Hkv * D, Hkv * D, D
    else:
        raise ValueError(cache_layout)
    out = np.empty((B, H, D), np.float32)
    bq = None if bias_q is None else _f(bias_q)
    bk = None if bias_k is None else _f(bias_k)
    bv = None if bias_v is None else _f(bias_v)
    _chk(lib().orc_decode_attn(
        _pf(q), _pf(k), _pf(v), C.c_long(H * D), C.c_long(Hkv * D), C.c_long(Hkv * D),
        _pf(bq), _pf(bk), _pf(bv), _pf(k_cache), _pf(v_cache),
        C.c_long(cs_b), C.c_long(cs_h), C.c_long(cs_s),
        C.c_int(B), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(step),
        C.c_float(step if rope_pos is None else rope_pos), C.c_int(D if rot_dim is None else rot_dim),
        C.c_float(rope_base), C.c_float(1.0 / np.sqrt(D) if scale is None else scale),
        _pf(out), C.c_long(H * D), C.c_int(1 if acc64 else 0)), "decode_attn")
    return out


def rmsnorm(x, gamma, eps):
    x = _f(x).copy()
    gamma = _f(gamma)
    T, h = x.shape
    _chk(lib().orc_rmsnorm(_pf(x), _pf(gamma), C.c_float(eps), C.c_int(T), C.c_int(h)), "rmsnorm")
    return x


def add_residual_rmsnorm(residual, decoder_out, bias, gamma, eps):
    """Returns (normed, new_residual)."""
    r = _f(residual).copy()
    y = _f(decoder_out).copy()
    b = None if bias is None else _f(bias)
    gamma = _f(gamma)
    T, h = y.shape
    _chk(lib().orc_add_residual_rmsnorm(_pf(r), _pf(y), _pf(b), _pf(gamma), C.c_float(eps), C.c_int(T),
                                        C.c_int(h)), "add_residual_rmsnorm")
    return y, r


def cal_padding_offset(seq_lens, max_q_len):
    seq_lens = np.ascontiguousarray(seq_lens, np.int32)
    B = len(seq_lens)
    po = np.zeros(int(seq_lens.sum()), np.int32)
    cum = np.zeros(B + 1, np.int32)
    n = lib().orc_cal_padding_offset(_pi(po), _pi(cum), _pi(seq_lens), C.c_int(B), C.c_int(max_q_len))
    return po, cum, int(n)


def build_causal_mask(q_lens, k_lens, max_q_len, max_k_len, attend_history=False):
    q_lens = np.ascontiguousarray(q_lens, np.int32)
    k_lens = np.ascontiguousarray(k_lens, np.int32)
    m = np.zeros((len(q_lens), max_q_len, max_k_len), np.float32)
    lib().orc_build_causal_mask(_pf(m), _pi(q_lens), _pi(k_lens), C.c_int(max_q_len), C.c_int(max_k_len),
                                C.c_int(len(q_lens)), C.c_int(1 if attend_history else 0))
    return m


def qkv_bias_rope_transpose(QKV, bias, padding_offset, history_length, batch_size, seq_len, H, Hkv,
                            rot_dim, base):
    QKV = _f(QKV)
    T, QH, D = QKV.shape
    assert QH == H + 2 * Hkv
    q = np.zeros((batch_size, H, seq_len, D), np.float32)
    k = np.zeros((batch_size, Hkv, seq_len, D), np.float32)
    v = np.zeros((batch_size, Hkv, seq_len, D), np.float32)
    b = None if bias is None else _f(bias)
    po = np.ascontiguousarray(padding_offset, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    _chk(lib().orc_qkv_bias_rope_transpose(_pf(q), _pf(k), _pf(v), _pf(QKV), _pf(b), _pi(po), _pi(hl),
                                           C.c_int(batch_size), C.c_int(seq_len), C.c_int(T), C.c_int(H),
                                           C.c_int(Hkv), C.c_int(D), C.c_int(rot_dim), C.c_float(base)),
         "qkv_bias_rope_transpose")
    return q, k, v


def append_kv_cache(dst, src, cur_query_length, history_length):
    """dst [B,Hkv,S,D] is modified in place from src [B,Hkv,max_q,D]."""
    assert dst.dtype == np.float32 and dst.flags.c_contiguous
    src = _f(src)
    B, Hkv, S, D = dst.shape
    ql = np.ascontiguousarray(cur_query_length, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    _chk(lib().orc_append_kv_cache(_pf(dst), _pf(src), _pi(ql), _pi(hl), C.c_int(B), C.c_int(Hkv),
                                   C.c_int(src.shape[2]), C.c_int(S), C.c_int(D)), "append_kv_cache")
    return dst


def repeat_kv(src, context_length, H, max_k_len):
    src = _f(src)
    B, Hkv, S, D = src.shape
    dst = np.zeros((B, H, max_k_len, D), np.float32)
    cl = np.ascontiguousarray(context_length, np.int32)
    lib().orc_repeat_kv(_pf(dst), _pf(src), _pi(cl), C.c_int(B), C.c_int(H), C.c_int(Hkv),
                        C.c_int(max_k_len), C.c_int(S), C.c_int(D))
    return dst


def scale_mask_softmax(qk, mask, scale):
    qk, mask = _f(qk), _f(mask)
    B, H, ql, kl = qk.shape
    out = np.empty_like(qk)
    lib().orc_scale_mask_softmax(_pf(out), _pf(qk), _pf(mask), C.c_int(B), C.c_int(H), C.c_int(ql),
                                 C.c_int(kl), C.c_float(scale))
    return out


def transpose_remove_padding(src, padding_offset, num_tokens):
    src = _f(src)
    B, H, S, D = src.shape
    po = np.ascontiguousarray(padding_offset, np.int32)
    dst = np.empty((num_tokens, H, D), np.float32)
    _chk(lib().orc_transpose_remove_padding(_pf(dst), _pf(src), _pi(po), C.c_int(num_tokens), C.c_int(B),
                                            C.c_int(S), C.c_int(H), C.c_int(D)), "transpose_remove_padding")
    return dst


def context_attn(q, k_cache, v_cache, input_length, history_length, scale=None):
    """q [T,H,D] packed tokens (biased + rotated); caches [B,Hkv,S,D]; returns [T,H,D]."""
    q = _f(q)
    k_cache, v_cache = _f(k_cache), _f(v_cache)
    T, H, D = q.shape
    B, Hkv, S, _ = k_cache.shape
    il = np.ascontiguousarray(input_length, np.int32)
    hl = np.ascontiguousarray(history_length, np.int32)
    out = np.empty_like(q)
    _chk(lib().orc_context_attn(_pf(q), _pf(k_cache), _pf(v_cache), C.c_long(Hkv * S * D), C.c_long(S * D),
                                C.c_long(D), _pi(il), _pi(hl), C.c_int(B), C.c_int(H), C.c_int(Hkv),
                                C.c_int(D), C.c_float(1.0 / np.sqrt(D) if scale is None else scale),
                                _pf(out)), "context_attn")
    return out


def gemm(x, W, w_is_nk=False):
    """y = x . W (W [K,N]) or x . W^T (W [N,K], ``w_is_nk``)."""
    x, W = _f(x), _f(W)
    M, K = x.shape
    N = W.shape[0] if w_is_nk else W.shape[1]
    assert (W.shape[1] if w_is_nk else W.shape[0]) == K
    y = np.empty((M, N), np.float32)
    _chk(lib().orc_gemm(_pf(x), _pf(W), _pf(y), C.c_int(M), C.c_int(N), C.c_int(K),
                        C.c_int(1 if w_is_nk else 0)), "gemm")
    return y


def swiglu(inp):
    """inp [T, 2, I] -> [T, I]."""
    inp = _f(inp)
    T, two, I = inp.shape
    assert two == 2
    out = np.empty((T, I), np.float32)
    _chk(lib().orc_swiglu(_pf(inp), _pf(out), C.c_int(T), C.c_int(I)), "swiglu")
    return out


def swiglu2(gate, up):
    gate, up = _f(gate), _f(up)
    out = np.empty_like(gate)
    _chk(lib().orc_swiglu2(_pf(gate), _pf(up), _pf(out), C.c_size_t(gate.size)), "swiglu2")
    return out


def embedding(ids, table):
    ids = np.ascontiguousarray(ids, np.int32)
    table = _f(table)
    out = np.empty(ids.shape + (table.shape[1],), np.float32)
    _chk(lib().orc_embedding(_pi(ids), _pf(out), _pf(table), C.c_int(ids.size), C.c_int(table.shape[1]),
                             C.c_int(table.shape[0])), "embedding")
    return out


def topk(logits, K, global_ids=False):
    logits = _f(logits)
    rows, vocab = logits.shape
    val = np.empty((rows, K), np.float32)
    idx = np.empty((rows, K), np.int32)
    _chk(lib().orc_topk(_pf(logits), C.c_int(rows), C.c_int(vocab), C.c_int(K), _pf(val), _pi(idx),
                        C.c_int(1 if global_ids else 0)), "topk")
    return val, idx


def topk_sample(topk_id, topk_val, u, *, temperature=1.0, vocab_size, end_id, literal=False, seqlen=None,
                finished=None):
    """Returns (output_id, seqlen, finished)."""
    topk_id = np.ascontiguousarray(topk_id, np.int32)
    topk_val = _f(topk_val)
    u = _f(u)
    B, K = topk_id.shape
    out = np.zeros(B, np.int32)
    sl = np.zeros(B, np.int32) if seqlen is None else np.ascontiguousarray(seqlen, np.int32).copy()
    fin = np.zeros(B, np.uint8) if finished is None else np.ascontiguousarray(finished, np.uint8).copy()
    _chk(lib().orc_topk_sample(_pi(topk_id), _pf(topk_val), _pf(u), C.c_int(B), C.c_int(K),
                               C.c_float(temperature), C.c_int(vocab_size), C.c_int(end_id),
                               C.c_int(1 if literal else 0), _pi(out), _pi(sl), fin.ctypes.data_as(_u8p)),
         "topk_sample")
    return out, sl, fin
