"""ctypes access to oracle/_ref/libonellm_ref.so (the reference's own code compiled in place).
TEST INFRASTRUCTURE ONLY.  `load()` returns None when the library has not been built."""
import ctypes as C
import os

import numpy as np

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libonellm_ref.so")
_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int)
_lib = None


def load():
    global _lib
    if _lib is None and os.path.exists(PATH):
        try:
            _lib = C.CDLL(PATH)
        except OSError:
            _lib = None
    return _lib


def fp(a):
    return a.ctypes.data_as(_f)


def ip(a):
    return a.ctypes.data_as(_i)


def cpu_swiglu(inp):
    inp = np.ascontiguousarray(inp, np.float32)
    out = np.zeros((inp.shape[0], inp.shape[2]), np.float32)
    load().ref_cpu_swiglu(fp(inp), fp(out), C.c_int(inp.shape[0]), C.c_int(inp.shape[2]))
    return out


def cpu_linear(weight_mk, input_kn):
    """The reference helper computes output[m,n] += weight[m,k] . input[k,n]."""
    w, x = np.ascontiguousarray(weight_mk, np.float32), np.ascontiguousarray(input_kn, np.float32)
    out = np.zeros((w.shape[0], x.shape[1]), np.float32)
    load().ref_cpu_linear(fp(x), fp(w), fp(out), C.c_int(w.shape[0]), C.c_int(w.shape[1]), C.c_int(x.shape[1]))
    return out


def cpu_embedding(ids, table):
    ids, table = np.ascontiguousarray(ids, np.int32), np.ascontiguousarray(table, np.float32)
    out = np.zeros((ids.size, table.shape[1]), np.float32)
    load().ref_cpu_embedding(ip(ids), fp(out), fp(table), C.c_int(ids.size), C.c_int(table.shape[1]), C.c_int(table.shape[0]))
    return out


def cpu_causal_mask(q_lens, k_lens, max_q, max_k):
    q, k = np.ascontiguousarray(q_lens, np.int32), np.ascontiguousarray(k_lens, np.int32)
    m = np.zeros((len(q), max_q, max_k), np.float32)
    load().ref_cpu_causal_mask(fp(m), ip(q), ip(k), C.c_int(max_q), C.c_int(max_k), C.c_int(len(q)))
    return m


def cpu_fused_resid_rmsnorm(residual, decoder_out, bias, scale, eps):
    r, y = np.ascontiguousarray(residual, np.float32).copy(), np.ascontiguousarray(decoder_out, np.float32).copy()
    b, s = np.ascontiguousarray(bias, np.float32), np.ascontiguousarray(scale, np.float32)
    load().ref_cpu_fused_resid_rmsnorm(fp(r), fp(y), fp(b), fp(s), C.c_float(eps), C.c_int(y.shape[1]), C.c_int(y.shape[0]))
    return y


def cpu_qkv_bias_rope_q(QKV_bshd, bias, history, batch, seq_len, H, Hkv, D, rot_dim, base):
    """q part of the reference helper: input and output laid out [B, S, H, D] (the helper's own indexing)."""
    x = np.ascontiguousarray(QKV_bshd, np.float32)
    q = np.zeros(batch * seq_len * H * D, np.float32)
    k = np.zeros(batch * seq_len * max(Hkv, 1) * D * 4, np.float32)
    v = np.zeros_like(k)
    big = np.zeros(batch * seq_len * (H + 2 * Hkv) * D * 2, np.float32)
    big[:x.size] = x.ravel()
    b = np.ascontiguousarray(bias, np.float32)
    hl = np.ascontiguousarray(history, np.int32)
    il = np.full(batch, seq_len, np.int32)
    po = np.zeros(batch * seq_len, np.int32)
    load().ref_cpu_qkv_bias_rope(fp(q), fp(k), fp(v), fp(big), fp(b), ip(po), ip(hl), ip(il), C.c_int(batch), C.c_int(seq_len),
                                 C.c_int(batch * seq_len), C.c_int(H), C.c_int(Hkv), C.c_int(D), C.c_int(rot_dim), C.c_float(base))
    return q.reshape(batch, seq_len, H, D)
