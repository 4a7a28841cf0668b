"""LLaMA decode on the CPU, composed from the oracle's operators.  TEST INFRASTRUCTURE ONLY.

Mirrors the sequencing of LlamaSelfDecoder::forward (src/layers/decoder/self_decoder.cpp:15-78
in the reference) with the residual stream kept apart from the normalised activations, which is
what the outline in src/models/llama/llama.cpp:1-32 describes.  Used by the GPU tests as the
checker and by the benchmark as the timed CPU baseline; never by the product.

``storage`` = "f16" rounds every tensor that the GPU engine stores in fp16 (activations between
kernels, the KV cache, logits) so that the comparison measures arithmetic, not storage.
"""
from __future__ import annotations

import os

import numpy as np

from . import (add_residual_rmsnorm, decode_attn, embedding, gemm, rmsnorm, swiglu2, topk, topk_sample)


def _r16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def random_weights(cfg, seed, std=0.02, attn_bias=False):
    """fp16-representable random weights in the reference's tensor shapes."""
    rng = np.random.default_rng(seed)
    h, D, H, Hkv, I, V, L = (cfg[k] for k in ("hidden", "head_size", "head_num", "kv_head_num", "inter_size",
                                              "vocab_size", "num_layers"))
    n = lambda *s: _r16(std * rng.standard_normal(s))
    w = {"norm": _r16(1 + 0.1 * rng.standard_normal(h)), "tok_embeddings": n(V, h), "output": n(V, h), "layers": []}
    for _ in range(L):
        lw = {"attention_norm": _r16(1 + 0.1 * rng.standard_normal(h)), "ffn_norm": _r16(1 + 0.1 * rng.standard_normal(h)),
              "w_qkv": n(h, (H + 2 * Hkv) * D), "wo": n(h, h), "w1": n(h, I), "w3": n(h, I), "w2": n(I, h)}
        if attn_bias:
            lw["b_qkv"] = n((H + 2 * Hkv) * D)
            lw["b_o"] = n(h)
        w["layers"].append(lw)
    return w


# file-name suffix of every per-layer tensor (src/weights/llama/layer_weights.cc:44-54)
LAYER_FILE_SUFFIX = {"attention_norm": ".attention_norm.weight", "ffn_norm": ".ffn_norm.weight",
                     "w_qkv": ".attention.w_qkv.weight", "wo": ".attention.wo.weight", "w1": ".feed_forward.w1.weight",
                     "w3": ".feed_forward.w3.weight", "w2": ".feed_forward.w2.weight", "b_qkv": ".attention.w_qkv.bias",
                     "b_o": ".attention.wo.bias"}


def save_bin(w, prefix, dtype=np.float32):
    """Writes the weights in the reference's on-disk layout: one raw array per tensor, names as in
    src/weights/llama/llama_weights.cc:39-45 and src/weights/llama/layer_weights.cc:44-54."""
    os.makedirs(os.path.dirname(prefix) or ".", exist_ok=True)
    w["norm"].astype(dtype).tofile(prefix + ".norm.weight")
    w["tok_embeddings"].astype(dtype).tofile(prefix + ".tok_embeddings.weight")
    w["output"].astype(dtype).tofile(prefix + ".output.weight")
    for l, lw in enumerate(w["layers"]):
        for k, a in lw.items():
            a.astype(dtype).tofile(f"{prefix}layers.{l}{LAYER_FILE_SUFFIX[k]}")


class LlamaRef:
    def __init__(self, cfg, weights, batch, storage="f16"):
        self.cfg, self.w, self.B = cfg, weights, batch
        self.rnd = _r16 if storage == "f16" else (lambda a: np.asarray(a, np.float32))
        L, Hkv, S, D = cfg["num_layers"], cfg["kv_head_num"], cfg["max_seq_len"], cfg["head_size"]
        self.k_cache = np.zeros((L, batch, Hkv, S, D), np.float32)
        self.v_cache = np.zeros((L, batch, Hkv, S, D), np.float32)
        self.cur_len = 0
        self.logits = None

    def step(self, ids, lm_head=True, layers=None):
        """One token per sequence at position cur_len; returns logits [B, V] (or None)."""
        c, w, r = self.cfg, self.w, self.rnd
        H, Hkv, D = c["head_num"], c["kv_head_num"], c["head_size"]
        eps = c.get("rms_eps", 1e-5)
        step = self.cur_len + 1
        res = embedding(np.asarray(ids, np.int32), w["tok_embeddings"])
        y = r(rmsnorm(res, w["layers"][0]["attention_norm"], eps))
        nl = c["num_layers"] if layers is None else layers
        for l in range(nl):
            lw = w["layers"][l]
            qkv = r(gemm(y, lw["w_qkv"])).reshape(self.B, H + 2 * Hkv, D)
            b = lw.get("b_qkv")
            bq = None if b is None else b[:H * D]
            bk = None if b is None else b[H * D:(H + Hkv) * D]
            bv = None if b is None else b[(H + Hkv) * D:]
            kc, vc = self.k_cache[l], self.v_cache[l]
            attn = decode_attn(qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:], kc, vc, step, rope_pos=step - 1,
                               rot_dim=c.get("rot_dim", D) or D, rope_base=c.get("rope_base", 10000.0), bias_q=bq,
                               bias_k=bk, bias_v=bv)
            kc[:, :, step - 1], vc[:, :, step - 1] = r(kc[:, :, step - 1]), r(vc[:, :, step - 1])
            o = r(gemm(r(attn).reshape(self.B, H * D), lw["wo"]))
            y, res = add_residual_rmsnorm(res, o, lw.get("b_o"), lw["ffn_norm"], eps)
            y, res = r(y), r(res)
            act = r(swiglu2(gemm(y, lw["w1"]), gemm(y, lw["w3"])))
            d = r(gemm(act, lw["w2"]))
            gamma = w["layers"][l + 1]["attention_norm"] if l + 1 < c["num_layers"] else w["norm"]
            y, res = add_residual_rmsnorm(res, d, None, gamma, eps)
            y, res = r(y), r(res)
        self.cur_len += 1
        if lm_head:
            self.logits = r(gemm(y, w["output"], w_is_nk=True))
            return self.logits
        return None

    def prefill(self, prompt):
        prompt = np.asarray(prompt, np.int32)
        for p in range(prompt.shape[1]):
            out = self.step(prompt[:, p], lm_head=(p == prompt.shape[1] - 1))
        return out

    @staticmethod
    def greedy(logits):
        return topk(logits, 1)[1][:, 0]


def tp_slice(w, cfg, rank, size):
    """The tensor-parallel slice rank `rank` of `size` keeps: query/KV heads and FFN columns, with the
    matching rows of wo / w2: what the engine's loader cuts from the files."""
    H, Hkv, D, I = cfg["head_num"], cfg["kv_head_num"], cfg["head_size"], cfg["inter_size"]
    Hl, Hkvl, Il = H // size, Hkv // size, I // size
    qs = slice(rank * Hl * D, (rank + 1) * Hl * D)
    ks = slice(H * D + rank * Hkvl * D, H * D + (rank + 1) * Hkvl * D)
    vs = slice((H + Hkv) * D + rank * Hkvl * D, (H + Hkv) * D + (rank + 1) * Hkvl * D)
    out = {"norm": w["norm"], "tok_embeddings": w["tok_embeddings"], "output": w["output"], "layers": []}
    for lw in w["layers"]:
        s = {"attention_norm": lw["attention_norm"], "ffn_norm": lw["ffn_norm"],
             "w_qkv": np.concatenate([lw["w_qkv"][:, qs], lw["w_qkv"][:, ks], lw["w_qkv"][:, vs]], axis=1),
             "wo": lw["wo"][rank * Hl * D:(rank + 1) * Hl * D], "w1": lw["w1"][:, rank * Il:(rank + 1) * Il],
             "w3": lw["w3"][:, rank * Il:(rank + 1) * Il], "w2": lw["w2"][rank * Il:(rank + 1) * Il]}
        if "b_qkv" in lw:
            s["b_qkv"] = np.concatenate([lw["b_qkv"][qs], lw["b_qkv"][ks], lw["b_qkv"][vs]])
            s["b_o"] = lw["b_o"]
        out["layers"].append({k: np.ascontiguousarray(v) for k, v in s.items()})
    return out


class LlamaRefTP(LlamaRef):
    """One tensor-parallel rank: local heads and FFN columns, `allreduce(array)` sums the partial
    o_proj / down_proj outputs over the ranks (any backend; the CPU tests use gloo)."""

    def __init__(self, cfg, weights, batch, rank, size, allreduce, storage="f16"):
        local = dict(cfg, head_num=cfg["head_num"] // size, kv_head_num=cfg["kv_head_num"] // size,
                     inter_size=cfg["inter_size"] // size)
        super().__init__(local, tp_slice(weights, cfg, rank, size), batch, storage)
        self.full_hidden = cfg["hidden"]
        self.allreduce = allreduce

    def step(self, ids, lm_head=True, layers=None):
        c, w, r = self.cfg, self.w, self.rnd
        H, Hkv, D = c["head_num"], c["kv_head_num"], c["head_size"]
        eps = c.get("rms_eps", 1e-5)
        step = self.cur_len + 1
        res = embedding(np.asarray(ids, np.int32), w["tok_embeddings"])
        y = r(rmsnorm(res, w["layers"][0]["attention_norm"], eps))
        for l in range(c["num_layers"]):
            lw = w["layers"][l]
            qkv = r(gemm(y, lw["w_qkv"])).reshape(self.B, H + 2 * Hkv, D)
            b = lw.get("b_qkv")
            bq = None if b is None else b[:H * D]
            bk = None if b is None else b[H * D:(H + Hkv) * D]
            bv = None if b is None else b[(H + Hkv) * D:]
            kc, vc = self.k_cache[l], self.v_cache[l]
            attn = decode_attn(qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:], kc, vc, step, rope_pos=step - 1,
                               rot_dim=c.get("rot_dim", D) or D, rope_base=c.get("rope_base", 10000.0), bias_q=bq,
                               bias_k=bk, bias_v=bv)
            kc[:, :, step - 1], vc[:, :, step - 1] = r(kc[:, :, step - 1]), r(vc[:, :, step - 1])
            o = r(self.allreduce(r(gemm(r(attn).reshape(self.B, H * D), lw["wo"]))))
            y, res = add_residual_rmsnorm(res, o, lw.get("b_o"), lw["ffn_norm"], eps)
            y, res = r(y), r(res)
            act = r(swiglu2(gemm(y, lw["w1"]), gemm(y, lw["w3"])))
            d = r(self.allreduce(r(gemm(act, lw["w2"]))))
            gamma = w["layers"][l + 1]["attention_norm"] if l + 1 < c["num_layers"] else w["norm"]
            y, res = add_residual_rmsnorm(res, d, None, gamma, eps)
            y, res = r(y), r(res)
        self.cur_len += 1
        if lm_head:
            self.logits = r(gemm(y, w["output"], w_is_nk=True))
            return self.logits
        return None
