"""Offline converter: a Hugging Face Llama checkpoint directory -> the raw per-tensor files and the config.ini that
this library's loader (onellm_llama_load_weights, onellm_llama_create_from_ini) and the reference's
LlamaWeight::loadWeights read.

    python -m onellm_b200.convert_hf -i <hf_checkpoint_dir> -o <out_dir> [--dtype fp16|fp32]

It does the job of tools/FT_convert_weight_to_bin_final.py of the reference, which writes a config.ini
(:43-64, the keys kept here) but tensor files the reference's own loader does not look for.  What is written:

* `<out_dir>/config.ini`, section [llama]: model_name, head_num, kv_head_num, hidden_size, head_size, inter_size,
  num_layer, vocab_size, bos_token_id, eos_token_id, weight_data_type, max_position_embeddings, rope_theta,
  rms_norm_eps, attention_bias, top_k.
* One headerless little-endian array per tensor, named as src/weights/llama/llama_weights.cc:39-45 and
  src/weights/llama/layer_weights.cc:44-54 name them for the weight path `<out_dir>/`:
      .norm.weight [hidden]   .tok_embeddings.weight [vocab, hidden]   .output.weight [vocab, hidden]
      layers.N.attention_norm.weight / .ffn_norm.weight [hidden]
      layers.N.attention.w_qkv.weight [hidden, (H + 2 Hkv) D]      (q, k, v columns side by side)
      layers.N.attention.wo.weight    [H D, hidden]
      layers.N.feed_forward.w1.weight / .w3.weight [hidden, inter] (gate, up)   .w2.weight [inter, hidden] (down)
      layers.N.attention.w_qkv.bias [(H + 2 Hkv) D], .attention.wo.bias [hidden]   (attention_bias checkpoints)

Two things change on the way.  Every projection is stored `[in, out]` (the layout launchLinearGemm multiplies by),
the transpose of the checkpoint's `[out, in]`.  And the rows of q_proj and k_proj are re-ordered inside every head:
the checkpoint pairs dimension i with i + D/2 for the rotary embedding (its `rotate_half`), the kernels here and in the
reference rotate the adjacent pair (2i, 2i + 1) (src/kernels/decoder_masked_attn.cu:95-108), so row i goes to 2i and
row i + D/2 to 2i + 1.  Scores q . k do not change under a re-ordering applied to both.

The checkpoint is read tensor by tensor (safetensors shards, or pytorch_model*.bin), so a 13B model needs little more
host memory than its largest tensor.  Needs torch and, for safetensors checkpoints, the safetensors package.
"""
from __future__ import annotations

import argparse
import configparser
import json
import os

import numpy as np


class _Checkpoint:
    """name -> tensor access over the shards of a checkpoint directory."""

    def __init__(self, path):
        self.path = path
        self.where = {}    # tensor name -> shard file
        self.loaded = {}   # shard file -> dict of torch tensors (pytorch_model*.bin only)
        names = os.listdir(path)
        for index in ("model.safetensors.index.json", "pytorch_model.bin.index.json"):
            if index in names:
                with open(os.path.join(path, index)) as f:
                    self.where = dict(json.load(f)["weight_map"])
                return
        shards = sorted(n for n in names if n.endswith(".safetensors")) or sorted(
            n for n in names if n.startswith("pytorch_model") and n.endswith(".bin"))
        if not shards:
            raise FileNotFoundError(f"{path}: no *.safetensors or pytorch_model*.bin found")
        for s in shards:
            for k in self._keys(s):
                self.where[k] = s

    def _keys(self, shard):
        full = os.path.join(self.path, shard)
        if shard.endswith(".safetensors"):
            from safetensors import safe_open
            with safe_open(full, framework="pt") as f:
                return list(f.keys())
        return list(self._bin(shard).keys())

    def _bin(self, shard):
        import torch
        if shard not in self.loaded:
            self.loaded = {shard: torch.load(os.path.join(self.path, shard), map_location="cpu", weights_only=True)}
        return self.loaded[shard]

    def __contains__(self, name):
        return name in self.where

    def get(self, name) -> np.ndarray:
        """The tensor as float32 numpy (bf16 and fp16 are widened exactly)."""
        shard = self.where[name]
        if shard.endswith(".safetensors"):
            from safetensors import safe_open
            with safe_open(os.path.join(self.path, shard), framework="pt") as f:
                t = f.get_tensor(name)
        else:
            t = self._bin(shard)[name]
        return t.float().numpy()


def interleave_rotary_rows(w: np.ndarray, heads: int, head_size: int) -> np.ndarray:
    """Rows (or elements, for a bias) of a q/k projection from the checkpoint's half-split rotary order to adjacent
    pairs: inside every head row i -> 2i and row i + D/2 -> 2i + 1."""
    tail = w.shape[1:]
    return np.ascontiguousarray(w.reshape(heads, 2, head_size // 2, *tail).swapaxes(1, 2)).reshape(heads * head_size, *tail)


def convert(in_dir: str, out_dir: str, dtype: str = "fp16", log=print) -> dict:
    """Converts the checkpoint in `in_dir`; returns the [llama] section it wrote as a dict."""
    with open(os.path.join(in_dir, "config.json")) as f:
        hf = json.load(f)
    np_dtype = {"fp16": np.float16, "fp32": np.float32}[dtype]
    H = int(hf["num_attention_heads"])
    Hkv = int(hf.get("num_key_value_heads") or H)
    hidden = int(hf["hidden_size"])
    D = int(hf.get("head_dim") or hidden // H)
    inter, L, V = int(hf["intermediate_size"]), int(hf["num_hidden_layers"]), int(hf["vocab_size"])
    bias = bool(hf.get("attention_bias", False))
    if hf.get("rope_scaling"):
        raise ValueError("rope_scaling checkpoints are not covered: the kernels apply the plain rotary embedding")
    if D % 2:
        raise ValueError(f"head size {D} is odd")
    ck = _Checkpoint(in_dir)
    os.makedirs(out_dir, exist_ok=True)
    prefix = os.path.join(out_dir, "")

    def first(x, default):
        if isinstance(x, (list, tuple)):
            return x[0] if x else default
        return default if x is None else x

    section = {
        "model_name": str(hf.get("_name_or_path") or os.path.basename(os.path.normpath(in_dir))),
        "head_num": str(H), "kv_head_num": str(Hkv), "hidden_size": str(hidden), "head_size": str(D),
        "inter_size": str(inter), "num_layer": str(L), "vocab_size": str(V),
        "bos_token_id": str(first(hf.get("bos_token_id"), 1)), "eos_token_id": str(first(hf.get("eos_token_id"), 2)),
        "weight_data_type": dtype, "max_position_embeddings": str(hf.get("max_position_embeddings", 2048)),
        "rope_theta": str(hf.get("rope_theta", 10000.0)), "rms_norm_eps": str(hf.get("rms_norm_eps", 1e-5)),
        "attention_bias": str(bias), "top_k": str(hf.get("top_k", 50)),
    }
    cp = configparser.ConfigParser()
    cp["llama"] = section
    with open(os.path.join(out_dir, "config.ini"), "w") as f:
        cp.write(f)

    def put(name, a, shape):
        a = np.ascontiguousarray(a)
        if tuple(a.shape) != tuple(shape):
            raise ValueError(f"{name}: shape {a.shape}, expected {tuple(shape)}")
        a.astype(np_dtype).tofile(prefix + name)

    emb = ck.get("model.embed_tokens.weight")
    put(".tok_embeddings.weight", emb, (V, hidden))
    put(".output.weight", ck.get("lm_head.weight") if "lm_head.weight" in ck else emb, (V, hidden))  # tied embeddings
    del emb
    put(".norm.weight", ck.get("model.norm.weight"), (hidden,))
    for l in range(L):
        p, o = f"model.layers.{l}.", f"layers.{l}."
        q = interleave_rotary_rows(ck.get(p + "self_attn.q_proj.weight"), H, D)
        k = interleave_rotary_rows(ck.get(p + "self_attn.k_proj.weight"), Hkv, D)
        v = ck.get(p + "self_attn.v_proj.weight")
        put(o + "attention.w_qkv.weight", np.concatenate([q.T, k.T, v.T], axis=1), (hidden, (H + 2 * Hkv) * D))
        del q, k, v
        put(o + "attention.wo.weight", ck.get(p + "self_attn.o_proj.weight").T, (H * D, hidden))
        put(o + "feed_forward.w1.weight", ck.get(p + "mlp.gate_proj.weight").T, (hidden, inter))
        put(o + "feed_forward.w3.weight", ck.get(p + "mlp.up_proj.weight").T, (hidden, inter))
        put(o + "feed_forward.w2.weight", ck.get(p + "mlp.down_proj.weight").T, (inter, hidden))
        put(o + "attention_norm.weight", ck.get(p + "input_layernorm.weight"), (hidden,))
        put(o + "ffn_norm.weight", ck.get(p + "post_attention_layernorm.weight"), (hidden,))
        if bias:
            bq = interleave_rotary_rows(ck.get(p + "self_attn.q_proj.bias"), H, D)
            bk = interleave_rotary_rows(ck.get(p + "self_attn.k_proj.bias"), Hkv, D)
            put(o + "attention.w_qkv.bias", np.concatenate([bq, bk, ck.get(p + "self_attn.v_proj.bias")]), ((H + 2 * Hkv) * D,))
            ob_name = p + "self_attn.o_proj.bias"
            put(o + "attention.wo.bias", ck.get(ob_name) if ob_name in ck else np.zeros(hidden, np.float32), (hidden,))
        log(f"layer {l + 1}/{L}")
    return section


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-i", "--in-dir", required=True, help="Hugging Face checkpoint directory (config.json + weights)")
    ap.add_argument("-o", "--out-dir", required=True, help="output directory; pass it with a trailing / as the weight path")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "fp32"], help="element type of the files written")
    a = ap.parse_args()
    s = convert(a.in_dir, a.out_dir, a.dtype)
    print(f"wrote {a.out_dir}: {s['num_layer']} layers, hidden {s['hidden_size']}, {s['head_num']} heads "
          f"({s['kv_head_num']} KV), vocab {s['vocab_size']}, {a.dtype}")


if __name__ == "__main__":
    main()
