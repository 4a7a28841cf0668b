"""The offline converter: a Hugging Face-style Llama checkpoint -> the loader's files.  The check is end to end: a small
forward pass written here in the CHECKPOINT's conventions ([out, in] projections, half-split rotary embedding) must give
the logits the oracle (and, on a GPU, the engine) computes from the CONVERTED files in the reference's conventions."""
import json
import os

import numpy as np
import pytest

from conftest import rel_err

HF = dict(num_attention_heads=4, num_key_value_heads=2, hidden_size=256, intermediate_size=160, num_hidden_layers=2,
          vocab_size=120, max_position_embeddings=64, rope_theta=10000.0, rms_norm_eps=1e-5, bos_token_id=1, eos_token_id=2,
          attention_bias=False, _name_or_path="toy-llama")


def _checkpoint(tmp_path, bias=False, tied=False, sharded=False):
    """Writes config.json + safetensors with random fp16-representable weights; returns (dir, state dict)."""
    from safetensors.numpy import save_file
    cfg = dict(HF, attention_bias=bias)
    rng = np.random.default_rng(5)
    h16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)  # fp16 files then lose nothing
    r = lambda *s: h16(0.05 * rng.standard_normal(s))
    H, Hkv, h, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    D = h // H
    sd = {"model.embed_tokens.weight": r(V, h), "model.norm.weight": h16(1 + r(h))}
    if not tied:
        sd["lm_head.weight"] = r(V, h)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        sd.update({p + "self_attn.q_proj.weight": r(H * D, h), p + "self_attn.k_proj.weight": r(Hkv * D, h),
                   p + "self_attn.v_proj.weight": r(Hkv * D, h), p + "self_attn.o_proj.weight": r(h, H * D),
                   p + "mlp.gate_proj.weight": r(I, h), p + "mlp.up_proj.weight": r(I, h), p + "mlp.down_proj.weight": r(h, I),
                   p + "input_layernorm.weight": h16(1 + r(h)), p + "post_attention_layernorm.weight": h16(1 + r(h))})
        if bias:
            sd.update({p + "self_attn.q_proj.bias": r(H * D), p + "self_attn.k_proj.bias": r(Hkv * D),
                       p + "self_attn.v_proj.bias": r(Hkv * D)})
    d = os.path.join(str(tmp_path), "hf")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    if sharded:
        names = sorted(sd)
        half = len(names) // 2
        parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
        for fn, ks in parts.items():
            save_file({k: sd[k] for k in ks}, os.path.join(d, fn))
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": {k: fn for fn, ks in parts.items() for k in ks}}, f)
    else:
        save_file(sd, os.path.join(d, "model.safetensors"))
    return d, sd, cfg


def _hf_forward(sd, cfg, ids):
    """Logits [B, T, V] of a causal Llama forward in the checkpoint's own conventions (float64)."""
    H, Hkv, h = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["hidden_size"]
    D, eps, base = h // H, cfg["rms_norm_eps"], cfg["rope_theta"]
    f = lambda k: sd[k].astype(np.float64)
    norm = lambda x, g: x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * g
    B, T = ids.shape
    pos = np.arange(T)
    inv = base ** (-np.arange(0, D, 2) / D)
    ang = np.concatenate([pos[:, None] * inv[None, :]] * 2, axis=1)        # [T, D]: the two halves share the angles
    cos, sin = np.cos(ang)[None, :, None, :], np.sin(ang)[None, :, None, :]
    rot = lambda x: np.concatenate([-x[..., D // 2:], x[..., :D // 2]], axis=-1)
    x = f("model.embed_tokens.weight")[ids]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        y = norm(x, f(p + "input_layernorm.weight"))
        b = (lambda n: f(p + n) if (p + n) in sd else 0.0)
        q = (y @ f(p + "self_attn.q_proj.weight").T + b("self_attn.q_proj.bias")).reshape(B, T, H, D)
        k = (y @ f(p + "self_attn.k_proj.weight").T + b("self_attn.k_proj.bias")).reshape(B, T, Hkv, D)
        v = (y @ f(p + "self_attn.v_proj.weight").T + b("self_attn.v_proj.bias")).reshape(B, T, Hkv, D)
        q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
        k, v = np.repeat(k, H // Hkv, axis=2), np.repeat(v, H // Hkv, axis=2)
        s = np.einsum("bthd,bshd->bhts", q, k) / np.sqrt(D)
        s = np.where(np.tril(np.ones((T, T), bool))[None, None], s, -np.inf)
        s = np.exp(s - s.max(-1, keepdims=True))
        a = np.einsum("bhts,bshd->bthd", s / s.sum(-1, keepdims=True), v).reshape(B, T, H * D)
        x = x + a @ f(p + "self_attn.o_proj.weight").T
        y = norm(x, f(p + "post_attention_layernorm.weight"))
        g, u = y @ f(p + "mlp.gate_proj.weight").T, y @ f(p + "mlp.up_proj.weight").T
        x = x + (g / (1 + np.exp(-g)) * u) @ f(p + "mlp.down_proj.weight").T
    head = f("lm_head.weight") if "lm_head.weight" in sd else f("model.embed_tokens.weight")
    return norm(x, f("model.norm.weight")) @ head.T


def _engine_cfg(section, max_seq_len=32, max_batch=4):
    return dict(num_layers=int(section["num_layer"]), hidden=int(section["hidden_size"]), head_num=int(section["head_num"]),
                kv_head_num=int(section["kv_head_num"]), head_size=int(section["head_size"]), inter_size=int(section["inter_size"]),
                vocab_size=int(section["vocab_size"]), max_seq_len=max_seq_len, max_batch=max_batch,
                rope_base=float(section["rope_theta"]), rms_eps=float(section["rms_norm_eps"]))


def _read_converted(out_dir, c, dtype, bias):
    from oracle.llama_ref import LAYER_FILE_SUFFIX
    h, D, H, Hkv, I, V = c["hidden"], c["head_size"], c["head_num"], c["kv_head_num"], c["inter_size"], c["vocab_size"]
    rd = lambda name, *shape: np.fromfile(os.path.join(out_dir, name), dtype).astype(np.float32).reshape(shape)
    w = {"norm": rd(".norm.weight", h), "tok_embeddings": rd(".tok_embeddings.weight", V, h), "output": rd(".output.weight", V, h),
         "layers": []}
    shapes = {"attention_norm": (h,), "ffn_norm": (h,), "w_qkv": (h, (H + 2 * Hkv) * D), "wo": (H * D, h), "w1": (h, I), "w3": (h, I),
              "w2": (I, h)}
    if bias:
        shapes.update({"b_qkv": ((H + 2 * Hkv) * D,), "b_o": (h,)})
    for l in range(c["num_layers"]):
        w["layers"].append({k: rd(f"layers.{l}{LAYER_FILE_SUFFIX[k]}", *s) for k, s in shapes.items()})
    return w


@pytest.mark.parametrize("dtype,bias,tied,sharded", [("fp32", False, False, False), ("fp16", True, False, True),
                                                     ("fp16", False, True, False)])
def test_converted_checkpoint_gives_the_checkpoints_logits_through_the_oracle(tmp_path, dtype, bias, tied, sharded):
    from onellm_b200.convert_hf import convert
    from oracle.llama_ref import LlamaRef
    d, sd, cfg = _checkpoint(tmp_path, bias=bias, tied=tied, sharded=sharded)
    out = os.path.join(str(tmp_path), "converted")
    section = convert(d, out, dtype, log=lambda *_: None)
    assert section["head_size"] == "64" and section["attention_bias"] == str(bias) and section["weight_data_type"] == dtype
    import configparser
    cp = configparser.ConfigParser()
    cp.read(os.path.join(out, "config.ini"))
    assert dict(cp["llama"]) == section
    c = _engine_cfg(section)
    w = _read_converted(out, c, np.float16 if dtype == "fp16" else np.float32, bias)
    ids = np.random.default_rng(3).integers(0, c["vocab_size"], (2, 9)).astype(np.int32)
    want = _hf_forward(sd, cfg, ids)[:, -1]
    got = LlamaRef(c, w, 2, storage="f32").prefill(ids)
    assert rel_err(got, want) < 2e-5


@pytest.mark.parametrize("fmt", ["pytorch_bin", "bf16_safetensors"])
def test_converter_reads_the_other_checkpoint_formats(tmp_path, fmt):
    """A single pytorch_model.bin, and safetensors holding bfloat16: the converted fp32 files equal the ones from the
    fp32 safetensors checkpoint (bf16 after the rounding the checkpoint itself carries)."""
    import torch
    from onellm_b200.convert_hf import convert
    d, sd, cfg = _checkpoint(tmp_path)
    ref_out = os.path.join(str(tmp_path), "ref")
    convert(d, ref_out, "fp32", log=lambda *_: None)
    d2 = os.path.join(str(tmp_path), "other")
    os.makedirs(d2)
    with open(os.path.join(d2, "config.json"), "w") as f:
        json.dump(cfg, f)
    if fmt == "pytorch_bin":
        torch.save({k: torch.from_numpy(v) for k, v in sd.items()}, os.path.join(d2, "pytorch_model.bin"))
        expect = lambda a: a
    else:
        from safetensors.torch import save_file
        save_file({k: torch.from_numpy(v).to(torch.bfloat16) for k, v in sd.items()}, os.path.join(d2, "model.safetensors"))
        expect = None
    out = os.path.join(str(tmp_path), "out")
    convert(d2, out, "fp32", log=lambda *_: None)
    names = sorted(n for n in os.listdir(ref_out) if n != "config.ini")
    assert names == sorted(n for n in os.listdir(out) if n != "config.ini") and len(names) == 3 + 7 * cfg["num_hidden_layers"]
    for n in names:
        a, b = np.fromfile(os.path.join(ref_out, n), np.float32), np.fromfile(os.path.join(out, n), np.float32)
        if expect is not None:
            assert np.array_equal(a, b), n
        else:  # what bfloat16 keeps of the same values
            want = torch.from_numpy(a).to(torch.bfloat16).float().numpy()
            assert np.array_equal(want, b), n


def test_interleave_rotary_rows_is_the_stated_permutation():
    from onellm_b200.convert_hf import interleave_rotary_rows
    heads, D = 3, 8
    w = np.arange(heads * D * 2, dtype=np.float32).reshape(heads * D, 2)
    got = interleave_rotary_rows(w, heads, D)
    for hd in range(heads):
        for i in range(D // 2):
            assert np.array_equal(got[hd * D + 2 * i], w[hd * D + i])
            assert np.array_equal(got[hd * D + 2 * i + 1], w[hd * D + i + D // 2])
    b = np.arange(heads * D, dtype=np.float32)
    assert np.array_equal(interleave_rotary_rows(b, heads, D), got[:, 0] / 2)


def test_converter_refuses_what_it_does_not_cover(tmp_path):
    from onellm_b200.convert_hf import convert
    d, sd, cfg = _checkpoint(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(dict(cfg, rope_scaling={"type": "linear", "factor": 2.0}), f)
    with pytest.raises(ValueError):
        convert(d, os.path.join(str(tmp_path), "o"), "fp16", log=lambda *_: None)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(dict(cfg, intermediate_size=96), f)  # does not match the tensors
    with pytest.raises(ValueError):
        convert(d, os.path.join(str(tmp_path), "o2"), "fp16", log=lambda *_: None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,bias", [("fp16", False), ("fp32", True)])
def test_engine_on_a_converted_checkpoint_gives_the_checkpoints_logits(ob, cuda, tmp_path, dtype, bias):
    """config.ini + files from the converter -> onellm_llama_create_from_ini + load_weights -> context phase and two
    decode steps against the forward pass in the checkpoint's conventions."""
    from onellm_b200.convert_hf import convert
    d, sd, cfg = _checkpoint(tmp_path, bias=bias)
    out = os.path.join(str(tmp_path), "converted")
    convert(d, out, dtype, log=lambda *_: None)
    m = ob.Llama.from_ini(os.path.join(out, "config.ini"), max_batch=4, max_seq_len=32)
    m.load_weights(os.path.join(out, ""))
    ids = np.random.default_rng(4).integers(0, cfg["vocab_size"], (3, 11)).astype(np.int32)
    first = m.prefill(ids)
    assert rel_err(m.logits(3), _hf_forward(sd, cfg, ids)[:, -1]) < 3e-3
    seq = ids
    nxt = np.zeros(3, np.int32)
    cur = first
    for _ in range(2):
        seq = np.concatenate([seq, cur[:, None].astype(np.int32)], axis=1)
        m.decode_step(None, nxt)
        assert rel_err(m.logits(3), _hf_forward(sd, cfg, seq)[:, -1]) < 3e-3
        cur = nxt.copy()
    m.close()
