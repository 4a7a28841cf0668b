"""The model class at the shapes the benchmark runs, against the CPU oracle's composition.

The other model tests use a toy configuration (hidden 256, head size 64); here the engine runs with the
Llama-2-7B and -13B layer shapes, so that the kernels it picks for them -- the tensor-core decode attention for
head size 128, the tcgen05 context attention and projections, the cluster split-K plans of the 4096 / 11008
(5120 / 13824) projections, the transposed LM-head copy, CUDA-graph replay -- are compared with the oracle as
one composition, with the strides and folded weights the model uses.  Depth is cut to one or two layers: the
oracle computes the prompt position by position.
"""
import os

import numpy as np
import pytest

from conftest import device_view, rel_err

pytestmark = pytest.mark.gpu


def _weights_on_device(torch, cfg, seed, std=0.02):
    """Random fp16-representable weights, generated on the GPU (numpy needs minutes for a 7B-shape layer).
    Returns (float32 numpy dict for the oracle, float16 numpy dict for the files)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    h, D, H, Hkv, I, V, L = (cfg[k] for k in ("hidden", "head_size", "head_num", "kv_head_num", "inter_size",
                                              "vocab_size", "num_layers"))

    def pair(t16):
        return t16.float().cpu().numpy(), t16.cpu().numpy()

    def n(*shape):
        return pair((std * torch.randn(*shape, device="cuda", generator=g)).half())

    def gamma():
        return pair((1 + 0.1 * torch.randn(h, device="cuda", generator=g)).half())

    w32, w16 = {"layers": []}, {"layers": []}
    for name, val in (("norm", gamma()), ("tok_embeddings", n(V, h)), ("output", n(V, h))):
        w32[name], w16[name] = val
    for _ in range(L):
        l32, l16 = {}, {}
        for name, val in (("attention_norm", gamma()), ("ffn_norm", gamma()), ("w_qkv", n(h, (H + 2 * Hkv) * D)),
                          ("wo", n(h, h)), ("w1", n(h, I)), ("w3", n(h, I)), ("w2", n(I, h))):
            l32[name], l16[name] = val
        w32["layers"].append(l32)
        w16["layers"].append(l16)
    return w32, w16


def _save_f16(w16, prefix):
    from oracle.llama_ref import LAYER_FILE_SUFFIX
    for name in ("norm", "tok_embeddings", "output"):
        w16[name].tofile(f"{prefix}.{name}.weight")
    for l, lw in enumerate(w16["layers"]):
        for k, a in lw.items():
            a.tofile(f"{prefix}layers.{l}{LAYER_FILE_SUFFIX[k]}")


@pytest.mark.parametrize("name,cfg,B,P", [
    ("7b", dict(num_layers=2, hidden=4096, head_num=32, kv_head_num=32, head_size=128, inter_size=11008,
                vocab_size=32000, max_seq_len=160, max_batch=8), 8, 130),
    ("13b", dict(num_layers=1, hidden=5120, head_num=40, kv_head_num=40, head_size=128, inter_size=13824,
                 vocab_size=32000, max_seq_len=160, max_batch=8), 8, 130),
])
def test_real_layer_shapes_against_oracle(ob, cuda, orc, tmp_path, name, cfg, B, P):
    torch = cuda
    from oracle.llama_ref import LlamaRef
    w32, w16 = _weights_on_device(torch, cfg, seed=7)
    prefix = os.path.join(str(tmp_path), name)
    _save_f16(w16, prefix)
    del w16
    m = ob.Llama(**cfg)
    m.load_weights(prefix)          # the loader at full row lengths (fp16 files)
    m.set_graphs(True)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, cfg["vocab_size"], (B, P)).astype(np.int32)   # M = B * P > 64, two query tiles per sequence
    ref = LlamaRef(cfg, w32, B)
    ref_logits = ref.prefill(prompt)
    first = m.prefill(prompt)
    got = m.logits(B)
    assert ob.lib().onellm_gemm_timeout_flag() == 0
    assert rel_err(got, ref_logits) < 3e-3
    assert np.array_equal(first, orc.topk(got, 1)[1][:, 0])   # ids exact given the engine's own logits
    ids, out = first.copy(), np.zeros(B, np.int32)
    for _ in range(5):                                         # eager step, captured step, replays
        ref_logits = ref.step(ids)
        m.decode_step(None, out)
        got = m.logits(B)
        assert rel_err(got, ref_logits) < 3e-3
        assert np.array_equal(out, orc.topk(got, 1)[1][:, 0])
        ids = out.copy()
    assert m.state()[0] == P + 5
    # the cache rows of the last layer: context-phase rows and the rows the decode steps appended
    L, Hkv, S, D = cfg["num_layers"], cfg["kv_head_num"], cfg["max_seq_len"], cfg["head_size"]
    kptr, vptr = m.kv_cache_ptrs(L - 1)
    for ptr, want in ((kptr, ref.k_cache[L - 1]), (vptr, ref.v_cache[L - 1])):
        have = device_view(torch, ptr, B * Hkv * S * D).view(B, Hkv, S, D)[:, :, :P + 5].float().cpu().numpy()
        assert rel_err(have, want[:B, :, :P + 5]) < 3e-3   # one or two layers of fp16 storage in front of these rows
    m.close()
