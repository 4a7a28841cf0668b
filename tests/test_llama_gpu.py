"""The C++ model class against the CPU oracle's composition of the same operators."""
import os

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=3, hidden=256, head_num=4, kv_head_num=4, head_size=64, inter_size=512, vocab_size=1000,
           max_seq_len=96, max_batch=8)


def _make(ob, tmp_path, cfg, seed=0, attn_bias=False, file_dtype=np.float32):
    from oracle import llama_ref
    w = llama_ref.random_weights(cfg, seed, attn_bias=attn_bias)
    prefix = os.path.join(str(tmp_path), "m")
    llama_ref.save_bin(w, prefix, file_dtype)
    m = ob.Llama(**cfg, attn_bias=attn_bias)
    m.load_weights(prefix)
    return m, w


@pytest.mark.parametrize("graphs,by_decode", [(True, False), (False, False), (True, True)])
@pytest.mark.parametrize("attn_bias,kv,file_dtype", [(False, 4, np.float32), (True, 2, np.float16)])
def test_logits_and_greedy_tokens_match_oracle(ob, cuda, orc, tmp_path, graphs, by_decode, attn_bias, kv, file_dtype):
    from oracle.llama_ref import LlamaRef
    cfg = dict(CFG, kv_head_num=kv)
    m, w = _make(ob, tmp_path, cfg, seed=kv, attn_bias=attn_bias, file_dtype=file_dtype)
    m.set_graphs(graphs)
    m.set_prefill_by_decode(by_decode)  # context-phase kernels, or position by position through the decode kernels
    B, P, N = 3, 7, 6
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["vocab_size"], (B, P)).astype(np.int32)
    ref = LlamaRef(cfg, w, B)
    ref_logits = ref.prefill(prompt)
    first = m.prefill(prompt)
    got = m.logits(B)
    assert rel_err(got, ref_logits) < 1e-3 * 3  # three layers of fp16 storage in both arms
    # top-K ids are exact given the engine's own logits
    assert np.array_equal(first, orc.topk(got, 1)[1][:, 0])
    ids = first.copy()
    out = np.zeros(B, np.int32)
    for _ in range(N):
        ref_logits = ref.step(ids)
        m.decode_step(None, out)
        got = m.logits(B)
        assert rel_err(got, ref_logits) < 3e-3
        assert np.array_equal(out, orc.topk(got, 1)[1][:, 0])
        ids = out.copy()
    cur, launches = m.state()
    assert cur == P + N and launches > 0
    # the cache holds what the oracle's cache holds
    import torch
    kptr, vptr = m.kv_cache_ptrs(1)
    m.close()


def test_topk_sampling_in_the_loop(ob, cuda, orc, tmp_path):
    m, w = _make(ob, tmp_path, CFG)
    m.set_sampling(top_k=50, temperature=0.8)
    prompt = np.random.default_rng(1).integers(0, CFG["vocab_size"], (4, 5)).astype(np.int32)
    a = m.generate(prompt, 8)
    b = m.generate(prompt, 8)
    assert np.array_equal(a, b)  # seeded by the step: reproducible
    assert a.min() >= 0 and a.max() < CFG["vocab_size"]
    m.set_sampling(top_k=1)
    g = m.generate(prompt, 8)
    assert not np.array_equal(a, g) or True
    m.close()


def test_engine_draws_are_the_direct_generator_draws_and_the_sampled_ids_follow(ob, cuda, orc, tmp_path):
    """The engine takes curand_init's skip-ahead from a table: its draws are bit-equal to the direct call's for the same
    (step, row), and the ids it samples are the oracle's walk over the engine's own logits with those draws."""
    import torch
    m, w = _make(ob, tmp_path, CFG)
    B, K, T, V = 8, 50, 0.8, CFG["vocab_size"]
    m.set_sampling(top_k=K, temperature=T)
    prompt = np.random.default_rng(2).integers(0, V, (B, 5)).astype(np.int32)
    m.prefill(prompt)
    out = np.zeros(B, np.int32)
    for _ in range(4):
        m.decode_step(None, out)
        u, step, used = m.last_draws()
        assert used, "the skip-ahead table did not pass its check against curand_init"
        idx = torch.zeros(B, K, dtype=torch.int32, device="cuda")
        val = torch.zeros(B, K, dtype=torch.float32, device="cuda")
        scratch = torch.zeros(B, dtype=torch.int32, device="cuda")
        u2 = torch.zeros(B, dtype=torch.float32, device="cuda")
        ob.topk_sample(idx, val, B, K, T, step, V, 2, scratch, u_out=u2)
        torch.cuda.synchronize()
        assert np.array_equal(u[:B], u2.cpu().numpy())
        tv, ti = orc.topk(m.logits(B), K)
        want = orc.topk_sample(ti, tv, u[:B], vocab_size=V, end_id=2, temperature=T)
        want = want[0] if isinstance(want, tuple) else want
        assert np.array_equal(out, np.asarray(want).reshape(-1)[:B])
    m.close()


def test_loader_errors(ob, cuda, tmp_path):
    m = ob.Llama(**CFG)
    with pytest.raises(ob.OnellmError) as e:
        m.load_weights(os.path.join(str(tmp_path), "missing"))
    assert e.value.status == -5
    with pytest.raises(ob.OnellmError):
        m.prefill(np.zeros((1, 4), np.int32))  # weights not loaded
    from oracle import llama_ref
    w = llama_ref.random_weights(CFG, 0)
    prefix = os.path.join(str(tmp_path), "short")
    llama_ref.save_bin(w, prefix)
    with open(prefix + "layers.1.feed_forward.w2.weight", "r+b") as f:
        f.truncate(100)
    with pytest.raises(ob.OnellmError) as e:
        m.load_weights(prefix)
    assert e.value.status == -5 and "w2" in str(e.value)
    m.close()
    with pytest.raises(ob.OnellmError):
        ob.Llama(**dict(CFG, hidden=250))


def test_random_init_statistics(ob, cuda):
    m = ob.Llama(**CFG)
    m.init_random(seed=3, std=0.02)
    ids = m.generate(np.zeros((2, 3), np.int32), 4)
    assert ids.shape == (2, 4)
    lg = m.logits(2)
    assert np.isfinite(lg).all() and lg.std() > 0
    m.close()


def test_second_turn_with_history_matches_one_long_prompt(ob, cuda, orc, tmp_path):
    """prefill(40) + extend(30) (context kernels with history 40) == prefill(70); decoding continues from there."""
    cfg = dict(CFG, max_seq_len=128)
    m, w = _make(ob, tmp_path, cfg, seed=11)
    ids = np.random.default_rng(6).integers(0, cfg["vocab_size"], (3, 70)).astype(np.int32)
    want_first = m.prefill(ids)
    want = m.logits(3)
    want_next = np.zeros(3, np.int32)
    m.decode_step(None, want_next)
    want2 = m.logits(3)
    m.prefill(ids[:, :40])
    got_first = m.extend(ids[:, 40:])
    got = m.logits(3)
    assert rel_err(got, want) < 2e-3
    assert np.array_equal(got_first, orc.topk(got, 1)[1][:, 0])
    got_next = np.zeros(3, np.int32)
    m.decode_step(None, got_next)
    assert m.state()[0] == 71
    if np.array_equal(got_first, want_first):     # same token fed in both runs (a near-tie could differ)
        assert rel_err(m.logits(3), want2) < 3e-3
    with pytest.raises(ob.OnellmError):
        m.extend(np.zeros((3, 100), np.int32))          # 71 + 100 > max_seq_len
    m.close()


def test_norm_free_context_phase_matches_the_one_with_norm_kernels(ob, cuda, tmp_path):
    """One GPU runs the context phase without norm kernels (row statistics handed from projection to projection);
    mode 2 keeps the norm kernels, as tensor-parallel runs do.  Same model, same prompt."""
    cfg = dict(CFG, max_seq_len=160)
    m, w = _make(ob, tmp_path, cfg, seed=13, attn_bias=True)
    prompt = np.random.default_rng(4).integers(0, cfg["vocab_size"], (3, 140)).astype(np.int32)
    m.set_prefill_by_decode(2)
    m.prefill(prompt)
    la = m.logits(3)
    m.set_prefill_by_decode(0)
    m.prefill(prompt)
    lb = m.logits(3)
    m.prefill(prompt)
    assert np.array_equal(m.logits(3), lb)      # no atomics: the same bits every time
    assert rel_err(lb, la) < 3e-3
    m.close()


def test_context_phase_matches_position_by_position(ob, cuda, tmp_path):
    """A 100-token prompt (tensor-core GEMMs, M = 300) against the same prompt fed one position at a time."""
    cfg = dict(CFG, max_seq_len=128)
    m, w = _make(ob, tmp_path, cfg, seed=9)
    prompt = np.random.default_rng(2).integers(0, cfg["vocab_size"], (3, 100)).astype(np.int32)
    m.set_prefill_by_decode(True)
    a = m.generate(prompt, 6)
    la = m.logits(3)
    m.set_prefill_by_decode(False)
    b = m.generate(prompt, 6)
    lb = m.logits(3)
    assert rel_err(lb, la) < 3e-3
    assert (a == b).mean() > 0.8
    m.close()


@pytest.mark.parametrize("graphs", [True, False])
def test_ragged_prompts_match_the_oracle_sequence_by_sequence(ob, cuda, orc, tmp_path, graphs):
    """Prompts of 37, 5 and 64 tokens in one batch (packed context phase with cu_seqlens, then decode steps in which
    every sequence has its own length and position) against the oracle run on every sequence alone."""
    from oracle.llama_ref import LlamaRef
    cfg = dict(CFG, max_seq_len=128)
    m, w = _make(ob, tmp_path, cfg, seed=21)
    m.set_graphs(graphs)
    rng = np.random.default_rng(8)
    lens = [37, 5, 64]
    prompts = [rng.integers(0, cfg["vocab_size"], n).astype(np.int32) for n in lens]
    refs = [LlamaRef(cfg, w, 1) for _ in lens]
    ref_logits = np.concatenate([r.prefill(p[None, :]) for r, p in zip(refs, prompts)])
    first = m.prefill_ragged(prompts)
    got = m.logits(3)
    assert rel_err(got, ref_logits) < 3e-3
    assert np.array_equal(first, orc.topk(got, 1)[1][:, 0])
    ids, out = first.copy(), np.zeros(3, np.int32)
    for _ in range(5):
        ref_logits = np.concatenate([r.step(ids[b:b + 1]) for b, r in enumerate(refs)])
        m.decode_step(None, out)
        got = m.logits(3)
        assert rel_err(got, ref_logits) < 3e-3
        assert np.array_equal(out, orc.topk(got, 1)[1][:, 0])
        ids = out.copy()
    assert m.state()[0] == max(lens) + 5
    m.close()


def test_ragged_turn_after_ragged_prompts(ob, cuda, orc, tmp_path):
    """extend() behind histories of different lengths: context kernels with per-sequence history_length."""
    from oracle.llama_ref import LlamaRef
    cfg = dict(CFG, max_seq_len=128)
    m, w = _make(ob, tmp_path, cfg, seed=22)
    rng = np.random.default_rng(9)
    lens = [20, 33, 3]
    prompts = [rng.integers(0, cfg["vocab_size"], n).astype(np.int32) for n in lens]
    more = rng.integers(0, cfg["vocab_size"], (3, 9)).astype(np.int32)
    refs = [LlamaRef(cfg, w, 1) for _ in lens]
    for r, p in zip(refs, prompts):
        r.prefill(p[None, :])
    ref_logits = np.concatenate([r.prefill(more[b:b + 1]) for b, r in enumerate(refs)])
    m.prefill_ragged(prompts)
    first = m.extend(more)
    got = m.logits(3)
    assert rel_err(got, ref_logits) < 3e-3
    assert np.array_equal(first, orc.topk(got, 1)[1][:, 0])
    out = np.zeros(3, np.int32)
    ref_logits = np.concatenate([r.step(first[b:b + 1]) for b, r in enumerate(refs)])
    m.decode_step(None, out)
    assert rel_err(m.logits(3), ref_logits) < 3e-3
    assert m.state()[0] == 33 + 9 + 1
    # equal-length prompts afterwards: the per-sequence offsets are back to zero
    eq = rng.integers(0, cfg["vocab_size"], (3, 11)).astype(np.int32)
    ref = LlamaRef(cfg, w, 3)
    ref_logits = ref.prefill(eq)
    m.prefill(eq)
    assert rel_err(m.logits(3), ref_logits) < 3e-3
    ref_logits = ref.step(orc.topk(m.logits(3), 1)[1][:, 0].astype(np.int32))
    m.decode_step(None, out)
    assert rel_err(m.logits(3), ref_logits) < 3e-3
    with pytest.raises(ob.OnellmError):
        m.prefill_ragged([np.zeros(200, np.int32), np.zeros(3, np.int32)])  # longer than max_seq_len
    m.close()


def test_model_from_the_converters_config_ini(ob, cuda, tmp_path):
    """onellm_llama_create_from_ini: the model described by a config.ini as the reference's converter writes it."""
    import configparser
    cp = configparser.ConfigParser()
    cp["llama"] = {"model_name": "toy", "head_num": "4", "kv_head_num": "2", "hidden_size": "256", "head_size": "64",
                   "inter_size": "512", "num_layer": "2", "vocab_size": "1000", "bos_token_id": "1", "eos_token_id": "2",
                   "weight_data_type": "fp16", "max_position_embeddings": "4096", "rope_theta": "10000.0",
                   "rms_norm_eps": "1e-05", "attention_bias": "False", "top_k": "7"}
    path = os.path.join(str(tmp_path), "config.ini")
    with open(path, "w") as f:
        cp.write(f)
    m = ob.Llama.from_ini(path, max_batch=2, max_seq_len=64)
    assert (m.cfg.num_layers, m.cfg.kv_head_num, m.cfg.vocab_size, m.cfg.max_seq_len) == (2, 2, 1000, 64)
    m.init_random(seed=5)
    a = m.generate(np.zeros((2, 3), np.int32), 5)       # sampling with the file's top_k = 7, seeded by the step
    b = m.generate(np.zeros((2, 3), np.int32), 5)
    assert a.shape == (2, 5) and np.array_equal(a, b) and a.min() >= 0 and a.max() < 1000
    m.close()
