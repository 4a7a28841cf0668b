"""Tensor-parallel slicing and the all-reduce points, on CPU with two gloo ranks.

Each rank holds its slice of the heads and FFN columns (the cut the engine's weight loader makes),
runs the oracle's decode steps and sums the partial o_proj / down_proj outputs with
torch.distributed (gloo).  The logits must match the single-rank run.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

CFG = dict(num_layers=2, hidden=128, head_num=4, kv_head_num=2, head_size=32, inter_size=192, vocab_size=300,
           max_seq_len=16, max_batch=2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, size, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    from oracle import llama_ref

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a, np.float32))
        dist.all_reduce(t)
        return t.numpy()

    w = llama_ref.random_weights(CFG, 5, attn_bias=True)
    m = llama_ref.LlamaRefTP(CFG, w, 2, rank, size, allreduce, storage="f32")
    prompt = np.random.default_rng(0).integers(0, CFG["vocab_size"], (2, 4)).astype(np.int32)
    logits = m.prefill(prompt)
    logits2 = m.step(np.array([1, 2], np.int32))
    if rank == 0:
        q.put((logits, logits2))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_single_rank():
    from oracle import llama_ref
    import oracle
    oracle.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got, got2 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = llama_ref.random_weights(CFG, 5, attn_bias=True)
    ref = llama_ref.LlamaRef(CFG, w, 2, storage="f32")
    prompt = np.random.default_rng(0).integers(0, CFG["vocab_size"], (2, 4)).astype(np.int32)
    want = ref.prefill(prompt)
    want2 = ref.step(np.array([1, 2], np.int32))
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
    assert np.abs(got2 - want2).max() / np.abs(want2).max() < 1e-5


def test_slices_tile_the_full_tensors():
    from oracle import llama_ref
    w = llama_ref.random_weights(CFG, 1)
    parts = [llama_ref.tp_slice(w, CFG, r, 2) for r in range(2)]
    lw = w["layers"][0]
    assert np.array_equal(np.concatenate([p["layers"][0]["wo"] for p in parts], axis=0), lw["wo"])
    assert np.array_equal(np.concatenate([p["layers"][0]["w1"] for p in parts], axis=1), lw["w1"])
    assert np.array_equal(np.concatenate([p["layers"][0]["w2"] for p in parts], axis=0), lw["w2"])
    H, Hkv, D = CFG["head_num"], CFG["kv_head_num"], CFG["head_size"]
    q = np.concatenate([p["layers"][0]["w_qkv"][:, :H // 2 * D] for p in parts], axis=1)
    assert np.array_equal(q, lw["w_qkv"][:, :H * D])
