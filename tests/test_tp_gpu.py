"""Tensor parallel engine on two GPUs against the single-GPU engine (skipped with fewer than 2 GPUs)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, hidden=512, head_num=8, kv_head_num=8, head_size=64, inter_size=1024, vocab_size=1000,
           max_seq_len=64, max_batch=4)


def _worker(rank, size, port, prefix, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import onellm_b200 as ob
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=size)  # rendezvous only; the engine owns NCCL
    ids = [ob.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    m = ob.Llama(**CFG, tp_rank=rank, tp_size=size)
    m.init_comm(ids[0])
    m.load_weights(prefix)
    prompt = np.random.default_rng(0).integers(0, CFG["vocab_size"], (3, 6)).astype(np.int32)
    out = m.generate(prompt, 5)
    logits = m.logits(3)
    if rank == 0:
        q.put((out, logits))
    dist.barrier()
    m.close()
    dist.destroy_process_group()


def test_tp2_matches_tp1(ob, cuda, tmp_path):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import llama_ref
    w = llama_ref.random_weights(CFG, 3)
    prefix = os.path.join(str(tmp_path), "m")
    llama_ref.save_bin(w, prefix, np.float16)
    m = ob.Llama(**CFG)
    m.load_weights(prefix)
    prompt = np.random.default_rng(0).integers(0, CFG["vocab_size"], (3, 6)).astype(np.int32)
    want = m.generate(prompt, 5)
    want_logits = m.logits(3)
    m.close()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, prefix, q)) for r in range(2)]
    for p in procs:
        p.start()
    got, got_logits = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert np.abs(got_logits - want_logits).max() / np.abs(want_logits).max() < 3e-3
    # greedy ids agree unless two logits tie within fp16 rounding; report rather than require all
    assert (got == want).mean() > 0.8
