"""Tensor parallel engine on two GPUs against the single-GPU engine (skipped with fewer than 2 GPUs)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, hidden=512, head_num=8, kv_head_num=8, head_size=64, inter_size=1024, vocab_size=1000,
           max_seq_len=64, max_batch=4)


def _worker(rank, size, port, prefix, q, p2p=False):
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
    if p2p:  # decode steps over peer memory; the context phase stays on NCCL
        handles = [None] * size
        dist.all_gather_object(handles, m.p2p_handle())
        m.p2p_connect(handles)
        dist.barrier()
    m.load_weights(prefix)
    prompt = np.random.default_rng(0).integers(0, CFG["vocab_size"], (3, 6)).astype(np.int32)
    out = m.generate(prompt, 5)
    logits = m.logits(3)
    err = m.p2p_error() if p2p else 0
    if rank == 0:
        q.put((out, logits, err))
    dist.barrier()
    m.close()
    dist.destroy_process_group()


def _p2p_worker(rank, size, port, q):
    """The all-reduce on its own: 40 calls on alternating buffers, then one call the peer never joins."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    import onellm_b200 as ob
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    rows, h = 8, 4096
    n = rows * h
    comm = ob.P2p(rank, size, n)
    handles = [None] * size
    dist.all_gather_object(handles, comm.handle())
    comm.connect(handles)
    dist.barrier()
    gen = torch.Generator().manual_seed(11)
    resid0 = torch.randn(rows, h, generator=gen).half()
    bias = torch.randn(h, generator=gen).half()
    parts = [[torch.randn(rows, h, generator=gen).half() for _ in range(size)] for _ in range(40)]  # same on every rank
    resid = resid0.cuda()
    d_bias = bias.cuda()
    row_ids = torch.arange(rows, device="cuda", dtype=torch.int32)
    want = resid0.clone()
    ok = True
    for i, per_rank in enumerate(parts):
        which = i % 2
        # the "projection": this rank's partial lands in the send buffer on the stream the all-reduce uses
        dst = comm.send_buffer(which)
        src = per_rank[rank].cuda()
        ob.embedding(ob.F16, row_ids, dst, src, rows, h, rows)   # a row gather with ids 0..rows-1 = a device copy on this stream
        comm.allreduce_add(which, resid, d_bias if which == 0 else None, n, h)
        acc = want.float()
        tot = torch.zeros_like(acc)
        for r in range(size):
            tot += per_rank[r].float()
        acc = tot + acc + (bias.float() if which == 0 else 0.0)
        want = acc.half()
        if i % 10 == 9:
            torch.cuda.synchronize()
            ok = ok and torch.equal(resid.cpu(), want)
    torch.cuda.synchronize()
    # the projection that reduces in its own epilogue: resid += bias + sum_r x_r . W_r, ten calls on alternating buffers
    K, N = 1024, h
    xs = [[(torch.randn(rows, K, generator=gen)).half() for _ in range(size)] for _ in range(10)]
    Ws = [(0.05 * torch.randn(K, N, generator=gen)).half() for _ in range(size)]
    d_W = Ws[rank].cuda()
    resid2 = resid0.cuda()
    want2 = resid0.clone().float()
    for i, per_rank in enumerate(xs):
        which = i % 2
        comm.gemm_allreduce_add(which, per_rank[rank].cuda(), d_W, resid2, d_bias if which == 0 else None, rows, N, K)
        tot = torch.zeros(rows, N)
        for r in range(size):
            tot += (per_rank[r].float() @ Ws[r].float()).half().float()     # every partial crosses the link as fp16
        want2 = (tot + want2 + (bias.float() if which == 0 else 0.0)).half().float()
    torch.cuda.synchronize()
    got2 = resid2.float().cpu()
    fused_err = float((got2 - want2).abs().max() / want2.abs().max())
    everyone = [None] * size
    dist.all_gather_object(everyone, resid2.cpu())
    ok = ok and fused_err < 2e-3 and all(torch.equal(everyone[0], t) for t in everyone)   # bit-identical on every rank
    # the two-shot form of the same exchange (partials to the owner of the token row, finished values back): the same
    # ten calls from the same residual give the same bits; then 64 tokens, which the tcgen05 projection kernel takes
    before = ob.p2p_two_shot_bytes(0)
    resid3 = resid0.cuda()
    for i, per_rank in enumerate(xs):
        which = i % 2
        comm.gemm_allreduce_add(which, per_rank[rank].cuda(), d_W, resid3, d_bias if which == 0 else None, rows, N, K)
    torch.cuda.synchronize()
    ok = ok and torch.equal(resid3, resid2)
    rows64 = 64
    comm64 = ob.P2p(rank, size, rows64 * h)
    handles = [None] * size
    dist.all_gather_object(handles, comm64.handle())
    comm64.connect(handles)
    dist.barrier()
    x64 = [[torch.randn(rows64, K, generator=gen).half() for _ in range(size)] for _ in range(4)]
    r64 = torch.randn(rows64, N, generator=gen).half()
    outs = []
    for form in (1 << 40, 0):  # one-shot, two-shot
        ob.p2p_two_shot_bytes(form)
        res = r64.cuda()
        for i, per_rank in enumerate(x64):
            comm64.gemm_allreduce_add(i % 2, per_rank[rank].cuda(), d_W, res, d_bias if i % 2 == 0 else None, rows64, N, K)
        torch.cuda.synchronize()
        outs.append(res.cpu())
    ob.p2p_two_shot_bytes(before)
    want64 = r64.float()
    for i, per_rank in enumerate(x64):
        tot = torch.zeros(rows64, N)
        for r in range(size):
            tot += (per_rank[r].float() @ Ws[r].float()).half().float()
        want64 = (tot + want64 + (bias.float() if i % 2 == 0 else 0.0)).half().float()
    err64 = float((outs[0].float() - want64).abs().max() / want64.abs().max())
    everyone = [None] * size
    dist.all_gather_object(everyone, outs[1])
    ok = ok and err64 < 2e-3 and torch.equal(outs[0], outs[1]) and all(torch.equal(everyone[0], t) for t in everyone)
    ok = ok and comm64.error() == 0
    comm64.close()
    first_err = comm.error()
    dist.barrier()
    # a call the last rank never joins: the others give up after about a second and say so
    timed_out = None
    if rank != size - 1:
        comm.allreduce_add(0, resid, None, n, h)
        torch.cuda.synchronize()
        timed_out = comm.error()
    dist.barrier()
    q.put((rank, ok, first_err, timed_out))
    comm.close()
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
    got, got_logits, _ = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert np.abs(got_logits - want_logits).max() / np.abs(want_logits).max() < 3e-3
    # greedy ids agree unless two logits tie within fp16 rounding; report rather than require all
    assert (got == want).mean() > 0.8
    # the same with the decode steps' all-reduce over peer memory
    q2 = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port + 1 if port < 65000 else port - 1, prefix, q2, True)) for r in range(2)]
    for p in procs:
        p.start()
    got2, got_logits2, err = q2.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert err == 0
    assert np.abs(got_logits2 - want_logits).max() / np.abs(want_logits).max() < 3e-3
    assert (got2 == want).mean() > 0.8


def test_p2p_allreduce_add_bit_exact_and_bounded_wait(ob, cuda):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    size = 4 if torch.cuda.device_count() >= 4 else 2  # four ranks where the box has them: owners that are not neighbours
    procs = [ctx.Process(target=_p2p_worker, args=(r, size, port, q)) for r in range(size)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in range(size))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, first_err, timed_out in results:
        assert ok and first_err == 0, (rank, ok, first_err)          # every rank holds the same, exact, sums
        assert timed_out == (1 if rank != size - 1 else None)        # the wait ran out, the kernel returned
