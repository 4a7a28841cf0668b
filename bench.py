#!/usr/bin/env python
"""Decode throughput of the LLaMA engine on B200 (Llama-2-7B shape, fp16, batch 8).

A "step" is one decode step for the whole batch (8 new tokens): embedding, 32 layers of
[QKV projection, fused RoPE + masked attention over the KV cache, o_proj, add-residual RMSNorm,
gate/up + SwiGLU, down_proj, add-residual RMSNorm], LM head, top-K (k=50) sampling.  The prompt
(512 random ids per sequence) is prefilled before the timed region, so the context grows from
512 during the run.  Weights are random N(0, 0.02) generated on the device; no dataset or
checkpoint is involved.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                     # the CPU arm (oracle port, host cores)

With N > 1 (launched by torch.distributed.run) the same model is split N-way tensor-parallel
(heads and FFN columns) with an all-reduce after o_proj and down_proj: total work is fixed, so
scaling is "strong".  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_7B = dict(num_layers=32, hidden=4096, head_num=32, kv_head_num=32, head_size=128, inter_size=11008,
                vocab_size=32000)
MODEL_13B = dict(num_layers=40, hidden=5120, head_num=40, kv_head_num=40, head_size=128, inter_size=13824,
                 vocab_size=32000)
WORKLOADS = {
    # name: (model, batch, prompt_len, max_seq_len, top_k, temperature)
    "llama7b_decode_b8_p512": (MODEL_7B, 8, 512, 2048, 50, 1.0),
    "llama7b_decode_b8_ctx2040": (MODEL_7B, 8, 1912, 2048, 50, 1.0),
    # BASELINE.json configs[4] (the tensor-parallel configuration; 133 GB of weights + cache also fit one GPU)
    "llama13b_decode_b64_ctx2000": (MODEL_13B, 64, 2000, 2048, 50, 0.8),
    "llama13b_decode_b64_ctx2040": (MODEL_13B, 64, 1912, 2048, 50, 0.8),
}
METRIC = "decode tokens/s (Llama-7B shape, 1/2/4/8 B200); attn HBM GB/s vs peak"


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (gate/up + SwiGLU at this
# exact shape), from the ncu capture summarised in profiles/skinny_kn_staged_gate_up_m8_4096x11008.md
NCU_TRAFFIC_GATE_UP = 184_805_632
NCU_TRAFFIC_SOURCE = "ncu capture of the same kernel and shape: 180.45 MB read + 4.36 MB written"

def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.

    The nvidia-smi process is started ahead of the warm-up steps, so that its start-up (driver
    initialisation, which stalls launches on every GPU of the box for tens of milliseconds) is over
    before the timed region begins; `mark_start` / `mark_end` bracket the timed region and only the
    samples that arrived between them (plus one period of slack after the end) are summarised.
    """

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 200

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index
        self.t0 = self.t1 = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.PERIOD_MS)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def wait_first(self, timeout_s):
        t_end = time.perf_counter() + timeout_s
        while self.proc and not self.rows and time.perf_counter() < t_end:
            time.sleep(0.01)

    def mark_start(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def __exit__(self, *a):
        if self.proc:
            time.sleep(self.PERIOD_MS * 1e-3 + 0.05)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lo = self.t0 if self.t0 is not None else 0.0
        hi = (self.t1 if self.t1 is not None else float("inf")) + self.PERIOD_MS * 1e-3
        for t, r in self.rows:
            if not (lo <= t <= hi):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "period_ms": self.PERIOD_MS}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle's decode step on the host cores, on a bounded sample of the workload.
# ---------------------------------------------------------------------------------------------
def cpu_decode_sample(model, batch, ctx, n_layers_sample, repeats):
    """Times `n_layers_sample` decoder layers + the LM head of one decode step at context `ctx`
    and scales the layers to the full depth.  Returns (tokens_per_s, description, threads)."""
    import oracle
    from oracle.llama_ref import LlamaRef
    cfg = dict(model, num_layers=n_layers_sample, max_seq_len=ctx + repeats + 1)
    rng = np.random.default_rng(0)
    h, D, H, I, V = cfg["hidden"], cfg["head_size"], cfg["head_num"], cfg["inter_size"], cfg["vocab_size"]
    n = lambda *s: (0.02 * rng.standard_normal(s, dtype=np.float32))
    w = {"norm": np.ones(h, np.float32), "tok_embeddings": n(V, h), "output": None, "layers": []}
    w["output"] = w["tok_embeddings"]  # same shape and cost; saves 0.5 GB of host memory
    for _ in range(n_layers_sample):
        w["layers"].append({"attention_norm": np.ones(h, np.float32), "ffn_norm": np.ones(h, np.float32),
                            "w_qkv": n(h, 3 * H * D), "wo": n(h, h), "w1": n(h, I), "w3": n(h, I), "w2": n(I, h)})
    ref = LlamaRef(cfg, w, batch, storage="f32")
    ref.k_cache[:, :, :, :ctx] = rng.uniform(-1, 1, ref.k_cache[:, :, :, :ctx].shape).astype(np.float32)
    ref.v_cache[:, :, :, :ctx] = rng.uniform(-1, 1, ref.v_cache[:, :, :, :ctx].shape).astype(np.float32)
    ref.cur_len = ctx
    ids = rng.integers(0, V, batch).astype(np.int32)
    t_layers, t_head = [], []
    for _ in range(repeats):
        t0 = time.perf_counter()
        ref.step(ids, lm_head=False)
        t1 = time.perf_counter()
        y = rng.standard_normal((batch, h)).astype(np.float32)
        lg = oracle.gemm(y, w["output"], w_is_nk=True)
        val, idx = oracle.topk(lg, 50)
        oracle.topk_sample(idx, val, np.full(batch, 0.5, np.float32), vocab_size=V, end_id=2)
        t2 = time.perf_counter()
        t_layers.append(t1 - t0)
        t_head.append(t2 - t1)
    per_layer = float(np.median(t_layers)) / n_layers_sample
    step_s = per_layer * model["num_layers"] + float(np.median(t_head))
    desc = (f"{n_layers_sample} of {model['num_layers']} decoder layers + LM head/top-K/sampling of one decode step, "
            f"batch {batch}, context {ctx}, fp32; layers scaled x{model['num_layers'] / n_layers_sample:g} "
            f"(extrapolated), median of {repeats}")
    return batch / step_s, desc, oracle.num_threads(), step_s


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, batch, prompt, smax, top_k, temp = WORKLOADS[workload]
    reps = max(1, args.steps)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_decode_sample(model, batch, prompt, 1, 1)
    tps, desc, threads, step_s = cpu_decode_sample(model, batch, prompt, 1, reps)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "batch": batch, "prompt_len": prompt, "max_seq_len": smax,
                       "parallelism": "host cores (OpenMP)"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def kernel_rooflines(ob, torch, model, batch, ctx, hbm_peak):
    """Times the hot kernels alone (CUDA events on the launching stream, rotating through
    buffers larger than L2) and returns their algorithmic GB/s."""
    h, D, H, I = model["hidden"], model["head_size"], model["head_num"], model["inter_size"]
    st = torch.cuda.current_stream()
    res = {}

    def timeit(fn, n_rot, iters=40, warm=5):
        for i in range(warm):
            fn(i % n_rot)
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for i in range(iters):
            fn(i % n_rot)
        e1.record(st)
        st.synchronize()
        return e0.elapsed_time(e1) / iters * 1e-3

    x = torch.randn(batch, h, device="cuda", dtype=torch.float16)
    # gate/up + SwiGLU: the kernel with the largest share of a step
    n_rot = 3  # 3 x 180 MB of weights > 126 MB L2
    wg = [(0.02 * torch.randn(h, I, device="cuda")).half() for _ in range(n_rot)]
    wu = [(0.02 * torch.randn(h, I, device="cuda")).half() for _ in range(n_rot)]
    out = torch.empty(batch, I, device="cuda", dtype=torch.float16)
    t = timeit(lambda i: ob.gemm_swiglu(ob.F16, x, wg[i], wu[i], out, batch, I, h), n_rot)
    bytes_ = 2 * h * I * 2 + batch * h * 2 + batch * I * 2
    res["gate_up_swiglu"] = {"kernel": "skinny_kn_staged_kernel<1,true,false>", "bytes": bytes_, "us": t * 1e6,
                             "gbs": bytes_ / t / 1e9, "frac": bytes_ / t / 1e9 / hbm_peak}
    del wg, wu
    # down projection
    wd = [(0.02 * torch.randn(I, h, device="cuda")).half() for _ in range(n_rot)]
    a = torch.randn(batch, I, device="cuda", dtype=torch.float16)
    y = torch.empty(batch, h, device="cuda", dtype=torch.float16)
    t = timeit(lambda i: ob.gemm(ob.F16, a, wd[i], y, batch, h, I), n_rot)
    bytes_ = h * I * 2 + batch * I * 2 + batch * h * 2
    res["down_proj"] = {"kernel": "skinny_kn_staged_kernel<1,false,false>", "bytes": bytes_, "us": t * 1e6,
                        "gbs": bytes_ / t / 1e9, "frac": bytes_ / t / 1e9 / hbm_peak}
    del wd
    # decode attention at the given context: one layer's K and V are 2 x B*H*ctx*D*2 bytes
    S = ctx + 8
    n_rot = max(2, int(200e6 // (2 * batch * H * S * D * 2)) + 1)
    kc = [torch.randn(batch, H, S, D, device="cuda", dtype=torch.float16) for _ in range(n_rot)]
    vc = [torch.randn(batch, H, S, D, device="cuda", dtype=torch.float16) for _ in range(n_rot)]
    qkv = torch.randn(batch, 3 * H, D, device="cuda", dtype=torch.float16)
    o = torch.empty(batch, H, D, device="cuda", dtype=torch.float16)
    wsb = ob.decode_attn_workspace_bytes(batch, H, D, S)
    ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
    p = qkv.data_ptr()
    step = ctx + 1

    def attn(i):
        ob.decode_attn(ob.F16, p, p + H * D * 2, p + 2 * H * D * 2, 3 * H * D, 3 * H * D, 3 * H * D, None, None, None,
                       kc[i], vc[i], H * S * D, S * D, D, batch, H, H, D, step, step - 1, D, 10000.0, D ** -0.5, o,
                       H * D, ws, wsb)

    t = timeit(attn, n_rot)
    bytes_ = 2 * ctx * batch * H * D * 2 + 5 * batch * H * D * 2
    res[f"decode_attn_ctx{ctx}"] = {"kernel": "decode_attn_mma_kernel<128,1>", "bytes": bytes_,
                                    "us": t * 1e6, "gbs": bytes_ / t / 1e9, "frac": bytes_ / t / 1e9 / hbm_peak}
    return res


def run_ours(args, workload):
    import torch
    import torch.distributed as dist
    import onellm_b200 as ob

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    model, batch, prompt_len, smax, top_k, temp = WORKLOADS[workload]
    m = ob.Llama(**model, max_seq_len=smax, max_batch=batch, tp_rank=rank, tp_size=world)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        ids = [ob.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        m.init_comm(ids[0])                       # NCCL: the context phase's large all-reduces
        if not args.tp_nccl_only:
            handles = [None] * world              # decode steps: one-shot all-reduce over peer memory
            dist.all_gather_object(handles, m.p2p_handle())
            m.p2p_connect(handles)
            dist.barrier()
    m.init_random(seed=1234, std=0.02)
    m.set_sampling(top_k=top_k, temperature=temp)
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, model["vocab_size"], (batch, prompt_len)).astype(np.int32)
    K, W = args.steps, args.warmup
    if prompt_len + 2 * (K + W) + 2 > smax:
        raise SystemExit("steps + warmup do not fit the KV cache")
    prefill_s = None
    if args.skip_prefill:
        first = prompt[:, -1].copy()
        m.seek(batch, prompt_len, first)  # profiling only: the cache holds zeros, timing is unaffected
    else:
        m.prefill(prompt)                  # warm: scratch allocation, tensor maps, first-use attributes
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = m.prefill(prompt)          # the call copies the ids in and the first tokens out, and synchronises
        prefill_s = time.perf_counter() - t0
    stream = torch.cuda.ExternalStream(m.stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # -- device-resident leg: ids never leave the GPU ------------------------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        clk.wait_first(3.0)  # the sampler's start-up is over before the warm-up, which re-heats the clocks
        for _ in range(W):
            m.decode_step(None, None)
        barrier()
        launches0 = m.state()[1]
        clk.mark_start()
        e0.record(stream)
        for _ in range(K):
            m.decode_step(None, None)
        e1.record(stream)
        barrier()
        clk.mark_end()
    launches = m.state()[1] - launches0
    dev_s = max_over_ranks(e0.elapsed_time(e1) * 1e-3)
    ctx_mid = prompt_len + W + K // 2

    # -- end-to-end leg: pinned host ids in, sampled ids out, every step -----------------------
    h_in = torch.from_numpy(first.copy()).pin_memory()
    h_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
    m.decode_step_raw(h_in.data_ptr(), h_out.data_ptr())
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(K):
        h_in.copy_(h_out)
        m.decode_step_raw(h_in.data_ptr(), h_out.data_ptr())
    e3.record(stream)
    barrier()
    e2e_s = max_over_ranks(e2.elapsed_time(e3) * 1e-3)

    hbm_peak, peak_kind = peaks()
    line = None
    if rank == 0:
        L, h, I, V, H, D = (model[k] for k in ("num_layers", "hidden", "inter_size", "vocab_size", "head_num", "head_size"))
        w_bytes = L * (h * 3 * h + h * h + 3 * h * I) * 2 // world + V * h * 2
        kv_bytes = 2 * ctx_mid * batch * H * D * 2 * L // world
        step_bytes = w_bytes + kv_bytes
        line = {"metric": METRIC, "value": batch * K / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": dev_s / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": workload, "batch": batch, "prompt_len": prompt_len, "max_seq_len": smax,
                           "top_k": top_k, "temperature": temp, "parallelism": f"tp{world}",
                           "allreduce": ("none" if world == 1 else ("nccl" if args.tp_nccl_only else
                                         "one-shot over peer memory, fused with the residual add (NCCL for the context phase)")),
                           "l2": "every step streams its weights and KV cache (>13 GB) once: inputs exceed the 126 MB L2",
                           "context_during_timing": [prompt_len + W, prompt_len + W + K],
                           "prefill": "skipped (cache seek, profiling)" if args.skip_prefill else "done before the timed region"},
                "e2e": {"value": batch * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                        "d2h_bytes_per_step": batch * 4},
                "prefill": (None if prefill_s is None else
                            {"tokens": batch * prompt_len, "ms": prefill_s * 1e3, "tokens_per_s": batch * prompt_len / prefill_s,
                             "tflops": 2.0 * (w_bytes // 2 - V * h + V * h * batch / (batch * prompt_len)) * batch * prompt_len / prefill_s / 1e12,
                             "note": "context phase of the whole batch through the public call (host ids in, first tokens out); "
                                     "flops = 2 x projection weights x tokens, attention not counted"}),
                "gpu_launches": int(launches), "clocks": clk.summary(),
                "step_roofline": {"bound": "hbm", "bytes_per_step_per_gpu": step_bytes,
                                  "achieved": step_bytes / (dev_s / K) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                                  "frac": step_bytes / (dev_s / K) / 1e9 / hbm_peak, "peak_kind": peak_kind}}
    m.close()
    if rank == 0 and args.no_kernels:
        print(json.dumps(line), flush=True)
    elif rank == 0:
        kr = kernel_rooflines(ob, torch, model, batch, 2048 - 8, hbm_peak)
        dom = kr["gate_up_swiglu"]
        line["roofline"] = {"bound": "hbm", "kernel": dom["kernel"], "achieved": dom["gbs"], "peak": hbm_peak,
                            "unit": "GB/s", "frac": dom["frac"], "traffic": NCU_TRAFFIC_GATE_UP, "traffic_source": NCU_TRAFFIC_SOURCE,
                            "peak_kind": peak_kind,
                            "algorithmic_bytes_per_launch": dom["bytes"], "us_per_launch": dom["us"]}
        line["kernels"] = kr
        if world == 1 and not args.no_cpu:
            tps, desc, threads, _ = cpu_decode_sample(model, batch, prompt_len, 1, 3)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_decode_b8_p512", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tp-nccl-only", action="store_true", help="N > 1: keep ncclAllReduce in the decode step (comparison)")
    ap.add_argument("--skip-prefill", action="store_true", help="profiling aid: seek to the prompt length instead of prefilling")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel roofline leg")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_ours(args, args.workload)


if __name__ == "__main__":
    main()
