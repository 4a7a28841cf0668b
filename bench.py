#!/usr/bin/env python
"""Decode throughput of the LLaMA engine on B200 (Llama-2-7B shape, fp16, batch 8).

A "step" is one decode step for the whole batch (8 new tokens): embedding, 32 layers of
[QKV projection, fused RoPE + masked attention over the KV cache, o_proj, add-residual RMSNorm,
gate/up + SwiGLU, down_proj, add-residual RMSNorm], LM head, top-K (k=50) sampling.  The prompt
(512 random ids per sequence) is prefilled before the timed region, so the context grows from
512 during the run.  Weights are random N(0, 0.02) generated on the device; no dataset or
checkpoint is involved.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                     # the CPU arm (host cores)

The K timed steps are run as a block, the block is repeated from the same cache state until about a
second has been timed, and the median block is reported (`blocks` holds the spread), so that one
number does not hang on 65 ms of GPU time and the clock sampler sees the region.

With N > 1 (launched by torch.distributed.run) the same model is split N-way tensor-parallel
(heads and FFN columns) with the partial o_proj / down_proj outputs summed over the ranks: total
work is fixed, so scaling is "strong".  Outside the timed region the ranks run the same four steps
through both exchanges (peer memory, NCCL) and compare (`tp_check`).  One JSON line is printed by
rank 0; the run fails when a peer wait or a tensor-core wait gave up.
"""
from __future__ import annotations

import argparse
import json
import math
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
    # the tensor-parallel configuration (13B shape, batch 64, context 2048); 133 GB of weights + cache also fit one GPU
    "llama13b_decode_b64_ctx2000": (MODEL_13B, 64, 2000, 2048, 50, 0.8),
    "llama13b_decode_b64_ctx2040": (MODEL_13B, 64, 1912, 2048, 50, 0.8),
}
METRIC = "decode tokens/s (Llama-7B shape, 1/2/4/8 B200); attn HBM GB/s vs peak"

# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of single kernels, keyed by
# (model, batch, tensor-parallel degree, kernel case); each entry names the summary under profiles/ it comes from
NCU_TRAFFIC = {
    ("7b", 8, 1, "gate_up"): (184_644_078, "profiles/skinny_kn_staged_decode_projections_7b_m8.md"),
    ("7b", 8, 1, "qkv"): (104_611_591, "profiles/skinny_kn_staged_decode_projections_7b_m8.md"),
    ("7b", 8, 1, "o_proj"): (33_713_661, "profiles/skinny_kn_staged_decode_projections_7b_m8.md"),
    ("7b", 8, 1, "down"): (94_489_093, "profiles/skinny_kn_staged_decode_projections_7b_m8.md"),
    ("7b", 8, 1, "decode_attn_ctx2040"): (272_267_275, "profiles/decode_attn_mma_f16_b8_h32_ctx2040.md"),
    ("7b", 8, 1, "decode_attn_ctx520"): (68_822_524, "profiles/decode_attn_mma_f16_b8_h32_ctx2040.md"),
    ("13b", 64, 1, "qkv"): (162_289_000, "profiles/skinny_tc_kernel_13b_m64.md"),  # the capture of the 256-column blocks
    ("13b", 64, 1, "lm_head_kn"): (332_545_000, "profiles/skinny_tc_kernel_13b_m64.md"),
    ("13b", 64, 1, "gate_up"): (287_671_566, "profiles/skinny_tc_kernel_13b_m64.md"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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
    PERIOD_MS = 100

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
# CPU arm: the oracle's decode step on the host cores, on a bounded sample of the workload, and the
# reference's own CPU helper functions (compiled from its unit-test sources) on the kernel-level cases.
# ---------------------------------------------------------------------------------------------
def cpu_decode_sample(model, batch, ctx, n_layers_sample, repeats):
    """Times `n_layers_sample` decoder layers + the LM head of one decode step at context `ctx`
    and scales the layers to the full depth.  Returns (tokens_per_s, description, threads, step_s, spread)."""
    import oracle
    from oracle.llama_ref import LlamaRef
    oracle.set_num_threads(host_threads())  # a launcher may have set OMP_NUM_THREADS=1 for its workers
    cfg = dict(model, num_layers=n_layers_sample, max_seq_len=ctx + repeats + 2)
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
    steps = []
    for i in range(repeats + 1):  # the first pass warms the caches and the thread pool
        t0 = time.perf_counter()
        ref.step(ids, lm_head=False)
        t1 = time.perf_counter()
        y = rng.standard_normal((batch, h)).astype(np.float32)
        lg = oracle.gemm(y, w["output"], w_is_nk=True)
        val, idx = oracle.topk(lg, 50)
        oracle.topk_sample(idx, val, np.full(batch, 0.5, np.float32), vocab_size=V, end_id=2)
        t2 = time.perf_counter()
        if i:
            steps.append((t1 - t0) / n_layers_sample * model["num_layers"] + (t2 - t1))
    step_s = float(np.median(steps))
    desc = (f"{n_layers_sample} of {model['num_layers']} decoder layers + LM head/top-K/sampling of one decode step, "
            f"batch {batch}, context {ctx}, fp32; layers scaled x{model['num_layers'] / n_layers_sample:g} "
            f"(extrapolated), median of {repeats} after one warm-up pass")
    spread = {"min_ms": min(steps) * 1e3, "median_ms": step_s * 1e3, "max_ms": max(steps) * 1e3}
    return batch / step_s, desc, oracle.num_threads(), step_s, spread


def reference_helper_timings():
    """The reference's own CPU functions (tests/unittests/*.cu of the reference, compiled unchanged into
    oracle/_ref/libonellm_ref.so), single-threaded as written, on the kernel-level configurations."""
    try:
        from oracle import ref_lib
        lib = ref_lib.load()
    except Exception as e:  # noqa: BLE001
        lib = None
        why = str(e)
    else:
        why = "oracle/_ref/libonellm_ref.so has not been built (needs the reference tree at build time)"
    if lib is None:
        return {"unavailable": why}
    rng = np.random.default_rng(1)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    out = []

    def timed(name, shape, fn, flops_or_bytes=None):
        best = float("inf")
        for _ in range(3):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        out.append({"fn": name, "case": shape, "ms": best * 1e3, "threads": 1})

    x, r, g, b = f(4096, 4096), f(4096, 4096), 1 + 0.1 * f(4096), np.zeros(4096, np.float32)
    import ctypes as C
    g = np.ascontiguousarray(g, np.float32)
    timed("CPUfusedresidandRMSNorm (tests/unittests/test_fused_addres_rms.cu:29-51)", "4096 tokens x hidden 4096, fp32, in place",
          lambda: lib.ref_cpu_fused_resid_rmsnorm(ref_lib.fp(r), ref_lib.fp(x), ref_lib.fp(b), ref_lib.fp(g), C.c_float(1e-5),
                                                  C.c_int(4096), C.c_int(4096)))
    a = f(1024, 2, 11008)
    timed("CPUSwiGLU (tests/unittests/test_activation.cu:11-21)", "1024 tokens x inter 11008, fp32", lambda: ref_lib.cpu_swiglu(a))
    xs, w = f(8, 4096), 0.02 * f(4096, 4096)
    timed("CPUlinear (tests/unittests/test_linear.cu:30-39)", "o_proj of a decode step: 8 tokens, 4096 x 4096 weights, fp32",
          lambda: ref_lib.cpu_linear(xs, w))
    ids, table = rng.integers(0, 32000, 8 * 512).astype(np.int32), f(32000, 4096)
    timed("cpuEmbedding (tests/unittests/test_input_embedding.cu)", "8 x 512 ids, table 32000 x 4096, fp32",
          lambda: ref_lib.cpu_embedding(ids, table))
    qkv, bias = f(1, 256, 96, 128), np.zeros(96 * 128, np.float32)
    timed("CPUfunc: bias + RoPE + transpose (tests/unittests/test_qkv_bias_and_rope.cu:28-92)", "1 sequence x 256 tokens, 32 heads x 128, fp32",
          lambda: ref_lib.cpu_qkv_bias_rope_q(qkv, bias, [0], 1, 256, 32, 32, 128, 128, 10000.0))
    out.append({"fn": "CPUMaskedAttn (tests/unittests/test_decoder_masked_attn.cu:13-101)",
                "unavailable": "its source file does not compile (the test calls the launcher with the wrong arguments); "
                               "the decode-attention arithmetic is timed through the oracle port above"})
    return {"functions": out, "cores": 1}


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, batch, prompt, smax, top_k, temp = WORKLOADS[workload]
    reps = max(5, args.steps)
    tps, desc, threads, step_s, spread = cpu_decode_sample(model, batch, prompt, 1, reps)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "batch": batch, "prompt_len": prompt, "max_seq_len": smax,
                       "parallelism": f"host cores (OpenMP, {threads} threads)",
                       "note": "the reference has no CPU implementation of the whole path (no model class, only unit-test "
                               "helpers): the timed step is the CPU restatement of its kernels (kind: port); the helpers "
                               "themselves are timed under cpu_baseline.reference_helpers"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc,
                             "spread": spread, "reference_helpers": reference_helper_timings()},
            "reference_gpu_kernels": reference_gpu_kernel_timings(),
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def model_key(model):
    return "13b" if model["hidden"] == 5120 else "7b"


def kernel_rooflines(torch, model, batch, world, ctx_list, hbm_peak):
    """The hot kernels of one decode step, each alone at this rank's shapes (CUDA events on the launching
    stream, rotating through buffers larger than L2), as algorithmic GB/s."""
    from onellm_b200 import kernel_cases as kc
    res = {}
    names = [("qkv", None), ("o_proj", None), ("gate_up", None), ("down", None), ("lm_head_kn", None)] + [("attn", c) for c in ctx_list]
    for name, ctx in names:
        case = kc.make_case(name, torch, model_key(model), batch, ctx or 2040, world)
        t = kc.time_case(case, torch, iters=30, warm=5, graph=True)  # replayed as a CUDA graph: a 10 us kernel is not host-bound
        key = name if ctx is None else f"decode_attn_ctx{ctx}"
        res[key] = {"kernel": case.kernel, "bytes": int(case.amount), "us": t * 1e6, "gbs": case.amount / t / 1e9,
                    "frac": case.amount / t / 1e9 / hbm_peak}
        del case
        torch.cuda.empty_cache()
    return res


def config_cases(torch, hbm_peak, tf_peak):
    """The kernel-level configurations next to the decode workload: the fp32 unit-test decode attention, the two
    norm kernels on 4096 x 4096 fp16, and one whole 7B-shape decoder layer of the context phase on 1024 tokens."""
    from onellm_b200 import kernel_cases as kc
    out = {}
    for key, name, kw in (("decode_attn_fp32_b2_h32_d128_step255", "attn_c1", {}),
                          ("rmsnorm_f16_4096x4096", "rmsnorm", {}),
                          ("add_residual_rmsnorm_f16_4096x4096", "norm", {})):
        case = kc.make_case(name, torch, "7b", 8, 2040, 1, **kw)
        t = kc.time_case(case, torch, iters=50, warm=5, graph=True)
        out[key] = {"kernel": case.kernel, "bytes": int(case.amount), "us": t * 1e6, "gbs": case.amount / t / 1e9,
                    "frac_of_hbm": case.amount / t / 1e9 / hbm_peak}
        del case
    case = kc.make_case("prefill_layer", torch, "7b", 1, 1024, 1)
    t = kc.time_case(case, torch, iters=10, warm=3)
    out["prefill_layer_f16_t1024"] = {"launches": case.launches, "flops_dense": case.amount, "ms": t * 1e3,
                                      "tflops": case.amount / t / 1e12, "frac_of_tensor_peak": case.amount / t / 1e12 / tf_peak,
                                      "note": "one decoder layer of the context phase as the model runs it on one GPU: QKV (RMS scale in "
                                              "the epilogue), RoPE + cache write, causal attention, o_proj + residual, gate/up + SwiGLU, "
                                              "down + residual; attention counted over the full square"}
    del case
    out.update(fp32_cases(torch, hbm_peak))
    torch.cuda.empty_cache()
    return out


def _time_rotating(torch, fn, n_buffers, iters=20, warm=3):
    """Mean seconds per call of fn(i) over rotating buffers; CUDA events on the current (legacy default) stream."""
    for i in range(warm):
        fn(i % n_buffers)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i % n_buffers)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


FP32_SHAPES = {"rmsnorm_f32_4096x4096": (4096, 4096), "swiglu_f32_4096x11008": (4096, 11008),
               "embedding_f32_4096_ids_32000x4096": (4096, 4096, 32000)}


def fp32_cases(torch, hbm_peak):
    """This library's kernels in fp32 on the shapes the reference arm times the reference's own (fp32-only) CUDA kernels on."""
    import onellm_b200 as ob
    out = {}
    T, Hd = FP32_SHAPES["rmsnorm_f32_4096x4096"]
    xs = [torch.randn(T, Hd, device="cuda") for _ in range(4)]  # 4 x 67 MB: past the 126 MB L2
    g = torch.ones(Hd, device="cuda")
    t = _time_rotating(torch, lambda i: ob.rmsnorm(ob.F32, xs[i], g, 1e-5, T, Hd), 4)
    nbytes = 2 * T * Hd * 4
    out["rmsnorm_f32_4096x4096"] = {"kernel": "rmsnorm_kernel<float>", "bytes": nbytes, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                                    "frac_of_hbm": nbytes / t / 1e9 / hbm_peak}
    del xs
    T, I = FP32_SHAPES["swiglu_f32_4096x11008"]
    ins = [torch.randn(T, 2, I, device="cuda") for _ in range(2)]
    o = torch.empty(T, I, device="cuda")
    t = _time_rotating(torch, lambda i: ob.swiglu(ob.F32, ins[i], o, T, I), 2)
    nbytes = 3 * T * I * 4
    out["swiglu_f32_4096x11008"] = {"kernel": "swiglu_kernel<float>", "bytes": nbytes, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                                    "frac_of_hbm": nbytes / t / 1e9 / hbm_peak}
    del ins, o
    n, Hd, V = FP32_SHAPES["embedding_f32_4096_ids_32000x4096"]
    table = torch.randn(V, Hd, device="cuda")
    ids = [torch.randint(0, V, (n,), device="cuda", dtype=torch.int32) for _ in range(4)]
    o = [torch.empty(n, Hd, device="cuda") for _ in range(4)]
    t = _time_rotating(torch, lambda i: ob.embedding(ob.F32, ids[i], o[i], table, n, Hd, V), 4)
    nbytes = 2 * n * Hd * 4
    out["embedding_f32_4096_ids_32000x4096"] = {"kernel": "embedding_kernel<float>", "bytes": nbytes, "us": t * 1e6,
                                                "gbs": nbytes / t / 1e9, "frac_of_hbm": nbytes / t / 1e9 / hbm_peak}
    return out


def reference_gpu_kernel_timings():
    """The reference's own CUDA kernels (its launch* functions compiled for sm_100a from the reference tree into
    oracle/_ref/libonellm_ref.so; fp32, the only type its launchers instantiate everywhere), timed with CUDA events on the
    shapes of fp32_cases.  Each export synchronises the device after its launch; the events bracket the launches only."""
    try:
        import torch
        from oracle import ref_lib
        lib = ref_lib.load()
        if lib is None:
            return {"unavailable": "oracle/_ref/libonellm_ref.so has not been built (needs the reference tree at build time)"}
        if not torch.cuda.is_available():
            return {"unavailable": "no GPU"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": str(e)}
    import ctypes as C
    p = lambda t: C.c_void_p(t.data_ptr())
    out = []
    T, Hd = FP32_SHAPES["rmsnorm_f32_4096x4096"]
    xs = [torch.randn(T, Hd, device="cuda") for _ in range(4)]
    g = torch.ones(Hd, device="cuda")
    t = _time_rotating(torch, lambda i: lib.ref_gpu_rmsnorm(p(xs[i]), p(g), C.c_float(1e-5), T, Hd), 4, iters=10)
    out.append({"fn": "launchRMSNorm (src/kernels/rmsnorm_kernel.cu)", "case": "rmsnorm_f32_4096x4096", "us": t * 1e6,
                "gbs": 2 * T * Hd * 4 / t / 1e9})
    del xs
    T, I = FP32_SHAPES["swiglu_f32_4096x11008"]
    ins = [torch.randn(T, 2, I, device="cuda") for _ in range(2)]
    o = torch.empty(T, I, device="cuda")
    t = _time_rotating(torch, lambda i: lib.ref_gpu_swiglu(p(ins[i]), p(o), T, I), 2, iters=10)
    out.append({"fn": "launchAct (src/kernels/activation_kernel.cu)", "case": "swiglu_f32_4096x11008", "us": t * 1e6,
                "gbs": 3 * T * I * 4 / t / 1e9})
    del ins, o
    n, Hd, V = FP32_SHAPES["embedding_f32_4096_ids_32000x4096"]
    table = torch.randn(V, Hd, device="cuda")
    ids = [torch.randint(0, V, (8, n // 8), device="cuda", dtype=torch.int32) for _ in range(4)]
    o = [torch.empty(n, Hd, device="cuda") for _ in range(4)]
    t = _time_rotating(torch, lambda i: lib.ref_gpu_embedding(p(ids[i]), p(o[i]), p(table), 8, n // 8, Hd, V), 4, iters=10)
    out.append({"fn": "launchInputEmbedding (src/kernels/input_embedding.cu)", "case": "embedding_f32_4096_ids_32000x4096",
                "us": t * 1e6, "gbs": 2 * n * Hd * 4 / t / 1e9})
    out.append({"fn": "launchDecoderMaskedMHA (src/kernels/decoder_masked_attn.cu)",
                "unavailable": "the kernel is well defined only for step <= head size (its softmax covers the first blockDim "
                               "logits) and Hkv == H in [S, B, H, D] caches; the bench shapes (step 255-2040) lie outside, so it "
                               "is not launched there.  Parity inside its range: tests/test_ref_kernels_gpu.py"})
    return {"kernels": out, "compare_with": "configs.*_f32_* of the line without --impl reference"}


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
    if args.two_shot_bytes >= 0:
        ob.p2p_two_shot_bytes(args.two_shot_bytes)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        ids = [ob.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        m.init_comm(ids[0])                       # NCCL: the context phase's large all-reduces
        if not args.tp_nccl_only:
            handles = [None] * world              # decode steps: the exchange over peer memory
            dist.all_gather_object(handles, m.p2p_handle())
            m.p2p_connect(handles)
            dist.barrier()
    m.init_random(seed=1234, std=0.02)
    m.set_sampling(top_k=top_k, temperature=temp)
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, model["vocab_size"], (batch, prompt_len)).astype(np.int32)
    K, W = args.steps, args.warmup
    if prompt_len + W + K + 2 > smax:
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

    def max_over_ranks(xs):
        if world == 1:
            return list(xs)
        t = torch.tensor(list(xs), device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    start_len = prompt_len + W

    def device_block():
        """K steps from the state behind the warm-up, ids staying on the device; returns seconds (this rank)."""
        m.seek(batch, start_len, first)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            m.decode_step(None, None)
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1) * 1e-3

    h_in = torch.from_numpy(first.copy()).pin_memory()
    h_out = torch.zeros(batch, dtype=torch.int32).pin_memory()

    def e2e_block():
        """The same K steps through the public call with pinned host ids in and sampled ids out, every step."""
        m.seek(batch, start_len, first)
        h_out.copy_(torch.from_numpy(first))
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            h_in.copy_(h_out)
            m.decode_step_raw(h_in.data_ptr(), h_out.data_ptr())
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1) * 1e-3

    # -- device-resident leg ------------------------------------------------------------------
    with ClockSampler(local) as clk:
        clk.wait_first(3.0)  # the sampler's start-up is over before the warm-up, which re-heats the clocks
        for _ in range(W):
            m.decode_step(None, None)
        probe = max_over_ranks([device_block()])[0]           # untimed: graph capture of this bucket, block length
        R = int(min(64, max(5, math.ceil(args.min_seconds / max(probe, 1e-6)))))
        launches0 = m.state()[1]
        clk.mark_start()
        blocks = [device_block() for _ in range(R)]
        clk.mark_end()
        launches = (m.state()[1] - launches0) // R
    blocks = max_over_ranks(blocks)
    dev_s = float(np.median(blocks))
    ctx_mid = start_len + K // 2

    # -- end-to-end leg -----------------------------------------------------------------------
    e2e_block()
    e2e_blocks = max_over_ranks([e2e_block() for _ in range(min(R, 9))])
    e2e_s = float(np.median(e2e_blocks))

    # -- result checks, outside the timed region ------------------------------------------------
    forced = np.random.default_rng(7).integers(0, model["vocab_size"], (4, batch)).astype(np.int32)

    def four_steps(peer_memory):
        """Four decode steps from the cache state behind the prompt, every step fed the same given ids (a sampled id
        fed back would turn one flipped near-tie into unrelated logits): the logits of every step."""
        if world > 1 and not args.tp_nccl_only:
            m.set_tp_exchange(peer_memory)
        m.seek(batch, prompt_len, first)
        out, logits = np.zeros(batch, np.int32), []
        for t in range(4):
            m.decode_step(forced[t], out)
            logits.append(m.logits(batch))
        return np.stack(logits)

    check = {}
    lg_a = four_steps(True)
    if world > 1 and not args.tp_nccl_only:
        lg_b = four_steps(False)
        m.set_tp_exchange(True)
        scale = max(float(np.max(np.abs(lg_b))), 1e-30)
        check["rel_err_logits"] = float(np.max(np.abs(lg_a - lg_b)) / scale)
        check["ids_equal"] = bool(np.array_equal(np.argmax(lg_a, axis=2), np.argmax(lg_b, axis=2)))
        check["compared"] = ("logits of 4 decode steps from the same cache state and input ids: exchange over peer memory "
                             "vs ncclAllReduce; ids = their argmax.  The two are different fp16 pipelines (the peer-memory "
                             "step sums the ranks' partials and the residual in fp32 and has no norm kernel; the NCCL step "
                             "rounds the partials, their fp16 sum and the normalised activations): they agree to rounding "
                             "accumulated over all layers, about 1e-2 of the largest logit at 32-40 layers, while a wrong "
                             "exchange gives errors of order 1; the run fails above 3e-2")
    if world > 1:
        # every rank must hold bit-identical logits (the peer-memory sums are taken in rank order on every rank)
        bits = np.ascontiguousarray(lg_a.astype(np.float16)).view(np.uint16).astype(np.int64).ravel()
        sig = torch.tensor([int(bits.sum()), int((bits * (np.arange(bits.size, dtype=np.int64) % 8191 + 1)).sum())], device="cuda",
                           dtype=torch.int64)
        lo, hi = sig.clone(), sig.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        check["ranks_bit_identical"] = bool(torch.equal(lo, hi))
    m.set_sampling(top_k=1, temperature=1.0)
    m.seek(batch, prompt_len, first)
    greedy = np.zeros(batch, np.int32)
    m.decode_step(None, greedy)
    lg = m.logits(batch)
    check["greedy_ids_are_argmax_of_logits"] = bool(np.array_equal(greedy, np.argmax(lg, axis=1).astype(np.int32)))
    check["logits_finite"] = bool(np.isfinite(lg_a).all() and np.isfinite(lg).all())
    check["p2p_error"] = int(m.p2p_error()) if world > 1 and not args.tp_nccl_only else 0
    check["tc_timeout_flag"] = int(ob.lib().onellm_gemm_timeout_flag())
    if world > 1:
        t = torch.tensor([check["p2p_error"], check["tc_timeout_flag"]], device="cuda", dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        check["p2p_error"], check["tc_timeout_flag"] = int(t[0].item()), int(t[1].item())
    failed = (check["p2p_error"] != 0 or check["tc_timeout_flag"] != 0 or not check["logits_finite"]
              or check.get("rel_err_logits", 0.0) > 3e-2 or not check.get("ranks_bit_identical", True))

    hbm_peak, tf_peak, peak_kind = peaks()
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
                                         "inside the o_proj / down_proj kernels over peer memory (NCCL for the context phase)")),
                           "two_shot": (bool((world > 2 or ob.p2p_two_shot_bytes() == 0) and
                                             (world - 1) * batch * model["hidden"] * 4 >= ob.p2p_two_shot_bytes())
                                        if world > 1 and not args.tp_nccl_only else None),
                           "l2": "every step streams its weights and KV cache (>13 GB) once: inputs exceed the 126 MB L2",
                           "context_during_timing": [start_len, start_len + K],
                           "prefill": "skipped (cache seek, profiling)" if args.skip_prefill else "done before the timed region"},
                "blocks": {"n": R, "steps_each": K, "ms_min": min(blocks) * 1e3, "ms_median": dev_s * 1e3, "ms_max": max(blocks) * 1e3,
                           "timed_s": float(sum(blocks)),
                           "note": "the K-step block is repeated from the same cache state; value = K steps / median block"},
                "e2e": {"value": batch * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                        "d2h_bytes_per_step": batch * 4, "blocks": len(e2e_blocks)},
                "prefill": (None if prefill_s is None else
                            {"tokens": batch * prompt_len, "ms": prefill_s * 1e3, "tokens_per_s": batch * prompt_len / prefill_s,
                             "tflops": 2.0 * (w_bytes // 2 - V * h + V * h * batch / (batch * prompt_len)) * batch * prompt_len / prefill_s / 1e12,
                             "note": "context phase of the whole batch through the public call (host ids in, first tokens out); "
                                     "flops = 2 x projection weights x tokens, attention not counted"}),
                "gpu_launches": int(launches), "clocks": clk.summary(),
                ("tp_check" if world > 1 else "check"): check,
                "step_roofline": {"bound": "hbm", "bytes_per_step_per_gpu": step_bytes,
                                  "achieved": step_bytes / (dev_s / K) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                                  "frac": step_bytes / (dev_s / K) / 1e9 / hbm_peak, "peak_kind": peak_kind}}
    m.close()
    if rank == 0 and not args.no_kernels:
        kr = kernel_rooflines(torch, model, batch, world, sorted({2040, max(64, ctx_mid // 8 * 8)}), hbm_peak)
        # the kernel with the largest share of a step's bytes at this workload
        per_layer = {"qkv": kr["qkv"]["bytes"], "o_proj": kr["o_proj"]["bytes"], "gate_up": kr["gate_up"]["bytes"],
                     "down": kr["down"]["bytes"], f"decode_attn_ctx{max(64, ctx_mid // 8 * 8)}": 2 * ctx_mid * batch * (H // world) * D * 2}
        dom_name = max(per_layer, key=per_layer.get)
        dom = kr[dom_name]
        traffic = NCU_TRAFFIC.get((model_key(model), batch, world, dom_name))
        line["roofline"] = {"bound": "hbm", "kernel": dom["kernel"], "case": dom_name, "achieved": dom["gbs"], "peak": hbm_peak,
                            "unit": "GB/s", "frac": dom["frac"], "traffic": traffic[0] if traffic else None,
                            "traffic_source": traffic[1] if traffic else "no ncu capture of this shape",
                            "peak_kind": peak_kind, "algorithmic_bytes_per_launch": dom["bytes"], "us_per_launch": dom["us"],
                            "shapes": f"per-rank shapes of tp{world}"}
        line["kernels"] = kr
        if world == 1 and not args.no_cases:
            line["configs"] = config_cases(torch, hbm_peak, tf_peak)
    if rank == 0 and world == 1 and not args.no_cpu:
        tps, desc, threads, _, spread = cpu_decode_sample(model, batch, prompt_len, 1, 5)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc,
                                "spread": spread, "reference_helpers": reference_helper_timings()}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        sys.stderr.write(f"bench: result check failed: {json.dumps(check)}\n")
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_decode_b8_p512", choices=sorted(WORKLOADS))
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the K-step block until this much has been timed")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-cases", action="store_true", help="skip the kernel-level configurations")
    ap.add_argument("--tp-nccl-only", action="store_true", help="N > 1: keep ncclAllReduce in the decode step (comparison)")
    ap.add_argument("--two-shot-bytes", type=int, default=-1,
                    help="N > 1: threshold of onellm_p2p_two_shot_bytes (0 = always two-shot, a huge value = never); default: the library's")
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
