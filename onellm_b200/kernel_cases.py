"""One hot kernel (or one fixed sequence of them) alone on a fixed case: the micro-benchmark behind the
per-kernel figures of `bench.py` and the target of every `ncu` capture summarised under `profiles/`.

    python -m onellm_b200.kernel_cases <case> [--model 7b|13b] [--batch B] [--ctx C] [--tp T] [--iters N] [--graph] [--plain]

Decode-step cases (HBM-bound, reported in GB/s of algorithmic bytes):
    qkv, o_proj, gate_up, down     the four projections as the decode step runs them (onellm_gemm_fused: RMS scale
                                   or residual add in the kernel); --plain times onellm_gemm / onellm_gemm_swiglu
    lm_head_kn, lm_head            LM head on the [hidden, vocab] copy the model keeps / on [vocab, hidden]
    attn                           decode attention over a cache of --ctx rows
    attn_c1                        the fp32 unit-test shape: batch 2, 32 heads x 128, step 255
    norm, rmsnorm                  fused add-residual RMSNorm / RMSNorm on 4096 x hidden fp16
    norm8                          the same on --batch rows
    topk, sample                   top-K (K = 50) over [batch, vocab] fp16 logits / the sampler behind it
    decode_layer                   the five kernels of one decoder layer in the decode step's order (QKV, attention, o_proj,
                                   gate/up, down); with --graph: the layer as the decode step runs it
Context-phase cases (reported in TFLOP/s, except prefill_rope):
    prefill_qkv, prefill_o, prefill_gate, prefill_down, prefill_lm     projections on --batch x --ctx token rows
    prefill_attn                   causal attention of --batch sequences x --ctx tokens
    prefill_rope                   bias + RoPE + KV-cache write (GB/s)
    prefill_layer                  one whole decoder layer on --batch x --ctx tokens as the model runs it: QKV projection (RMS scale
                                   in its epilogue), RoPE + cache write, attention, o_proj (+ residual), gate/up + SwiGLU, down (+ residual)

Every case holds a few hundred MB on the device (more than the 126 MB L2, far less than a model) and runs on
rotating buffers.  `--tp T` uses the per-rank shapes of T-way tensor parallelism; `--graph` times the launches as
one CUDA graph, i.e. back to back on the device without the host's launch cost (what a decode step sees).
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass
from typing import Callable

import onellm_b200 as ob

MODELS = {
    "7b": dict(hidden=4096, head_num=32, head_size=128, inter_size=11008, vocab_size=32000),
    "13b": dict(hidden=5120, head_num=40, head_size=128, inter_size=13824, vocab_size=32000),
}

DECODE_CASES = ["qkv", "o_proj", "gate_up", "down", "lm_head_kn", "lm_head", "attn", "attn_c1", "norm", "rmsnorm", "norm8",
                "topk", "sample", "decode_layer"]
PREFILL_CASES = ["prefill_qkv", "prefill_o", "prefill_gate", "prefill_down", "prefill_lm", "prefill_attn", "prefill_rope",
                 "prefill_layer"]


@dataclass
class Case:
    fn: Callable[[int], None]   # fn(i) launches the case on rotating buffer set i
    rot: int                    # number of buffer sets
    amount: float               # algorithmic bytes (unit "B") or flops (unit "flop") per call of fn
    unit: str
    kernel: str                 # the kernel that dominates the case
    launches: int = 1           # kernel launches per call of fn
    keep: tuple = ()            # buffers kept alive


def _projection_kernel(tokens, dual):
    """Name of the kernel a [K, N] projection of `tokens` rows runs on."""
    if tokens >= ob.gemm_tc_min_tokens() and tokens <= 64:
        return f"skinny_tc_kernel<{'true' if dual else 'false'}>"
    mb = 1 if tokens <= 8 else 2 if tokens <= 16 else 4 if tokens <= 32 else 8
    return f"skinny_kn_staged_kernel<{mb},{'true' if dual else 'false'},false>"


def make_case(name, torch, model="7b", batch=8, ctx=2040, tp=1, plain=False) -> Case:
    m = MODELS[model] if isinstance(model, str) else model
    HID, D, V = m["hidden"], m["head_size"], m["vocab_size"]
    H, INTER = m["head_num"] // tp, m["inter_size"] // tp
    B = batch
    F16 = ob.F16
    half = dict(device="cuda", dtype=torch.float16)
    rnd = lambda *s: (0.02 * torch.randn(*s, device="cuda")).half()
    act = lambda *s: torch.randn(*s, device="cuda").half()
    n_rot = lambda nbytes, target=400e6: max(2, int(target // nbytes) + 1)

    if name in ("qkv", "gate_up"):
        N = 3 * H * D if name == "qkv" else INTER
        dual = name == "gate_up"
        rot = n_rot(HID * N * 2 * (2 if dual else 1))
        x, w = act(B, HID), [rnd(HID, N) for _ in range(rot)]
        wu = [rnd(HID, N) for _ in range(rot)] if dual else [None] * rot
        out = torch.empty(B, N, **half)
        if plain and dual:
            fn = lambda i: ob.gemm_swiglu(F16, x, w[i], wu[i], out, B, N, HID)
        elif plain:
            fn = lambda i: ob.gemm(F16, x, w[i], out, B, N, HID, ob.W_KN)
        else:  # as in the decode step: raw residual stream in, scaled by rsqrt(mean(x^2) + eps) on the way out
            fn = lambda i: ob.gemm_fused(F16, x, w[i], wu[i], out, B, N, HID, 1e-5, None, None)
        nbytes = (2 if dual else 1) * HID * N * 2 + B * HID * 2 + B * N * 2
        kern = _projection_kernel(B, dual)
        return Case(fn, rot, nbytes, "B", kern, keep=(x, w, wu, out))
    if name in ("o_proj", "down"):
        K = H * D if name == "o_proj" else INTER
        rot = n_rot(K * HID * 2)
        x, w = act(B, K), [rnd(K, HID) for _ in range(rot)]
        res = act(B, HID)
        out = torch.empty(B, HID, **half)
        if plain:
            fn = lambda i: ob.gemm(F16, x, w[i], out, B, HID, K, ob.W_KN)
        else:  # as in the decode step: the result is added to the residual stream in the epilogue
            fn = lambda i: ob.gemm_fused(F16, x, w[i], None, res, B, HID, K, -1.0, res, None)
        nbytes = K * HID * 2 + B * K * 2 + (1 if plain else 2) * B * HID * 2
        return Case(fn, rot, nbytes, "B", _projection_kernel(B, False), keep=(x, w, res, out))
    if name in ("lm_head", "lm_head_kn"):
        lay = ob.W_NK if name == "lm_head" else ob.W_KN
        rot = 2
        x = act(B, HID)
        w = [rnd(V, HID) if lay == ob.W_NK else rnd(HID, V) for _ in range(rot)]
        out = torch.empty(B, V, **half)
        fn = lambda i: ob.gemm(F16, x, w[i], out, B, V, HID, lay)
        kern = "skinny_nk_kernel" if lay == ob.W_NK else _projection_kernel(B, False)
        return Case(fn, rot, V * HID * 2 + B * HID * 2 + B * V * 2, "B", kern, keep=(x, w, out))
    if name == "attn":
        S = ctx + 8
        rot = n_rot(2 * B * H * S * D * 2, 300e6)
        kc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        vc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        qkv = torch.randn(B, 3 * H, D, **half)
        o = torch.empty(B, H, D, **half)
        wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
        ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
        p, step = qkv.data_ptr(), ctx + 1
        tickets = torch.zeros(B * H, device="cuda", dtype=torch.int32)
        fn = lambda i: ob.decode_attn(F16, p, p + H * D * 2, p + 2 * H * D * 2, 3 * H * D, 3 * H * D, 3 * H * D, None, None, None,
                                      kc[i], vc[i], H * S * D, S * D, D, B, H, H, D, step, step - 1, D, 10000.0, D ** -0.5, o,
                                      H * D, ws, wsb)
        if plain:  # the one-launch form (splits merged by the last block), which the model class does not use
            fn = lambda i: ob.decode_attn_merged(F16, p, p + H * D * 2, p + 2 * H * D * 2, 3 * H * D, 3 * H * D, 3 * H * D, None,
                                                 None, None, kc[i], vc[i], H * S * D, S * D, D, B, H, H, D, step, None, step - 1, D,
                                                 10000.0, D ** -0.5, o, H * D, ws, wsb, tickets)
        return Case(fn, rot, 2 * ctx * B * H * D * 2 + 5 * B * H * D * 2, "B", "decode_attn_mma_kernel<128,1>",
                    keep=(kc, vc, qkv, o, ws, tickets))
    if name == "attn_c1":
        # the reference's unit-test shape in fp32: 16.9 MB per launch, far below L2 -> rotate over > 126 MB of caches
        Bc, Hc, Dc, Sc, step = 2, 32, 128, 256, 255
        rot = 10
        f32 = dict(device="cuda", dtype=torch.float32)
        kc = [torch.rand(Bc, Hc, Sc, Dc, **f32) * 2 - 1 for _ in range(rot)]
        vc = [torch.rand(Bc, Hc, Sc, Dc, **f32) * 2 - 1 for _ in range(rot)]
        qkv = torch.rand(Bc, 3 * Hc, Dc, **f32) * 2 - 1
        o = torch.empty(Bc, Hc, Dc, **f32)
        wsb = ob.decode_attn_workspace_bytes(Bc, Hc, Dc, Sc)
        ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
        p = qkv.data_ptr()
        fn = lambda i: ob.decode_attn(ob.F32, p, p + Hc * Dc * 4, p + 2 * Hc * Dc * 4, 3 * Hc * Dc, 3 * Hc * Dc, 3 * Hc * Dc, None,
                                      None, None, kc[i], vc[i], Hc * Sc * Dc, Sc * Dc, Dc, Bc, Hc, Hc, Dc, step, step, Dc, 10000.0,
                                      Dc ** -0.5, o, Hc * Dc, ws, wsb)
        return Case(fn, rot, 2 * (step - 1) * Bc * Hc * Dc * 4 + 245760, "B", "decode_attn_kernel<float,128>", keep=(kc, vc, qkv, o, ws))
    if name in ("norm", "rmsnorm", "norm8"):
        T = B if name == "norm8" else 4096
        rot = 4
        xs, rs = [act(T, HID) for _ in range(rot)], [act(T, HID) for _ in range(rot)]
        g = (1 + 0.1 * torch.randn(HID, device="cuda")).half()
        if name == "rmsnorm":
            fn = lambda i: ob.rmsnorm(F16, xs[i], g, 1e-5, T, HID)
            nbytes = 2 * T * HID * 2 + HID * 2
        else:
            fn = lambda i: ob.add_residual_rmsnorm(F16, rs[i], xs[i], None, g, 1e-5, T, HID)
            nbytes = 4 * T * HID * 2 + 2 * HID * 2
        return Case(fn, rot, nbytes, "B", "rmsnorm_kernel", keep=(xs, rs, g))
    if name in ("topk", "sample"):
        rot = 4
        lg = [torch.randn(B, V, **half) for _ in range(rot)]
        val = torch.empty(B, 64, device="cuda", dtype=torch.float32)
        idx = torch.empty(B, 64, device="cuda", dtype=torch.int32)
        if name == "topk":
            fn = lambda i: ob.topk(F16, lg[i], B, V, 50, val, idx)
            return Case(fn, rot, B * V * 2 + B * 50 * 8, "B", "topk_kernel", keep=(lg, val, idx))
        ob.topk(F16, lg[0], B, V, 50, val, idx)
        out = torch.empty(B, device="cuda", dtype=torch.int32)
        fn = lambda i: ob.topk_sample(idx, val, B, 50, 1.0, 7 + i, V, 2, out)
        return Case(fn, rot, B * 50 * 8 + B * 4, "B", "sample_kernel", keep=(lg, val, idx, out))

    if name == "decode_layer":
        S = ctx + 8
        rot = 2
        w_qkv, w_o = [rnd(HID, 3 * H * D) for _ in range(rot)], [rnd(H * D, HID) for _ in range(rot)]
        w_g, w_u, w_d = [rnd(HID, INTER) for _ in range(rot)], [rnd(HID, INTER) for _ in range(rot)], [rnd(INTER, HID) for _ in range(rot)]
        kc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        vc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        res, qkv = act(B, HID), torch.empty(B, 3 * H, D, **half)
        o, a = torch.empty(B, H * D, **half), torch.empty(B, INTER, **half)
        wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
        ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
        p, step = qkv.data_ptr(), ctx + 1

        def fn(i):
            ob.gemm_fused(F16, res, w_qkv[i], None, qkv, B, 3 * H * D, HID, 1e-5, None, None)
            ob.decode_attn(F16, p, p + H * D * 2, p + 2 * H * D * 2, 3 * H * D, 3 * H * D, 3 * H * D, None, None, None, kc[i], vc[i],
                           H * S * D, S * D, D, B, H, H, D, step, step - 1, D, 10000.0, D ** -0.5, o, H * D, ws, wsb)
            ob.gemm_fused(F16, o, w_o[i], None, res, B, HID, H * D, -1.0, res, None)
            ob.gemm_fused(F16, res, w_g[i], w_u[i], a, B, INTER, HID, 1e-5, None, None)
            ob.gemm_fused(F16, a, w_d[i], None, res, B, HID, INTER, -1.0, res, None)

        nbytes = (HID * 3 * H * D + H * D * HID + 3 * HID * INTER) * 2 + 2 * ctx * B * H * D * 2
        return Case(fn, rot, nbytes, "B", "skinny_kn_staged_kernel + decode_attn_mma_kernel", launches=5,
                    keep=(w_qkv, w_o, w_g, w_u, w_d, kc, vc, res, qkv, o, a, ws))

    # ---- context phase: --batch sequences of --ctx new tokens each ---------------------------------------
    P = ctx
    T = B * P
    if name in ("prefill_qkv", "prefill_o", "prefill_gate", "prefill_down", "prefill_lm"):
        K, N, lay = {"prefill_qkv": (HID, 3 * H * D, ob.W_KN), "prefill_o": (H * D, HID, ob.W_KN), "prefill_gate": (HID, INTER, ob.W_KN),
                     "prefill_down": (INTER, HID, ob.W_KN), "prefill_lm": (HID, V, ob.W_KN)}[name]
        rot = 2
        x = act(T, K)
        w = [rnd(K, N) for _ in range(rot)]
        out = torch.empty(T, N, **half)
        if name == "prefill_gate":
            wu = [rnd(K, N) for _ in range(rot)]
            fn = lambda i: ob.gemm_swiglu(F16, x, w[i], wu[i], out, T, N, K)
            return Case(fn, rot, 4.0 * T * N * K, "flop", "gemm_tc_kernel<2>", keep=(x, w, wu, out))
        fn = lambda i: ob.gemm(F16, x, w[i], out, T, N, K, lay)
        return Case(fn, rot, 2.0 * T * N * K, "flop", "gemm_tc_kernel<0>", keep=(x, w, out))
    S = max(2048, P)
    cu = torch.arange(0, B + 1, device="cuda", dtype=torch.int32) * P
    hl = torch.zeros(B, device="cuda", dtype=torch.int32)
    if name == "prefill_attn":
        rot = 2
        q = torch.randn(T, 3 * H * D, **half)
        kc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        vc = [torch.randn(B, H, S, D, **half) for _ in range(rot)]
        out = torch.empty(T, H * D, **half)
        fn = lambda i: ob.context_attn(F16, q, 3 * H * D, kc[i], vc[i], H * S * D, S * D, D, cu, hl, B, P, H, H, D, D ** -0.5, out)
        return Case(fn, rot, float(B * H * 4 * D * P * (P + 1) / 2), "flop", "context_attn_tc_kernel", keep=(q, kc, vc, out, cu, hl))
    if name == "prefill_rope":
        rot = 3
        q = [torch.randn(T, 3 * H * D, **half) for _ in range(rot)]
        kc, vc = torch.zeros(B, H, S, D, **half), torch.zeros(B, H, S, D, **half)
        flag = torch.zeros(1, device="cuda", dtype=torch.int32)
        fn = lambda i: ob.qkv_bias_rope_kvcache(F16, q[i], None, cu, hl, kc, vc, H * S * D, S * D, D, T, B, H, H, D, D, 10000.0, S, flag)
        # reads the packed rows, writes q and k back in place and k, v into the cache
        return Case(fn, rot, T * 3 * H * D * 2 + T * 2 * H * D * 2 + T * 2 * H * D * 2, "B", "qkv_rope_kvcache_vec_kernel",
                    keep=(q, kc, vc, flag, cu, hl))
    if name == "prefill_layer":
        rot = 2
        w_qkv, w_o = [rnd(HID, 3 * H * D) for _ in range(rot)], [rnd(H * D, HID) for _ in range(rot)]
        w_g, w_u, w_d = [rnd(HID, INTER) for _ in range(rot)], [rnd(HID, INTER) for _ in range(rot)], [rnd(INTER, HID) for _ in range(rot)]
        g = torch.ones(HID, **half)
        x0 = act(T, HID)
        y, res = torch.empty(T, HID, **half), torch.zeros(T, HID, **half)
        qkv, attn, a = torch.empty(T, 3 * H * D, **half), torch.empty(T, H * D, **half), torch.empty(T, INTER, **half)
        kc, vc = torch.zeros(B, H, S, D, **half), torch.zeros(B, H, S, D, **half)
        flag = torch.zeros(1, device="cuda", dtype=torch.int32)

        n_parts = ob.gemm_rows_parts(HID)
        ss_a = torch.ones(T, n_parts, device="cuda", dtype=torch.float32)
        ss_b = torch.ones(T, n_parts, device="cuda", dtype=torch.float32)

        def fn(i):
            # one layer of the context phase as the model runs it on one GPU: what LlamaContextDecoder::forward does per layer
            # (src/layers/decoder/context_decoder.cpp:95-131) without norm kernels -- the projections behind a norm scale their
            # rows from the statistics the projection before them left, o_proj and down_proj add into the residual stream
            ob.gemm_rows(F16, res, w_qkv[i], None, qkv, T, 3 * H * D, HID, row_ss=ss_a, ss_parts=n_parts)
            ob.qkv_bias_rope_kvcache(F16, qkv, None, cu, hl, kc, vc, H * S * D, S * D, D, T, B, H, H, D, D, 10000.0, S, flag)
            ob.context_attn(F16, qkv, 3 * H * D, kc, vc, H * S * D, S * D, D, cu, hl, B, P, H, H, D, D ** -0.5, attn)
            ob.gemm_rows(F16, attn, w_o[i], None, res, T, HID, H * D, resid=res, row_ss_out=ss_b)
            ob.gemm_rows(F16, res, w_g[i], w_u[i], a, T, INTER, HID, row_ss=ss_b, ss_parts=n_parts)
            ob.gemm_rows(F16, a, w_d[i], None, res, T, HID, INTER, resid=res, row_ss_out=ss_a)

        # dense flops: projections + both attention products over the full square (the causal half is skipped)
        flops = 2.0 * T * HID * (3 * H * D + H * D) + 6.0 * T * HID * INTER + 4.0 * B * H * D * P * P
        return Case(fn, rot, flops, "flop", "gemm_tc_kernel", launches=6,
                    keep=(w_qkv, w_o, w_g, w_u, w_d, g, x0, y, res, qkv, attn, a, kc, vc, flag, cu, hl, ss_a, ss_b))
    raise ValueError(f"unknown case {name}")


def time_case(case: Case, torch, iters=20, warm=5, graph=False) -> float:
    """Mean seconds per call of case.fn: CUDA events on the launching stream, after warm-up, rotating buffers."""
    st = torch.cuda.current_stream()
    for i in range(warm):
        case.fn(i % case.rot)
    st.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                case.fn(i % case.rot)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
    else:
        e0.record(st)
        for i in range(iters):
            case.fn(i % case.rot)
        e1.record(st)
        st.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=DECODE_CASES + PREFILL_CASES)
    ap.add_argument("--model", default="7b", choices=sorted(MODELS))
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=None, help="cache rows (decode cases, default 2040) / new tokens per sequence (prefill cases, default 512)")
    ap.add_argument("--graph", action="store_true", help="time a CUDA graph of the launches (device-side back-to-back)")
    ap.add_argument("--tp", type=int, default=1, help="per-rank shapes of a tensor-parallel degree (heads and FFN columns divided)")
    ap.add_argument("--plain", action="store_true", help="projections through onellm_gemm / onellm_gemm_swiglu instead of onellm_gemm_fused; attn: onellm_decode_attn_merged (splits merged inside the kernel) instead of onellm_decode_attn")
    a = ap.parse_args()
    ctx = a.ctx if a.ctx is not None else (512 if a.case.startswith("prefill_") else 2040)
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    case = make_case(a.case, torch, a.model, a.batch, ctx, a.tp, a.plain)
    t = time_case(case, torch, iters=a.iters, warm=3, graph=a.graph)
    flag = ob.lib().onellm_gemm_timeout_flag()
    if case.unit == "flop":
        print(f"{a.case}: {t * 1e6:.1f} us/call, {case.amount / t / 1e12:.0f} TFLOP/s ({case.amount:.0f} flops, {case.launches} launch(es)), "
              f"time-out flag {flag}")
    else:
        print(f"{a.case}: {t * 1e6:.1f} us/launch, {case.amount / t / 1e9:.0f} GB/s algorithmic ({int(case.amount)} bytes), kernel {case.kernel}")


if __name__ == "__main__":
    main()
