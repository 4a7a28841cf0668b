"""Runs one hot kernel alone on a fixed, small case: the target of `ncu` captures.

    python -m onellm_b200.kernel_cases gate_up|down|qkv|o_proj|lm_head|lm_head_kn|attn|norm|prefill_* [--iters N] [--batch B] [--ctx C]
                                       [--tp T] [--graph]

Each case holds a few hundred MB on the device (more than the 126 MB L2, far less than a
full model) and launches the kernel `--iters` times on rotating buffers; it prints the mean
time per launch from CUDA events and the algorithmic GB/s (TFLOP/s for the prefill cases).
`--tp T` uses the per-rank shapes of T-way tensor parallelism; `--graph` times the launches as
one CUDA graph, i.e. back to back on the device without the host's launch cost (what a decode
step sees).
"""
from __future__ import annotations

import argparse

import torch

import onellm_b200 as ob

H_, D_, HID, INTER, VOCAB = 32, 128, 4096, 11008, 32000


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gate_up", "down", "qkv", "o_proj", "lm_head", "lm_head_kn", "attn", "norm", "gate_up_fused", "qkv_fused", "norm8", "prefill_qkv", "prefill_down", "prefill_gate", "prefill_lm", "prefill_attn"])
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2040)
    ap.add_argument("--graph", action="store_true", help="time a CUDA graph of the launches (device-side back-to-back)")
    ap.add_argument("--tp", type=int, default=1, help="per-rank shapes of a tensor-parallel degree (heads and FFN columns divided)")
    a = ap.parse_args()
    B = a.batch
    global H_, INTER
    H_, INTER = H_ // a.tp, INTER // a.tp
    QKV_N, ATT_K = 3 * HID // a.tp, HID // a.tp
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    st = torch.cuda.current_stream()
    rnd = lambda *s: (0.02 * torch.randn(*s, device="cuda")).half()
    rot = 3
    if a.case == "gate_up":
        rot = max(3, int(400e6 // (HID * INTER * 4)) + 1)
        x, wg, wu = torch.randn(B, HID, device="cuda").half(), [rnd(HID, INTER) for _ in range(rot)], [rnd(HID, INTER) for _ in range(rot)]
        out = torch.empty(B, INTER, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.gemm_swiglu(ob.F16, x, wg[i], wu[i], out, B, INTER, HID)
        nbytes = 2 * HID * INTER * 2 + B * HID * 2 + B * INTER * 2
    elif a.case in ("down", "qkv", "o_proj"):
        K, N = {"down": (INTER, HID), "qkv": (HID, QKV_N), "o_proj": (ATT_K, HID)}[a.case]
        rot = max(3, int(400e6 // (K * N * 2)) + 1)
        x, w = torch.randn(B, K, device="cuda").half(), [rnd(K, N) for _ in range(rot)]
        out = torch.empty(B, N, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.gemm(ob.F16, x, w[i], out, B, N, K, ob.W_KN)
        nbytes = K * N * 2 + B * K * 2 + B * N * 2
    elif a.case in ("gate_up_fused", "qkv_fused"):
        N = INTER if a.case == "gate_up_fused" else 3 * HID
        x, r = torch.randn(B, HID, device="cuda").half(), torch.randn(B, HID, device="cuda").half()
        r2 = torch.empty_like(r)
        g = torch.ones(HID, device="cuda", dtype=torch.float16)
        w = [rnd(HID, N) for _ in range(rot)]
        wu = [rnd(HID, N) for _ in range(rot)] if a.case == "gate_up_fused" else [None] * rot
        out = torch.empty(B, N, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.add_residual_rmsnorm_gemm(ob.F16, x, r, None, g, 1e-5, r2, w[i], wu[i], out, B, N, HID)
        nbytes = (2 if a.case == "gate_up_fused" else 1) * HID * N * 2 + 3 * B * HID * 2 + B * N * 2
    elif a.case == "prefill_attn":
        # context attention of one layer: --batch sequences of --ctx new tokens each (default 2040 -> use e.g. --ctx 512)
        P, S = a.ctx, 2048
        T = B * P
        q = torch.randn(T, 3 * H_ * D_, device="cuda", dtype=torch.float16)
        kc = [torch.randn(B, H_, S, D_, device="cuda", dtype=torch.float16) for _ in range(2)]
        vc = [torch.randn(B, H_, S, D_, device="cuda", dtype=torch.float16) for _ in range(2)]
        rot = 2
        cu = torch.arange(0, B + 1, device="cuda", dtype=torch.int32) * P
        hl = torch.zeros(B, device="cuda", dtype=torch.int32)
        out = torch.empty(T, H_ * D_, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.context_attn(ob.F16, q.data_ptr(), 3 * H_ * D_, kc[i].data_ptr(), vc[i].data_ptr(), H_ * S * D_, S * D_, D_,
                                       cu.data_ptr(), hl.data_ptr(), B, P, H_, H_, D_, D_ ** -0.5, out.data_ptr())
        nbytes = int(B * H_ * 4 * D_ * P * (P + 1) / 2)  # causal-useful flops
    elif a.case.startswith("prefill_"):
        T = 4096 if a.batch == 8 else a.batch
        K, N, lay = {"prefill_qkv": (HID, 3 * HID, ob.W_KN), "prefill_down": (INTER, HID, ob.W_KN),
                     "prefill_gate": (HID, INTER, ob.W_KN), "prefill_lm": (HID, VOCAB, ob.W_NK)}[a.case]
        x = torch.randn(T, K, device="cuda").half()
        w = [rnd(N, K) if lay == ob.W_NK else rnd(K, N) for _ in range(2)]
        rot = 2
        out = torch.empty(T, N, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.gemm(ob.F16, x, w[i], out, T, N, K, lay)
        nbytes = 2 * T * N * K  # flops, reported as "GB/s" = GFLOP/s below
    elif a.case == "norm8":
        xs = [torch.randn(B, HID, device="cuda").half() for _ in range(rot)]
        rs = [torch.randn(B, HID, device="cuda").half() for _ in range(rot)]
        g = torch.ones(HID, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.add_residual_rmsnorm(ob.F16, rs[i], xs[i], None, g, 1e-5, B, HID)
        nbytes = 4 * B * HID * 2
    elif a.case == "lm_head":
        x, w = torch.randn(B, HID, device="cuda").half(), [rnd(VOCAB, HID) for _ in range(2)]
        rot = 2
        out = torch.empty(B, VOCAB, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.gemm(ob.F16, x, w[i], out, B, VOCAB, HID, ob.W_NK)
        nbytes = VOCAB * HID * 2 + B * HID * 2 + B * VOCAB * 2
    elif a.case == "lm_head_kn":
        # the layout the model keeps its LM head in: [hidden, vocab], streamed by the staged kernel
        x, w = torch.randn(B, HID, device="cuda").half(), [rnd(HID, VOCAB) for _ in range(2)]
        rot = 2
        out = torch.empty(B, VOCAB, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.gemm(ob.F16, x, w[i], out, B, VOCAB, HID, ob.W_KN)
        nbytes = VOCAB * HID * 2 + B * HID * 2 + B * VOCAB * 2
    elif a.case == "attn":
        S = a.ctx + 8
        rot = max(2, int(300e6 // (2 * B * H_ * S * D_ * 2)) + 1)
        kc = [torch.randn(B, H_, S, D_, device="cuda", dtype=torch.float16) for _ in range(rot)]
        vc = [torch.randn(B, H_, S, D_, device="cuda", dtype=torch.float16) for _ in range(rot)]
        qkv = torch.randn(B, 3 * H_, D_, device="cuda", dtype=torch.float16)
        o = torch.empty(B, H_, D_, device="cuda", dtype=torch.float16)
        wsb = ob.decode_attn_workspace_bytes(B, H_, D_, S)
        ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
        p, step = qkv.data_ptr(), a.ctx + 1
        fn = lambda i: ob.decode_attn(ob.F16, p, p + H_ * D_ * 2, p + 2 * H_ * D_ * 2, 3 * H_ * D_, 3 * H_ * D_, 3 * H_ * D_,
                                      None, None, None, kc[i], vc[i], H_ * S * D_, S * D_, D_, B, H_, H_, D_, step, step - 1,
                                      D_, 10000.0, D_ ** -0.5, o, H_ * D_, ws, wsb)
        nbytes = 2 * a.ctx * B * H_ * D_ * 2 + 5 * B * H_ * D_ * 2
    else:
        T = 4096
        rot = 4
        xs = [torch.randn(T, HID, device="cuda").half() for _ in range(rot)]
        rs = [torch.randn(T, HID, device="cuda").half() for _ in range(rot)]
        g = torch.ones(HID, device="cuda", dtype=torch.float16)
        fn = lambda i: ob.add_residual_rmsnorm(ob.F16, rs[i], xs[i], None, g, 1e-5, T, HID)
        nbytes = 4 * T * HID * 2 + HID * 2
    for i in range(3):
        fn(i % rot)
    st.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.graph:
        # the launches of one timing pass as a CUDA graph: back to back on the device, no host launch cost
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(a.iters):
                fn(i % rot)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
    else:
        e0.record(st)
        for i in range(a.iters):
            fn(i % rot)
        e1.record(st)
        st.synchronize()
    t = e0.elapsed_time(e1) / a.iters * 1e-3
    if a.case.startswith("prefill_"):
        print(f"{a.case}: {t * 1e6:.1f} us/launch, {nbytes / t / 1e12:.0f} TFLOP/s ({nbytes} flops), timeout flag "
              f"{ob.lib().onellm_gemm_timeout_flag()}")
    else:
        print(f"{a.case}: {t * 1e6:.1f} us/launch, {nbytes / t / 1e9:.0f} GB/s algorithmic ({nbytes} bytes)")


if __name__ == "__main__":
    main()
