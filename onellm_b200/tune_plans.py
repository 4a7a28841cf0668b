"""Sweeps the launch plan (K split, ring depth) of the four decode-step projections of a model shape.

    python -m onellm_b200.tune_plans [--model 7b|13b] [--batch B] [--ctx C] [--tp T]

The objective is one decoder layer (QKV, attention, o_proj, gate/up, down) timed as a CUDA graph, i.e. the kernels
back to back as a decode step runs them: a plan that is fastest for a projection alone is not always fastest
between its neighbours.  Coordinate descent, two rounds over the four projections; prints the plans the library
would choose, the best plans found and the layer time before and after.  The plans it finds for a shape can be
forced at run time with onellm_gemm_plan_override or added to the table in csrc/skinny_gemm_staged.cu.
"""
from __future__ import annotations

import argparse
import itertools

import onellm_b200 as ob
from onellm_b200 import kernel_cases as kc


def main():
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="7b", choices=sorted(kc.MODELS))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=520)
    ap.add_argument("--tp", type=int, default=1)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    m = kc.MODELS[a.model]
    HID, D, H, INTER = m["hidden"], m["head_size"], m["head_num"] // a.tp, m["inter_size"] // a.tp
    shapes = {"qkv": (3 * H * D, HID, False), "o_proj": (HID, H * D, False), "gate_up": (INTER, HID, True),
              "down": (HID, INTER, False)}
    case = kc.make_case("decode_layer", torch, a.model, a.batch, a.ctx, a.tp)

    def measure(iters=24, reps=4):
        for i in range(2):
            case.fn(i % case.rot)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                case.fn(i % case.rot)
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / iters * 1e3)
        return min(ts)

    cur = {}
    for name, (N, K, dual) in shapes.items():
        ks, nst, blocks = ob.gemm_plan_query(a.batch, N, K, dual)
        cur[name] = (ks, nst)
        print(f"library plan {name}: N={N} K={K} k_split={ks} ring_depth={nst} blocks={blocks}")
    base = best_t = measure()
    print(f"layer with the library's plans: {base:.2f} us")
    for rnd in range(2):
        for name, (N, K, dual) in shapes.items():
            results = []
            for ks, nst in itertools.product(range(1, 9), [3, 4, 5, 6, 7, 8, 9, 10, 12]):
                if ks > 1 and K // 32 // ks < 4:
                    continue
                ob.gemm_plan_override(N, K, dual, ks, nst)
                try:
                    results.append((measure(reps=3), ks, nst))
                except ob.OnellmError:
                    continue
            results.sort()
            print(f"round {rnd} {name}: best (us, k_split, ring_depth) {[(round(t, 2), k, n) for t, k, n in results[:5]]}")
            if results and results[0][0] < best_t - 0.15:
                best_t, cur[name] = results[0][0], (results[0][1], results[0][2])
            ob.gemm_plan_override(N, K, dual, *cur[name])
    print(f"plans {cur}: layer {measure(reps=5):.2f} us (library's plans: {base:.2f} us)")


if __name__ == "__main__":
    main()
