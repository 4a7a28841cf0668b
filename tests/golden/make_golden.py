"""Generates tests/golden/ref_cpu_vectors.npz from the reference's own CPU helper functions.

    python oracle/build_ref.py /path/to/oneLLM     # compiles the reference sources in place
    python tests/golden/make_golden.py

The helpers (tests/unittests/*.cu of the reference: CPUSwiGLU, CPUlinear, cpuEmbedding,
CPUbuildCasualMask, CPUfusedresidandRMSNorm, CPUfunc) are run on seeded inputs on which they are well
defined; inputs and outputs are stored so that the oracle stays pinned to them where the reference tree
is not available.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_lib  # noqa: E402


def main():
    assert ref_lib.load() is not None, "build oracle/_ref first"
    rng = np.random.default_rng(2024)
    d = {}
    d["swiglu_in"] = rng.standard_normal((4, 2, 96)).astype(np.float32) * 3
    d["swiglu_out"] = ref_lib.cpu_swiglu(d["swiglu_in"])
    d["linear_w"], d["linear_x"] = rng.standard_normal((7, 24)).astype(np.float32), rng.standard_normal((24, 12)).astype(np.float32)
    d["linear_out"] = ref_lib.cpu_linear(d["linear_w"], d["linear_x"])
    d["emb_table"], d["emb_ids"] = rng.standard_normal((40, 16)).astype(np.float32), rng.integers(0, 40, 11).astype(np.int32)
    d["emb_out"] = ref_lib.cpu_embedding(d["emb_ids"], d["emb_table"])
    d["mask_q"], d["mask_k"] = np.array([3, 5, 1, 4], np.int32), np.array([5, 5, 4, 9], np.int32)
    d["mask_out"] = ref_lib.cpu_causal_mask(d["mask_q"], d["mask_k"], 6, 10)
    # fused norm: exact in the helper when residual = bias = 0 and the input is constant per row
    d["norm_x"] = np.repeat(rng.standard_normal((3, 1)).astype(np.float32), 64, axis=1)
    d["norm_gamma"] = rng.standard_normal(64).astype(np.float32)
    d["norm_out"] = ref_lib.cpu_fused_resid_rmsnorm(np.zeros((3, 64), np.float32), d["norm_x"], np.zeros(64, np.float32),
                                                    d["norm_gamma"], 1e-5)
    # RoPE: the helper's indexing is self-consistent for a constant input (its own test uses ones and bias 2)
    B, S, H, Hkv, D = 1, 32, 2, 1, 8
    d["rope_hist"] = np.array([4], np.int32)
    d["rope_q"] = ref_lib.cpu_qkv_bias_rope_q(np.ones((B, S, H, D), np.float32), np.full((H + 2 * Hkv) * D, 2.0, np.float32),
                                              d["rope_hist"], B, S, H, Hkv, D, 128, 10000.0)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_vectors.npz"), **d)
    print({k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main()
