"""The oracle against outputs of the REFERENCE's own code.

1. tests/golden/ref_cpu_vectors.npz: inputs and outputs of the reference's CPU helper functions
   (tests/unittests/*.cu), produced by tests/golden/make_golden.py from the reference tree.  Always run.
2. The same helpers called live through oracle/_ref/libonellm_ref.so when that library has been built
   (skipped otherwise).
"""
import os

import numpy as np
import pytest

from conftest import rel_err

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cpu_vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_swiglu_fixture(orc, gold):
    assert rel_err(orc.swiglu(gold["swiglu_in"]), gold["swiglu_out"]) < 1e-6


def test_linear_fixture(orc, gold):
    # the reference helper multiplies weight[m,k] by input[k,n]: x = weight, W = input in the oracle's terms
    assert rel_err(orc.gemm(gold["linear_w"], gold["linear_x"]), gold["linear_out"]) < 1e-6


def test_embedding_fixture(orc, gold):
    assert np.array_equal(orc.embedding(gold["emb_ids"], gold["emb_table"]), gold["emb_out"])


def test_causal_mask_fixture(orc, gold):
    assert np.array_equal(orc.build_causal_mask(gold["mask_q"], gold["mask_k"], 6, 10), gold["mask_out"])


def test_fused_norm_fixture(orc, gold):
    y, r = orc.add_residual_rmsnorm(np.zeros_like(gold["norm_x"]), gold["norm_x"], np.zeros(64, np.float32), gold["norm_gamma"], 1e-5)
    assert rel_err(y, gold["norm_out"]) < 1e-6
    assert rel_err(orc.rmsnorm(gold["norm_x"], gold["norm_gamma"], 1e-5), gold["norm_out"]) < 1e-6


def test_rope_fixture(orc, gold):
    # reference helper: q = 1 + bias 2 = 3 everywhere, rotated at position history + s, pairs (2i, 2i+1),
    # angle position / base^(2i/rot_dim) with rot_dim = 128 although the head is 8 wide (its own test's values)
    B, S, H, D = gold["rope_q"].shape
    x = np.full((S * H, D), 3.0, np.float32)
    pos = np.repeat(np.arange(S, dtype=np.float32) + gold["rope_hist"][0], H)
    want = gold["rope_q"].reshape(S * H, D)
    assert rel_err(orc.rope(x, D, 128, 10000.0, pos), want) < 1e-5


def test_live_reference_helpers(orc):
    from oracle import ref_lib
    if ref_lib.load() is None:
        pytest.skip("oracle/_ref has not been built (needs the reference tree)")
    rng = np.random.default_rng(7)
    inp = rng.standard_normal((5, 2, 200)).astype(np.float32) * 4
    assert rel_err(orc.swiglu(inp), ref_lib.cpu_swiglu(inp)) < 1e-6
    w, x = rng.standard_normal((9, 33)).astype(np.float32), rng.standard_normal((33, 17)).astype(np.float32)
    assert rel_err(orc.gemm(w, x), ref_lib.cpu_linear(w, x)) < 1e-6
    table, ids = rng.standard_normal((100, 24)).astype(np.float32), rng.integers(0, 100, 50).astype(np.int32)
    assert np.array_equal(orc.embedding(ids, table), ref_lib.cpu_embedding(ids, table))
    ql, kl = rng.integers(1, 6, 8).astype(np.int32), rng.integers(6, 12, 8).astype(np.int32)
    assert np.array_equal(orc.build_causal_mask(ql, kl, 6, 12), ref_lib.cpu_causal_mask(ql, kl, 6, 12))
