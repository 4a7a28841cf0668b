"""The CPU oracle against the reference's own known answers.

Every case below restates the inputs of one of the reference's unit-test mains
(tests/unittests/*.cu in the oneLLM tree) and the value that test expects, which for these
constant inputs follows from the arithmetic alone.  Cases that need the reference's CPU
helper functions compiled from its tree live in test_oracle_vs_ref.py.
"""
import numpy as np
import pytest

from conftest import rel_err


def test_rmsnorm_known_answer(orc):
    # tests/unittests/test_rmsnorm.cu:64-98: x = 1, gamma = 1, eps = 0.5, 2 tokens x 32 -> 1/sqrt(1.5)
    y = orc.rmsnorm(np.ones((2, 32), np.float32), np.ones(32, np.float32), 0.5)
    assert np.allclose(y, 1.0 / np.sqrt(1.5), atol=1e-6)


def test_fused_add_residual_rmsnorm_known_answer(orc):
    # tests/unittests/test_fused_addres_rms.cu:64-98: decoder_out = 1, residual = 0, bias = 0, gamma = 1, eps = 0.5
    y, r = orc.add_residual_rmsnorm(np.zeros((2, 32), np.float32), np.ones((2, 32), np.float32),
                                    np.zeros(32, np.float32), np.ones(32, np.float32), 0.5)
    assert np.allclose(y, 1.0 / np.sqrt(1.5), atol=1e-6)
    assert np.allclose(r, 1.0, atol=0)


def test_fused_add_residual_rmsnorm_is_sum_then_norm(orc):
    rng = np.random.default_rng(1)
    x, r = rng.standard_normal((5, 64), np.float32), rng.standard_normal((5, 64), np.float32)
    b, g = rng.standard_normal(64, np.float32), rng.standard_normal(64, np.float32)
    y, rn = orc.add_residual_rmsnorm(r, x, b, g, 1e-5)
    s = x + r + b
    assert np.array_equal(rn, s)
    assert rel_err(y, orc.rmsnorm(s, g, 1e-5)) < 1e-6
    y2, rn2 = orc.add_residual_rmsnorm(r, x, None, g, 1e-5)
    assert np.array_equal(rn2, x + r)


def test_decode_attn_known_answer(orc):
    # tests/unittests/test_decoder_masked_attn.cu:113-176: B=1, H=2, Hkv=1, D=16, step=4, max_seq 32,
    # q = k = v = cache = 1, bias = 2: the scores are equal, softmax is uniform, output = V = 1.
    B, H, Hkv, D, step, S = 1, 2, 1, 16, 4, 32
    q, k, v = np.ones((B, H, D), np.float32), np.ones((B, Hkv, D), np.float32), np.ones((B, Hkv, D), np.float32)
    kc, vc = np.zeros((S, B, Hkv, D), np.float32), np.zeros((S, B, Hkv, D), np.float32)
    kc[:step], vc[:step] = 1.0, 1.0
    out = orc.decode_attn(q, k, v, kc, vc, step, rot_dim=0, bias_q=np.full(H * D, 2.0, np.float32),
                          bias_k=np.full(Hkv * D, 2.0, np.float32), cache_layout="sbhd")
    assert np.allclose(out, 1.0, atol=1e-6)
    assert np.allclose(vc[step - 1], 1.0) and np.allclose(kc[step - 1], 3.0)  # k + bias, no rotation


def test_decode_attn_matches_plain_numpy(orc):
    rng = np.random.default_rng(0)
    B, H, Hkv, D, step, S = 2, 4, 2, 32, 9, 16
    q = rng.uniform(-1, 1, (B, H, D)).astype(np.float32)
    k = rng.uniform(-1, 1, (B, Hkv, D)).astype(np.float32)
    v = rng.uniform(-1, 1, (B, Hkv, D)).astype(np.float32)
    kc = rng.uniform(-1, 1, (B, Hkv, S, D)).astype(np.float32)
    vc = rng.uniform(-1, 1, (B, Hkv, S, D)).astype(np.float32)
    kc0, vc0 = kc.copy(), vc.copy()
    out = orc.decode_attn(q, k, v, kc, vc, step, rope_pos=step, cache_layout="bhsd")
    # independent restatement
    pos = np.full(B * H, step, np.float32)
    qr = orc.rope(q.reshape(-1, D), D, D, 10000.0, pos).reshape(B, H, D)
    kr = orc.rope(k.reshape(-1, D), D, D, 10000.0, pos[:B * Hkv]).reshape(B, Hkv, D)
    kc0[:, :, step - 1], vc0[:, :, step - 1] = kr, v
    assert np.array_equal(kc, kc0) and np.array_equal(vc, vc0)
    ref = np.zeros_like(out)
    for b in range(B):
        for h in range(H):
            s = kc0[b, h // 2, :step].astype(np.float64) @ qr[b, h].astype(np.float64) / np.sqrt(D)
            p = np.exp(s - s.max())
            ref[b, h] = (p / p.sum()) @ vc0[b, h // 2, :step].astype(np.float64)
    assert rel_err(out, ref) < 1e-6
    # both cache orders describe the same computation
    kc2 = np.ascontiguousarray(kc0.transpose(2, 0, 1, 3))
    vc2 = np.ascontiguousarray(vc0.transpose(2, 0, 1, 3))
    out2 = orc.decode_attn(q, k, v, kc2, vc2, step, rope_pos=step, cache_layout="sbhd")
    assert np.array_equal(out, out2)


def test_rope_known_values(orc):
    # pairs (2i, 2i+1), angle = pos / base^(2i/rot_dim): src/kernels/decoder_masked_attn.cu:95-108
    D, pos, base = 8, 5.0, 10000.0
    x = np.arange(1, D + 1, dtype=np.float32)[None]
    y = orc.rope(x, D, D, base, np.array([pos], np.float32))[0]
    for i in range(D // 2):
        a = np.float32(pos) / np.float32(base) ** np.float32(2 * i / D)
        c, s = np.cos(a), np.sin(a)
        assert abs(y[2 * i] - (c * x[0, 2 * i] - s * x[0, 2 * i + 1])) < 1e-5
        assert abs(y[2 * i + 1] - (c * x[0, 2 * i + 1] + s * x[0, 2 * i])) < 1e-5
    # rot_dim smaller than the head: the tail is untouched
    y2 = orc.rope(x, D, 4, base, np.array([pos], np.float32))[0]
    assert np.array_equal(y2[4:], x[0, 4:])


def test_swiglu_reference_vector(orc):
    # tests/unittests/test_activation.cu:35-49: input[i] = i over [16, 2, 11008]
    B, I = 16, 11008
    inp = np.arange(B * 2 * I, dtype=np.float32).reshape(B, 2, I)
    out = orc.swiglu(inp)
    g, u = inp[:, 0].astype(np.float64), inp[:, 1].astype(np.float64)
    assert rel_err(out, g / (1 + np.exp(-g)) * u) < 1e-6
    assert out[0, 0] == 0.0


def test_linear_known_answer(orc):
    # tests/unittests/test_linear.cu:52-71: ones [16,16] x ones [16,16] -> 16
    y = orc.gemm(np.ones((16, 16), np.float32), np.ones((16, 16), np.float32))
    assert np.array_equal(y, np.full((16, 16), 16.0, np.float32))
    rng = np.random.default_rng(3)
    x, W = rng.standard_normal((5, 48), np.float32), rng.standard_normal((48, 24), np.float32)
    assert rel_err(orc.gemm(x, W), x.astype(np.float64) @ W.astype(np.float64)) < 1e-6
    assert rel_err(orc.gemm(x, np.ascontiguousarray(W.T), w_is_nk=True), x.astype(np.float64) @ W) < 1e-6


def test_padding_offset_known_answer(orc):
    # tests/unittests/test_cal_paddingoffset.cu:56-58: seq_lens 3,3,3, max_q_len 5 (comment lists
    # padding_offset 0,0,0,2,2,2,4,4,4 and cum_seqlens 0,3,6,9)
    po, cum, n = orc.cal_padding_offset([3, 3, 3], 5)
    assert po.tolist() == [0, 0, 0, 2, 2, 2, 4, 4, 4]
    assert cum.tolist() == [0, 3, 6, 9] and n == 9


def test_causal_mask_known_answer(orc):
    # src/kernels/build_casual_mask.cu:19-25 (comment): q_len 3, k_len 5 (2 rows of history)
    m = orc.build_causal_mask([3], [5], 3, 5)[0]
    assert m.tolist() == [[0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 1, 1, 1]]
    # tests/unittests/test_casual_mask.cu:41-63: q = k = 3 padded to 5 x 5 -> lower triangle of the 3x3 corner
    m = orc.build_causal_mask([3], [3], 5, 5)[0]
    exp = np.zeros((5, 5), np.float32)
    exp[:3, :3] = np.tril(np.ones((3, 3)))
    assert np.array_equal(m, exp)


def test_sampling_reference_case(orc):
    # tests/unittests/test_topK_sampling.cu:6-43: K = 3, values 2,1,0 per row, step 5, end_id 10
    ids = np.array([[4, 5, 6], [7, 10, 9]], np.int32)
    vals = np.array([[2, 1, 0], [2, 1, 0]], np.float32)
    w = np.exp(vals[0] - 2.0)
    for u, want in [(0.0, 0), (w[0] / w.sum() - 1e-3, 0), (w[0] / w.sum() + 1e-3, 1), (0.9999, 2)]:
        out, sl, fin = orc.topk_sample(ids, vals, np.array([u, u], np.float32), vocab_size=30000, end_id=10)
        assert out.tolist() == [ids[0, want], ids[1, want]]
        assert sl.tolist() == [1, 1]
        assert fin.tolist() == [0, 1 if ids[1, want] == 10 else 0]
    # the shipped walk subtracts w_0 = 1 on every iteration (src/kernels/topK_sampling.cu:31-33)
    out, _, _ = orc.topk_sample(ids, vals, np.array([0.9, 0.9], np.float32), vocab_size=30000, end_id=10,
                                literal=True)
    thr = 0.9 * w.sum()
    assert out[0] == ids[0, int(np.floor(thr))]
    # a finished sequence does not grow
    _, sl, _ = orc.topk_sample(ids, vals, np.zeros(2, np.float32), vocab_size=30000, end_id=10,
                               seqlen=[7, 7], finished=[1, 0])
    assert sl.tolist() == [7, 8]


def test_topk_reference_case_and_ties(orc):
    # tests/unittests/test_beamsearch_topK.cu:12-25: probs[i] = i over [batch*beam, 30000], K = 2
    rows, V = 4, 30000
    probs = np.arange(rows * V, dtype=np.float32).reshape(rows, V)
    val, idx = orc.topk(probs, 2, global_ids=True)
    for r in range(rows):
        assert idx[r].tolist() == [r * V + V - 1, r * V + V - 2]
        assert val[r].tolist() == [probs[r, -1], probs[r, -2]]
    x = np.array([[1, 5, 5, 3, 5, 0]], np.float32)
    val, idx = orc.topk(x, 4)
    assert idx.tolist() == [[1, 2, 4, 3]] and val.tolist() == [[5, 5, 5, 3]]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 1000)).astype(np.float32)
    val, idx = orc.topk(x, 50)
    order = np.argsort(-x, axis=1, kind="stable")[:, :50]
    assert np.array_equal(idx, order.astype(np.int32))


def test_prefill_pipeline_pieces(orc):
    """qkv bias+RoPE+transpose, KV append, GQA repeat, softmax, transpose-back compose to context_attn."""
    rng = np.random.default_rng(7)
    B, H, Hkv, D, S_max = 2, 4, 2, 16, 12
    in_len, hist = np.array([3, 5], np.int32), np.array([2, 0], np.int32)
    max_q = int(in_len.max())
    T = int(in_len.sum())
    po, cum, n = orc.cal_padding_offset(in_len, max_q)
    QKV = rng.standard_normal((T, H + 2 * Hkv, D)).astype(np.float32)
    bias = rng.standard_normal((H + 2 * Hkv) * D).astype(np.float32)
    q, k, v = orc.qkv_bias_rope_transpose(QKV, bias, po, hist, B, max_q, H, Hkv, D, 10000.0)
    kc = rng.standard_normal((B, Hkv, S_max, D)).astype(np.float32)
    vc = rng.standard_normal((B, Hkv, S_max, D)).astype(np.float32)
    orc.append_kv_cache(kc, k, in_len, hist)
    orc.append_kv_cache(vc, v, in_len, hist)
    ctx = hist + in_len
    max_k = int(ctx.max())
    kr, vr = orc.repeat_kv(kc, ctx, H, max_k), orc.repeat_kv(vc, ctx, H, max_k)
    mask = orc.build_causal_mask(in_len, ctx, max_q, max_k, attend_history=True)
    qk = np.einsum("bhqd,bhkd->bhqk", q, kr)
    p = orc.scale_mask_softmax(qk, mask, 1 / np.sqrt(D))
    o = np.einsum("bhqk,bhkd->bhqd", p, vr).astype(np.float32)
    packed = orc.transpose_remove_padding(o, po, T)
    # fused form
    q_packed = np.stack([q[(t + po[t]) // max_q, :, (t + po[t]) % max_q] for t in range(T)])
    fused = orc.context_attn(q_packed, kc, vc, in_len, hist)
    assert rel_err(packed, fused) < 1e-5
    # first new token of sequence 0 sits at position hist[0]
    x = QKV[0, 0] + bias[:D]
    assert rel_err(q[0, 0, 0], orc.rope(x[None], D, D, 10000.0, np.array([hist[0]], np.float32))[0]) < 1e-6


def test_embedding(orc):
    rng = np.random.default_rng(2)
    table = rng.standard_normal((50, 8)).astype(np.float32)
    ids = np.array([[3, 49], [0, 7]], np.int32)
    assert np.array_equal(orc.embedding(ids, table), table[ids])
    with pytest.raises(ValueError):
        orc.embedding(np.array([50], np.int32), table)
