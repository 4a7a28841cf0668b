"""The one-to-one replacements for the reference's context-attention launchers, stage by stage against
the CPU oracle, and the whole nine-step sequence of src/layers/attention/context_attention.cpp:101-158
against the fused context-phase kernels."""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

CASES = [
    # B, H, Hkv, D, lens, hist
    (1, 2, 2, 8, [8], [0]),                       # the reference unit tests' tiny shapes
    (2, 8, 2, 64, [5, 9], [0, 3]),
    (3, 8, 8, 128, [17, 1, 40], [0, 30, 7]),
]


def _dev(torch, a, dt):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dt)


def _ivec(torch, a):
    return torch.tensor(list(a), device="cuda", dtype=torch.int32)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("B,H,Hkv,D,lens,hist", CASES)
def test_nine_step_sequence(ob, cuda, orc, dt, B, H, Hkv, D, lens, hist):
    torch = cuda
    tdt, odt = (torch.float16, ob.F16) if dt == "f16" else (torch.float32, ob.F32)
    tol = 2e-3 if dt == "f16" else 1e-5
    rnd = (lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)) if dt == "f16" else (lambda a: np.asarray(a, np.float32))
    rng = np.random.default_rng(100 + B + D)
    T, max_q = int(np.sum(lens)), max(lens)
    ctx = [l + h for l, h in zip(lens, hist)]
    max_k, S = max(ctx), max(ctx) + 5
    QH = H + 2 * Hkv
    QKV = rnd(rng.standard_normal((T, QH, D)))
    bias = rnd(0.1 * rng.standard_normal(QH * D))
    kc0, vc0 = rnd(rng.standard_normal((B, Hkv, S, D))), rnd(rng.standard_normal((B, Hkv, S, D)))

    # ---- oracle, stage by stage
    po, cum, n = orc.cal_padding_offset(lens, max_q)
    mask = orc.build_causal_mask(lens, ctx, max_q, max_k, attend_history=True)
    q_r, k_r, v_r = orc.qkv_bias_rope_transpose(QKV, bias, po, hist, B, max_q, H, Hkv, D, 10000.0)
    kc, vc = kc0.copy(), vc0.copy()
    orc.append_kv_cache(kc, k_r, lens, hist)
    orc.append_kv_cache(vc, v_r, lens, hist)
    k_rep, v_rep = orc.repeat_kv(kc, ctx, H, max_k), orc.repeat_kv(vc, ctx, H, max_k)
    qk = np.einsum("bhqd,bhkd->bhqk", rnd(q_r), rnd(k_rep)).astype(np.float32)
    p = orc.scale_mask_softmax(rnd(qk), mask, D ** -0.5)
    pv = np.einsum("bhqk,bhkd->bhqd", rnd(p), rnd(v_rep)).astype(np.float32)
    out_ref = orc.transpose_remove_padding(rnd(pv), po, T)

    # ---- device, same nine calls
    d_lens, d_hist, d_ctx = _ivec(torch, lens), _ivec(torch, hist), _ivec(torch, ctx)
    d_po = torch.zeros(T, device="cuda", dtype=torch.int32)
    d_cum = torch.zeros(B + 1, device="cuda", dtype=torch.int32)
    assert ob.cal_padding_offset(d_po, d_cum, d_lens, B, max_q) == n == T
    assert np.array_equal(d_po.cpu().numpy(), po) and np.array_equal(d_cum.cpu().numpy(), cum)

    d_mask = torch.full((B, max_q, max_k), -1, device="cuda", dtype=tdt)
    ob.build_causal_mask(odt, d_mask, d_lens, d_ctx, max_q, max_k, B, attend_history=True)
    assert np.array_equal(d_mask.float().cpu().numpy(), mask)
    d_mask0 = torch.full((B, max_q, max_k), -1, device="cuda", dtype=tdt)
    ob.build_causal_mask(odt, d_mask0, d_lens, d_ctx, max_q, max_k, B, attend_history=False)
    assert np.array_equal(d_mask0.float().cpu().numpy(), orc.build_causal_mask(lens, ctx, max_q, max_k, attend_history=False))

    d_q = torch.zeros(B, H, max_q, D, device="cuda", dtype=tdt)
    d_k = torch.zeros(B, Hkv, max_q, D, device="cuda", dtype=tdt)
    d_v = torch.zeros(B, Hkv, max_q, D, device="cuda", dtype=tdt)
    ob.qkv_bias_rope_transpose(odt, d_q, d_k, d_v, _dev(torch, QKV, tdt), _dev(torch, bias, tdt), d_po, d_hist, B, max_q, T, H,
                               Hkv, D, D, 10000.0)
    for got, want in ((d_q, q_r), (d_k, k_r), (d_v, v_r)):
        assert rel_err(got.float().cpu().numpy(), want) < tol

    d_kc, d_vc = _dev(torch, kc0, tdt), _dev(torch, vc0, tdt)
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    ob.append_kv_cache(odt, d_kc, d_k, d_lens, d_hist, B, Hkv, max_q, S, D, flag)
    ob.append_kv_cache(odt, d_vc, d_v, d_lens, d_hist, B, Hkv, max_q, S, D, flag)
    assert int(flag.item()) == 0
    assert rel_err(d_kc.float().cpu().numpy(), kc) < tol and rel_err(d_vc.float().cpu().numpy(), vc) < tol

    d_krep = torch.zeros(B, H, max_k, D, device="cuda", dtype=tdt)
    d_vrep = torch.zeros(B, H, max_k, D, device="cuda", dtype=tdt)
    ob.repeat_kv(odt, d_krep, d_kc, d_ctx, B, H, Hkv, max_k, S, D)
    ob.repeat_kv(odt, d_vrep, d_vc, d_ctx, B, H, Hkv, max_k, S, D)
    assert rel_err(d_krep.float().cpu().numpy(), k_rep) < tol

    d_qk = torch.zeros(B, H, max_q, max_k, device="cuda", dtype=tdt)
    ob.batched_gemm(odt, d_q, d_krep, d_qk, B * H, max_q, max_k, D, trans_b=True)
    assert rel_err(d_qk.float().cpu().numpy(), qk) < 5 * tol
    d_p = torch.zeros_like(d_qk)
    ob.scale_mask_softmax(odt, d_p, d_qk, d_mask, B, H, max_q, max_k, D ** -0.5)
    assert rel_err(d_p.float().cpu().numpy(), p) < 5 * tol
    d_pv = torch.zeros(B, H, max_q, D, device="cuda", dtype=tdt)
    ob.batched_gemm(odt, d_p, d_vrep, d_pv, B * H, max_q, D, max_k)
    d_out = torch.zeros(T, H * D, device="cuda", dtype=tdt)
    ob.transpose_remove_padding(odt, d_out, d_pv, d_po, T, B, max_q, H, D)
    got = d_out.float().cpu().numpy().reshape(T, H, D)
    assert rel_err(got, out_ref) < 5 * tol

    # ---- and the two fused kernels give the same tokens from the same inputs
    if dt == "f16" and D in (64, 128):
        d_qkv = _dev(torch, QKV, tdt)
        f_kc, f_vc = _dev(torch, kc0, tdt), _dev(torch, vc0, tdt)
        ob.qkv_bias_rope_kvcache(odt, d_qkv, _dev(torch, bias, tdt), d_cum, d_hist, f_kc, f_vc, Hkv * S * D, S * D, D, T, B, H, Hkv,
                                 D, D, 10000.0, S, flag)
        fused = torch.zeros(T, H, D, device="cuda", dtype=tdt)
        ob.context_attn(odt, d_qkv, QH * D, f_kc, f_vc, Hkv * S * D, S * D, D, d_cum, d_hist, B, max_q, H, Hkv, D, D ** -0.5, fused)
        assert rel_err(fused.float().cpu().numpy(), out_ref) < 2e-3
        assert rel_err(f_kc.float().cpu().numpy(), kc) < tol and rel_err(f_vc.float().cpu().numpy(), vc) < tol


def test_append_kv_cache_overflow_is_flagged_not_written(ob, cuda):
    torch = cuda
    B, Hkv, max_q, S, D = 1, 2, 4, 6, 8
    src = torch.ones(B, Hkv, max_q, D, device="cuda")
    dst = torch.zeros(B, Hkv, S + 2, D, device="cuda")     # two guard rows behind each head's S rows
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    # rows 4..7 requested, the cache holds 6: rows 4 and 5 are written, 6 and 7 dropped
    view = dst[:, :, :S].contiguous()
    ob.append_kv_cache(ob.F32, view, src, _ivec(torch, [4]), _ivec(torch, [4]), B, Hkv, max_q, S, D, flag)
    assert int(flag.item()) == 1
    assert float(view[:, :, 4:6].min()) == 1.0 and float(view[:, :, :4].abs().max()) == 0.0


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_batched_gemm_layouts(ob, cuda, ta, tb):
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(3)
    batch, m, n, k = 3, 37, 21, 50
    A = torch.randn(batch, k, m, device="cuda", generator=g) if ta else torch.randn(batch, m, k, device="cuda", generator=g)
    Bm = torch.randn(batch, n, k, device="cuda", generator=g) if tb else torch.randn(batch, k, n, device="cuda", generator=g)
    Cm = torch.zeros(batch, m, n, device="cuda")
    ob.batched_gemm(ob.F32, A, Bm, Cm, batch, m, n, k, trans_a=ta, trans_b=tb)
    ref = torch.matmul((A.transpose(1, 2) if ta else A).double(), (Bm.transpose(1, 2) if tb else Bm).double())
    assert float((Cm.double() - ref).abs().max() / ref.abs().max()) < 1e-5


def test_softmax_fully_masked_row_is_zero(ob, cuda):
    torch = cuda
    qk = torch.randn(1, 2, 3, 40, device="cuda")
    mask = torch.ones(1, 3, 40, device="cuda")
    mask[0, 1] = 0
    out = torch.full_like(qk, 7.0)
    ob.scale_mask_softmax(ob.F32, out, qk, mask, 1, 2, 3, 40, 0.5)
    assert float(out[0, :, 1].abs().max()) == 0.0
    ref = torch.softmax(0.5 * qk[0, :, 0].double(), -1)
    assert float((out[0, :, 0].double() - ref).abs().max()) < 1e-6
