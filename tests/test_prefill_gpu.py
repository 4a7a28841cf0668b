"""Context-phase kernels against the CPU oracle's restatement of the reference pipeline."""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _r16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("B,H,Hkv,D,lens,hist", [
    (1, 2, 1, 8, [32], [4]),                       # tests/unittests/test_qkv_bias_and_rope.cu:111-143 (S=32, history 4)
    (2, 8, 2, 64, [5, 9], [0, 3]), (3, 32, 32, 128, [17, 1, 40], [0, 100, 7]),
])
def test_qkv_bias_rope_kvcache(ob, cuda, orc, dt, B, H, Hkv, D, lens, hist):
    torch = cuda
    tdt = torch.float16 if dt == "f16" else torch.float32
    rnd = _r16 if dt == "f16" else (lambda a: np.asarray(a, np.float32))
    rng = np.random.default_rng(B + D)
    T, S = int(np.sum(lens)), 160
    if (B, H) == (1, 2):
        QKV, bias = np.ones((T, H + 2 * Hkv, D), np.float32), np.full((H + 2 * Hkv) * D, 2.0, np.float32)  # the reference's inputs
    else:
        QKV, bias = rnd(rng.standard_normal((T, H + 2 * Hkv, D))), rnd(0.1 * rng.standard_normal((H + 2 * Hkv) * D))
    po, cum, n = orc.cal_padding_offset(lens, max(lens))
    q_ref, k_ref, v_ref = orc.qkv_bias_rope_transpose(QKV, bias, po, hist, B, max(lens), H, Hkv, D, 10000.0)
    kc = np.zeros((B, Hkv, S, D), np.float32)
    vc = np.zeros((B, Hkv, S, D), np.float32)
    orc.append_kv_cache(kc, k_ref, lens, hist)
    orc.append_kv_cache(vc, v_ref, lens, hist)
    d_qkv = torch.from_numpy(QKV).to("cuda", tdt)
    d_kc, d_vc = torch.zeros(B, Hkv, S, D, device="cuda", dtype=tdt), torch.zeros(B, Hkv, S, D, device="cuda", dtype=tdt)
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    ob.qkv_bias_rope_kvcache(ob.F16 if dt == "f16" else ob.F32, d_qkv, torch.from_numpy(bias).to("cuda", tdt),
                             torch.from_numpy(cum).cuda(), torch.tensor(hist, device="cuda", dtype=torch.int32), d_kc, d_vc,
                             Hkv * S * D, S * D, D, T, B, H, Hkv, D, D, 10000.0, S, flag)
    tol = 1e-3 if dt == "f16" else 1e-5
    assert int(flag.item()) == 0
    assert rel_err(d_kc.float().cpu().numpy(), kc) < tol and rel_err(d_vc.float().cpu().numpy(), vc) < tol
    got_q = d_qkv.float().cpu().numpy()[:, :H]
    want_q = np.stack([q_ref[(t + po[t]) // max(lens), :, (t + po[t]) % max(lens)] for t in range(T)])
    assert rel_err(got_q, want_q) < tol
    # a position beyond the cache is refused, not written
    ob.qkv_bias_rope_kvcache(ob.F16 if dt == "f16" else ob.F32, d_qkv, None, torch.from_numpy(cum).cuda(),
                             torch.full((B,), S, device="cuda", dtype=torch.int32), d_kc, d_vc, Hkv * S * D, S * D, D, T, B, H,
                             Hkv, D, D, 10000.0, S, flag)
    assert int(flag.item()) == 1


@pytest.mark.parametrize("B,H,Hkv,D,lens,hist", [
    (1, 4, 4, 128, [64], [0]), (2, 8, 2, 64, [5, 130], [0, 3]), (3, 8, 8, 128, [17, 1, 200], [0, 100, 7]),
    (1, 32, 32, 128, [1024], [0]), (8, 4, 1, 128, [65] * 8, [63] * 8),
])
def test_context_attn(ob, cuda, orc, B, H, Hkv, D, lens, hist):
    torch = cuda
    rng = np.random.default_rng(H + D)
    T = int(np.sum(lens))
    S = max(l + h for l, h in zip(lens, hist)) + 8
    qkv = _r16(rng.standard_normal((T, H + 2 * Hkv, D)))
    kc, vc = _r16(rng.standard_normal((B, Hkv, S, D))), _r16(rng.standard_normal((B, Hkv, S, D)))
    ref = orc.context_attn(qkv[:, :H], kc, vc, lens, hist)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    d_qkv = torch.from_numpy(qkv).cuda().half()
    out = torch.zeros(T, H, D, device="cuda", dtype=torch.float16)
    ob.context_attn(ob.F16, d_qkv, (H + 2 * Hkv) * D, torch.from_numpy(kc).cuda().half(), torch.from_numpy(vc).cuda().half(),
                    Hkv * S * D, S * D, D, torch.from_numpy(cu).cuda(), torch.tensor(hist, device="cuda", dtype=torch.int32), B,
                    max(lens), H, Hkv, D, D ** -0.5, out)
    assert rel_err(out.float().cpu().numpy(), ref) < 1e-3


@pytest.mark.parametrize("B,H,Hkv,lens,hist", [(2, 4, 2, [100, 257], [0, 30]), (1, 2, 2, [128], [128])])
def test_context_attn_ignores_whatever_lies_behind_the_sequences(ob, cuda, orc, B, H, Hkv, lens, hist):
    """Cache rows behind history + length hold NaN and Inf bit patterns (a cache that was never cleared): they
    must not reach the result, although whole 128-row tiles of the cache are loaded."""
    torch = cuda
    D = 128
    rng = np.random.default_rng(9)
    T = int(np.sum(lens))
    S = 512
    qkv = _r16(rng.standard_normal((T, H + 2 * Hkv, D)))
    kc, vc = _r16(rng.standard_normal((B, Hkv, S, D))), _r16(rng.standard_normal((B, Hkv, S, D)))
    ref = orc.context_attn(qkv[:, :H], kc, vc, lens, hist)
    for b in range(B):
        end = lens[b] + hist[b]
        kc[b, :, end:] = np.nan
        vc[b, :, end:] = np.nan
        vc[b, :, end::2] = np.inf
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    d_qkv = torch.from_numpy(qkv).cuda().half()
    out = torch.zeros(T, H, D, device="cuda", dtype=torch.float16)
    ob.context_attn(ob.F16, d_qkv, (H + 2 * Hkv) * D, torch.from_numpy(kc).cuda().half(), torch.from_numpy(vc).cuda().half(),
                    Hkv * S * D, S * D, D, torch.from_numpy(cu).cuda(), torch.tensor(hist, device="cuda", dtype=torch.int32), B,
                    max(lens), H, Hkv, D, D ** -0.5, out)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_err(got, ref) < 1e-3
    assert ob.lib().onellm_gemm_timeout_flag() == 0


def test_context_attn_tensor_core_kernel_never_gives_up_a_wait(ob, cuda, orc):
    """8 sequences x 512 tokens x 32 heads (the context phase of the benchmark), launched 50 times: no block may
    raise the time-out flag (a block that gives up a bounded wait skips its stores), and the last launch still
    matches the oracle.  The oracle is run on two of the 32 heads (the per-head arithmetic is identical)."""
    torch = cuda
    B, H, D, P = 8, 32, 128, 512
    rng = np.random.default_rng(5)
    T, S = B * P, P
    qkv = _r16(rng.standard_normal((T, 3 * H, D)))
    kc, vc = _r16(rng.standard_normal((B, H, S, D))), _r16(rng.standard_normal((B, H, S, D)))
    lens, hist = [P] * B, [0] * B
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    d_qkv = torch.from_numpy(qkv).cuda().half()
    d_kc, d_vc = torch.from_numpy(kc).cuda().half(), torch.from_numpy(vc).cuda().half()
    d_cu, d_hist = torch.from_numpy(cu).cuda(), torch.zeros(B, device="cuda", dtype=torch.int32)
    out = torch.zeros(T, H, D, device="cuda", dtype=torch.float16)
    ob.lib().onellm_gemm_timeout_flag()  # clear
    for i in range(50):
        if i == 49:
            out.zero_()
        ob.context_attn(ob.F16, d_qkv, 3 * H * D, d_kc, d_vc, H * S * D, S * D, D, d_cu, d_hist, B, P, H, H, D, D ** -0.5, out)
        if i % 7 == 0:
            torch.cuda.synchronize()  # launches both back to back and into an idle GPU
    torch.cuda.synchronize()
    assert ob.lib().onellm_gemm_timeout_flag() == 0
    got = out.float().cpu().numpy()
    for h in (0, 31):
        ref = orc.context_attn(np.ascontiguousarray(qkv[:, h:h + 1]), np.ascontiguousarray(kc[:, h:h + 1]),
                               np.ascontiguousarray(vc[:, h:h + 1]), lens, hist)
        assert rel_err(got[:, h:h + 1], ref) < 1e-3
