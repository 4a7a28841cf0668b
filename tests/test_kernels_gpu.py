"""Parity of the CUDA kernels with the CPU oracle, through the C ABI.

Tolerances (relative to the largest magnitude of the reference tensor, see conftest.rel_err):
1e-5 for fp32, 1e-3 for fp16 storage -- the figures the project states for this path.
Integer results (top-K ids, sampled ids) must be identical.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

TOL = {"f32": 1e-5, "f16": 1e-3}


def _dt(torch, name):
    return torch.float32 if name == "f32" else torch.float16


def _round(a, name):
    return a.astype(np.float16).astype(np.float32) if name == "f16" else a.astype(np.float32)


def _dev(torch, a, name):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype=_dt(torch, name))


def _run_decode_attn(ob, torch, orc, dt, B, H, Hkv, D, step, S, layout, seed, bias=False, rope_pos=None,
                     rot_dim=None, use_step_dev=False):
    rng = np.random.default_rng(seed)
    u = lambda *s: _round(rng.uniform(-1, 1, s), dt)
    qkv = u(B, H + 2 * Hkv, D)  # the fused buffer the layer hands to the kernel
    shape = (B, Hkv, S, D) if layout == "bhsd" else (S, B, Hkv, D)
    kc, vc = u(*shape), u(*shape)
    if layout == "bhsd":
        kc[:, :, step - 1:], vc[:, :, step - 1:] = 0, 0
        cs = (Hkv * S * D, S * D, D)
    else:
        kc[step - 1:], vc[step - 1:] = 0, 0
        cs = (Hkv * D, D, B * Hkv * D)
    bq = u(H * D) if bias else None
    bk = u(Hkv * D) if bias else None
    bv = u(Hkv * D) if bias else None
    rope_pos = step if rope_pos is None else rope_pos
    rot_dim = D if rot_dim is None else rot_dim
    q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
    kc_ref, vc_ref = kc.copy(), vc.copy()
    ref = orc.decode_attn(q, k, v, kc_ref, vc_ref, step, rope_pos=rope_pos, rot_dim=rot_dim, bias_q=bq, bias_k=bk,
                          bias_v=bv, cache_layout=layout)

    es = 1
    d_qkv = _dev(torch, qkv, dt)
    d_kc, d_vc = _dev(torch, kc, dt), _dev(torch, vc, dt)
    d_b = [None if b is None else _dev(torch, b, dt) for b in (bq, bk, bv)]
    out = torch.zeros(B, H, D, device="cuda", dtype=_dt(torch, dt))
    wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
    ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
    esz = d_qkv.element_size()
    base = d_qkv.data_ptr()
    host_step = S if use_step_dev else step
    step_dev = torch.tensor([step], device="cuda", dtype=torch.int32) if use_step_dev else None
    ob.decode_attn(ob.F16 if dt == "f16" else ob.F32, base, base + H * D * esz, base + (H + Hkv) * D * esz,
                   (H + 2 * Hkv) * D, (H + 2 * Hkv) * D, (H + 2 * Hkv) * D, d_b[0], d_b[1], d_b[2], d_kc, d_vc,
                   cs[0], cs[1], cs[2], B, H, Hkv, D, host_step, rope_pos + (host_step - step), rot_dim, 10000.0,
                   1.0 / np.sqrt(D), out, H * D, ws, wsb, step_dev=step_dev)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    return got, ref, d_kc.float().cpu().numpy(), d_vc.float().cpu().numpy(), kc_ref, vc_ref


def test_decode_attn_config1_fp32(ob, cuda, orc):
    """B=2, H=32, D=128, step 255 of 256, fp32, U[-1,1] from seed 0, both cache orders."""
    for layout in ("bhsd", "sbhd"):
        got, ref, kc, vc, kc_ref, vc_ref = _run_decode_attn(ob, cuda, orc, "f32", 2, 32, 32, 128, 255, 256, layout, 0)
        assert rel_err(got, ref) < TOL["f32"]
        assert rel_err(kc, kc_ref) < TOL["f32"] and np.array_equal(vc, vc_ref)


def test_decode_attn_reference_known_answer(ob, cuda):
    # tests/unittests/test_decoder_masked_attn.cu:113-176: all ones, bias 2, B=1 H=2 Hkv=1 D=16 step=4 -> 1.0
    torch = cuda
    B, H, Hkv, D, step, S = 1, 2, 1, 16, 4, 32
    qkv = torch.ones(B, H + 2 * Hkv, D, device="cuda")
    bias = torch.full(((H + 2 * Hkv) * D,), 2.0, device="cuda")
    kc = torch.zeros(S, B, Hkv, D, device="cuda")
    vc = torch.zeros(S, B, Hkv, D, device="cuda")
    kc[:step], vc[:step] = 1.0, 1.0
    out = torch.zeros(B, H, D, device="cuda")
    p = qkv.data_ptr()
    ob.decode_attn(ob.F32, p, p + H * D * 4, p + (H + Hkv) * D * 4, 4 * D, 4 * D, 4 * D, bias.data_ptr(),
                   bias.data_ptr() + H * D * 4, None, kc, vc, Hkv * D, D, B * Hkv * D, B, H, Hkv, D, step, step, 0,
                   10000.0, 0.25, out, H * D, None, 0)
    torch.cuda.synchronize()
    assert torch.allclose(out, torch.ones_like(out), atol=1e-6)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("B,H,Hkv,D,step,S", [
    (1, 8, 8, 128, 1, 64), (1, 8, 8, 128, 2, 64), (8, 32, 32, 128, 127, 2048), (8, 32, 32, 128, 128, 2048),
    (8, 32, 32, 128, 129, 2048), (3, 8, 2, 128, 700, 1024), (2, 8, 1, 64, 333, 512), (2, 6, 2, 128, 90, 128),
    (64, 5, 5, 128, 300, 512), (8, 32, 32, 128, 2048, 2048),
])
def test_decode_attn_shapes(ob, cuda, orc, dt, B, H, Hkv, D, step, S):
    got, ref, kc, vc, kc_ref, vc_ref = _run_decode_attn(ob, cuda, orc, dt, B, H, Hkv, D, step, S, "bhsd",
                                                        seed=step + B, bias=(step % 2 == 1), rope_pos=step - 1)
    assert rel_err(got, ref) < TOL[dt]
    assert rel_err(kc, kc_ref) < TOL[dt] and rel_err(vc, vc_ref) < TOL[dt]


def test_decode_attn_step_from_device_and_determinism(ob, cuda, orc):
    a = _run_decode_attn(ob, cuda, orc, "f16", 4, 8, 8, 128, 500, 1024, "bhsd", 11, use_step_dev=True, rope_pos=499)
    assert rel_err(a[0], a[1]) < TOL["f16"]
    b = _run_decode_attn(ob, cuda, orc, "f16", 4, 8, 8, 128, 500, 1024, "bhsd", 11, use_step_dev=True, rope_pos=499)
    assert np.array_equal(a[0], b[0])
    c = _run_decode_attn(ob, cuda, orc, "f16", 4, 8, 8, 128, 500, 1024, "bhsd", 11, rope_pos=499)
    assert rel_err(c[0], a[0]) < TOL["f16"]


@pytest.mark.parametrize("dt,H,Hkv,D,steps,S", [("f16", 8, 8, 128, (333, 100, 17, 1), 512), ("f16", 8, 2, 64, (700, 699, 3), 1024),
                                               ("f32", 4, 4, 128, (60, 255, 2), 256)])
def test_decode_attn_ragged_batch(ob, cuda, orc, dt, H, Hkv, D, steps, S):
    """Every sequence of the batch has its own row count and position (step + step_offset[b]); each must equal the
    oracle run on that sequence alone.  The step itself comes from device memory, as in a captured decode step."""
    torch = cuda
    B = len(steps)
    rng = np.random.default_rng(12)
    u = lambda *s: _round(rng.uniform(-1, 1, s), dt)
    qkv, kc, vc = u(B, H + 2 * Hkv, D), u(B, Hkv, S, D), u(B, Hkv, S, D)
    bq, bk, bv = u(H * D), u(Hkv * D), u(Hkv * D)
    for b, st in enumerate(steps):
        kc[b, :, st - 1:], vc[b, :, st - 1:] = 0, 0
    refs, kc_ref, vc_ref = [], kc.copy(), vc.copy()
    for b, st in enumerate(steps):
        kb, vb = np.ascontiguousarray(kc_ref[b:b + 1]), np.ascontiguousarray(vc_ref[b:b + 1])
        refs.append(orc.decode_attn(qkv[b:b + 1, :H], qkv[b:b + 1, H:H + Hkv], qkv[b:b + 1, H + Hkv:], kb, vb, st, rope_pos=st - 1,
                                    bias_q=bq, bias_k=bk, bias_v=bv))
        kc_ref[b], vc_ref[b] = kb[0], vb[0]
    ref = np.concatenate(refs)
    longest = max(steps)
    d_qkv, d_kc, d_vc = _dev(torch, qkv, dt), _dev(torch, kc, dt), _dev(torch, vc, dt)
    d_b = [_dev(torch, x, dt) for x in (bq, bk, bv)]
    off = torch.tensor([st - longest for st in steps], device="cuda", dtype=torch.int32)
    step_dev = torch.tensor([longest], device="cuda", dtype=torch.int32)
    out = torch.zeros(B, H, D, device="cuda", dtype=_dt(torch, dt))
    wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
    ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
    esz, base, ld = d_qkv.element_size(), d_qkv.data_ptr(), (H + 2 * Hkv) * D
    ob.decode_attn_ragged(ob.F16 if dt == "f16" else ob.F32, base, base + H * D * esz, base + (H + Hkv) * D * esz, ld, ld, ld,
                          d_b[0], d_b[1], d_b[2], d_kc, d_vc, Hkv * S * D, S * D, D, B, H, Hkv, D, S, off, S - 1, D, 10000.0,
                          1.0 / np.sqrt(D), out, H * D, ws, wsb, step_dev=step_dev)
    torch.cuda.synchronize()
    assert rel_err(out.float().cpu().numpy(), ref) < TOL[dt]
    assert rel_err(d_kc.float().cpu().numpy(), kc_ref) < TOL[dt]
    assert rel_err(d_vc.float().cpu().numpy(), vc_ref) < TOL[dt]


@pytest.mark.parametrize("dt,H,Hkv,D,steps,S,splits", [
    ("f16", 8, 8, 128, (700, 300, 65), 1024, 5), ("f16", 8, 2, 64, (900, 899), 1024, 8), ("f16", 4, 4, 128, (2000,), 2048, 16),
    ("f16", 32, 32, 128, (520, 520, 519, 2), 1024, 0), ("f32", 4, 4, 128, (500, 130, 1), 512, 0)])
def test_decode_attn_merged_in_the_kernel_equals_the_two_launch_form(ob, cuda, orc, dt, H, Hkv, D, steps, S, splits):
    """Split launches merged by the last block of each (sequence, head group) give the bits the separate merge kernel
    gives for the same plan, leave the ticket array zero (a second call on it gives the same bits), and match the oracle."""
    torch = cuda
    B = len(steps)
    rng = np.random.default_rng(S + B)
    u = lambda *s: _round(rng.uniform(-1, 1, s), dt)
    qkv, kc, vc = u(B, H + 2 * Hkv, D), u(B, Hkv, S, D), u(B, Hkv, S, D)
    for b, st in enumerate(steps):
        kc[b, :, st - 1:], vc[b, :, st - 1:] = 0, 0
    refs = []
    for b, st in enumerate(steps):
        kb, vb = np.ascontiguousarray(kc[b:b + 1]).copy(), np.ascontiguousarray(vc[b:b + 1]).copy()
        refs.append(orc.decode_attn(qkv[b:b + 1, :H], qkv[b:b + 1, H:H + Hkv], qkv[b:b + 1, H + Hkv:], kb, vb, st, rope_pos=st - 1))
    ref = np.concatenate(refs)
    longest = max(steps)
    d_qkv = _dev(torch, qkv, dt)
    off = torch.tensor([st - longest for st in steps], device="cuda", dtype=torch.int32)
    step_dev = torch.tensor([longest], device="cuda", dtype=torch.int32)
    wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
    esz, base, ld = d_qkv.element_size(), d_qkv.data_ptr(), (H + 2 * Hkv) * D
    code = ob.F16 if dt == "f16" else ob.F32
    tickets = torch.zeros(B * H, device="cuda", dtype=torch.int32)
    outs = []
    try:
        ob.decode_attn_plan_override(0, splits)
        for form in ("two launches", "merged", "merged again"):
            d_kc, d_vc = _dev(torch, kc, dt), _dev(torch, vc, dt)
            ws = torch.full((wsb,), 0x7f, device="cuda", dtype=torch.uint8)  # stale partials must not matter
            out = torch.zeros(B, H, D, device="cuda", dtype=_dt(torch, dt))
            args = (code, base, base + H * D * esz, base + (H + Hkv) * D * esz, ld, ld, ld, None, None, None, d_kc, d_vc,
                    Hkv * S * D, S * D, D, B, H, Hkv, D, S, off, S - 1, D, 10000.0, 1.0 / np.sqrt(D), out, H * D, ws, wsb)
            if form == "two launches":
                ob.decode_attn_ragged(*args, step_dev=step_dev)
            else:
                ob.decode_attn_merged(*args, tickets, step_dev=step_dev)
            torch.cuda.synchronize()
            outs.append(out.float().cpu().numpy())
            assert int(tickets.abs().sum().item()) == 0
    finally:
        ob.decode_attn_plan_override(0, 0)
    assert rel_err(outs[0], ref) < TOL[dt]
    assert np.array_equal(outs[0], outs[1])  # the same plan in both forms
    assert np.array_equal(outs[1], outs[2])


def test_decode_attn_partial_rotary(ob, cuda, orc):
    got, ref, *_ = _run_decode_attn(ob, cuda, orc, "f32", 2, 4, 4, 128, 40, 64, "bhsd", 5, rot_dim=64)
    assert rel_err(got, ref) < TOL["f32"]


def test_decode_attn_rejects_bad_arguments(ob, cuda):
    torch = cuda
    t = torch.zeros(4096, device="cuda")
    with pytest.raises(ob.OnellmError):  # D*4 = 48 bytes is not a supported row
        ob.decode_attn(ob.F32, t, t, t, 12, 12, 12, None, None, None, t, t, 12, 12, 12, 1, 1, 1, 12, 1, 1, 12, 1e4,
                       1.0, t, 12, None, 0)
    with pytest.raises(ob.OnellmError):  # H not a multiple of Hkv
        ob.decode_attn(ob.F32, t, t, t, 64, 64, 64, None, None, None, t, t, 64, 64, 16, 1, 3, 2, 16, 1, 1, 16, 1e4,
                       1.0, t, 48, None, 0)
    with pytest.raises(ob.OnellmError):  # split needed but no workspace
        big = torch.zeros(2 * 4096 * 128, device="cuda")
        ob.decode_attn(ob.F32, t, t, t, 128, 128, 128, None, None, None, big, big, 4096 * 128, 4096 * 128, 128, 1, 1, 1,
                       128, 4000, 4000, 128, 1e4, 1.0, t, 128, None, 0)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("T,h", [(1, 32), (8, 4096), (4096, 4096), (8, 5120), (3, 11008), (2, 16384)])
def test_rmsnorm_and_fused(ob, cuda, orc, dt, T, h):
    torch = cuda
    rng = np.random.default_rng(1)
    x, r = _round(rng.standard_normal((T, h)), dt), _round(rng.standard_normal((T, h)), dt)
    g, b = _round(1 + 0.1 * rng.standard_normal(h), dt), _round(0.1 * rng.standard_normal(h), dt)
    code = ob.F16 if dt == "f16" else ob.F32
    dx = _dev(torch, x, dt)
    ob.rmsnorm(code, dx, _dev(torch, g, dt), 1e-5, T, h)
    assert rel_err(dx.float().cpu().numpy(), orc.rmsnorm(x, g, 1e-5)) < TOL[dt]
    for bias in (None, b):
        dy, dr = _dev(torch, x, dt), _dev(torch, r, dt)
        ob.add_residual_rmsnorm(code, dr, dy, None if bias is None else _dev(torch, bias, dt), _dev(torch, g, dt),
                                1e-5, T, h)
        y_ref, r_ref = orc.add_residual_rmsnorm(r, x, bias, g, 1e-5)
        assert rel_err(dy.float().cpu().numpy(), y_ref) < TOL[dt]
        assert rel_err(dr.float().cpu().numpy(), r_ref) < TOL[dt]


def test_norm_reference_known_answers(ob, cuda):
    # tests/unittests/test_rmsnorm.cu:64-98 and test_fused_addres_rms.cu:64-98 -> 1/sqrt(1.5)
    torch = cuda
    x = torch.ones(2, 32, device="cuda")
    ob.rmsnorm(ob.F32, x, torch.ones(32, device="cuda"), 0.5, 2, 32)
    assert torch.allclose(x, torch.full_like(x, 1 / np.sqrt(1.5)), atol=1e-6)
    y, r = torch.ones(2, 32, device="cuda"), torch.zeros(2, 32, device="cuda")
    ob.add_residual_rmsnorm(ob.F32, r, y, torch.zeros(32, device="cuda"), torch.ones(32, device="cuda"), 0.5, 2, 32)
    assert torch.allclose(y, torch.full_like(y, 1 / np.sqrt(1.5)), atol=1e-6)
    assert torch.equal(r, torch.ones_like(r))


GEMM_SHAPES = [  # (N, K): 7B and 13B projections, full and 8-way sliced
    (12288, 4096), (4096, 4096), (11008, 4096), (4096, 11008), (1376, 4096), (4096, 1376), (1536, 4096),
    (15360, 5120), (1728, 5120), (5120, 1728), (5120, 640),
]


@pytest.mark.parametrize("M", [1, 8, 13, 64])
@pytest.mark.parametrize("N,K", GEMM_SHAPES)
def test_gemm_f16_decode_shapes(ob, cuda, orc, M, N, K):
    torch = cuda
    rng = np.random.default_rng(N + K + M)
    x = _round(rng.standard_normal((M, K)), "f16")
    W = _round(0.02 * rng.standard_normal((K, N)), "f16")
    y = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    ob.gemm(ob.F16, _dev(torch, x, "f16"), _dev(torch, W, "f16"), y, M, N, K, ob.W_KN)
    assert rel_err(y.float().cpu().numpy(), orc.gemm(x, W)) < TOL["f16"]


@pytest.mark.parametrize("M", [1, 8, 64])
def test_gemm_f16_lm_head(ob, cuda, orc, M):
    torch = cuda
    N, K = 32000, 4096
    rng = np.random.default_rng(M)
    x = _round(rng.standard_normal((M, K)), "f16")
    W = _round(0.02 * rng.standard_normal((N, K)), "f16")
    y = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    ob.gemm(ob.F16, _dev(torch, x, "f16"), _dev(torch, W, "f16"), y, M, N, K, ob.W_NK)
    assert rel_err(y.float().cpu().numpy(), orc.gemm(x, W, w_is_nk=True)) < TOL["f16"]


def test_gemm_is_deterministic(ob, cuda):
    torch = cuda
    torch.manual_seed(0)
    x = torch.randn(8, 4096, device="cuda", dtype=torch.float16)
    W = (0.02 * torch.randn(4096, 4096, device="cuda")).half()
    y1, y2 = torch.zeros(8, 4096, device="cuda", dtype=torch.float16), torch.zeros(8, 4096, device="cuda", dtype=torch.float16)
    ob.gemm(ob.F16, x, W, y1, 8, 4096, 4096)
    ob.gemm(ob.F16, x, W, y2, 8, 4096, 4096)
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("M,N,K,nk", [(16, 16, 16, False), (5, 70, 33, False), (130, 65, 100, True), (8, 4096, 512, False)])
def test_gemm_f32(ob, cuda, orc, M, N, K, nk):
    torch = cuda
    rng = np.random.default_rng(K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = rng.standard_normal((N, K) if nk else (K, N)).astype(np.float32)
    if (M, N, K) == (16, 16, 16):  # tests/unittests/test_linear.cu:52-71: ones -> 16
        x[:], W[:] = 1, 1
    y = torch.zeros(M, N, device="cuda")
    ob.gemm(ob.F32, _dev(torch, x, "f32"), _dev(torch, W, "f32"), y, M, N, K, ob.W_NK if nk else ob.W_KN)
    assert rel_err(y.cpu().numpy(), orc.gemm(x, W, w_is_nk=nk)) < TOL["f32"]


@pytest.mark.parametrize("M", [1, 8, 16, 32])
@pytest.mark.parametrize("I,K", [(11008, 4096), (1376, 4096), (1728, 5120)])
def test_gemm_swiglu_fused(ob, cuda, orc, M, I, K):
    torch = cuda
    rng = np.random.default_rng(I + M)
    x = _round(rng.standard_normal((M, K)), "f16")
    Wg, Wu = _round(0.02 * rng.standard_normal((K, I)), "f16"), _round(0.02 * rng.standard_normal((K, I)), "f16")
    out = torch.zeros(M, I, device="cuda", dtype=torch.float16)
    ob.gemm_swiglu(ob.F16, _dev(torch, x, "f16"), _dev(torch, Wg, "f16"), _dev(torch, Wu, "f16"), out, M, I, K)
    ref = orc.swiglu2(orc.gemm(x, Wg), orc.gemm(x, Wu))
    assert rel_err(out.float().cpu().numpy(), ref) < TOL["f16"]


@pytest.mark.parametrize("M,I,K", [(128, 256, 64), (65, 1376, 4096), (300, 11008, 4096), (1024, 11008, 4096), (200, 1000, 528)])
def test_gemm_swiglu_tensor_core_tiles(ob, cuda, orc, M, I, K):
    """M > 64: gate and up share one tcgen05 tile (128 + 128 accumulator columns), SwiGLU in the epilogue; ragged M, I, K."""
    torch = cuda
    rng = np.random.default_rng(I + M)
    x = _round(rng.standard_normal((M, K)), "f16")
    Wg, Wu = _round(0.02 * rng.standard_normal((K, I)), "f16"), _round(0.02 * rng.standard_normal((K, I)), "f16")
    out = torch.full((M + 1, I), 7.0, device="cuda", dtype=torch.float16)   # one guard row behind the output
    ob.gemm_swiglu(ob.F16, _dev(torch, x, "f16"), _dev(torch, Wg, "f16"), _dev(torch, Wu, "f16"), out, M, I, K)
    ref = orc.swiglu2(orc.gemm(x, Wg), orc.gemm(x, Wu))
    assert rel_err(out[:M].float().cpu().numpy(), ref) < TOL["f16"]
    assert float(out[M].float().min()) == 7.0 and float(out[M].float().max()) == 7.0
    assert ob.lib().onellm_gemm_timeout_flag() == 0


@pytest.mark.parametrize("dt", ["f16", "f32"])
def test_swiglu_standalone(ob, cuda, orc, dt):
    torch = cuda
    # tests/unittests/test_activation.cu:35-49 uses input[i] = i, B=16, I=11008 (fp32); fp16 gets N(0,1)
    B, I = 16, 11008
    if dt == "f32":
        inp = np.arange(B * 2 * I, dtype=np.float32).reshape(B, 2, I)
    else:
        inp = _round(np.random.default_rng(0).standard_normal((B, 2, I)), dt)
    out = torch.zeros(B, I, device="cuda", dtype=_dt(torch, dt))
    ob.swiglu(ob.F16 if dt == "f16" else ob.F32, _dev(torch, inp, dt), out, B, I)
    assert rel_err(out.float().cpu().numpy(), orc.swiglu(inp)) < TOL[dt]


@pytest.mark.parametrize("dt", ["f16", "f32"])
def test_embedding(ob, cuda, orc, dt):
    torch = cuda
    rng = np.random.default_rng(0)
    V, h = 32000, 4096
    table = _round(rng.standard_normal((V, h)), dt)
    ids = rng.integers(0, V, size=(8, 16)).astype(np.int32)
    out = torch.zeros(8 * 16, h, device="cuda", dtype=_dt(torch, dt))
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    ob.embedding(ob.F16 if dt == "f16" else ob.F32, torch.from_numpy(ids).cuda(), out, _dev(torch, table, dt), ids.size,
                 h, V, flag)
    assert np.array_equal(out.float().cpu().numpy().reshape(8, 16, h), orc.embedding(ids, table))
    assert int(flag.item()) == 0
    bad = torch.tensor([5, V, -1], device="cuda", dtype=torch.int32)
    ob.embedding(ob.F16 if dt == "f16" else ob.F32, bad, out, _dev(torch, table, dt), 3, h, V, flag)
    assert int(flag.item()) == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("rows,V,K", [(8, 32000, 50), (64, 32000, 1), (3, 1000, 64), (2, 100, 7), (2, 40000, 50), (3, 1003, 64),
                                       (2, 32768, 64), (1, 32769, 5)])
def test_topk_bit_exact(ob, cuda, orc, dt, rows, V, K):
    torch = cuda
    rng = np.random.default_rng(V + K)
    x = _round(rng.standard_normal((rows, V)), dt)  # fp16 rounding makes ties common
    x[0, :5] = x[0].max()  # forced ties at the top
    val = torch.zeros(rows, K, device="cuda")
    idx = torch.zeros(rows, K, device="cuda", dtype=torch.int32)
    ob.topk(ob.F16 if dt == "f16" else ob.F32, _dev(torch, x, dt), rows, V, K, val, idx)
    rv, ri = orc.topk(x, K)
    assert np.array_equal(idx.cpu().numpy(), ri)
    assert np.array_equal(val.cpu().numpy(), rv)


@pytest.mark.parametrize("dt", ["f16", "f32"])
def test_topk_special_values(ob, cuda, orc, dt):
    """All-equal rows (pure ties), NaN and infinities, negative-only rows."""
    torch = cuda
    V, K = 5000, 16
    x = np.zeros((4, V), np.float32)
    x[0, :] = 1.5                                   # every column ties: the K lowest columns win
    x[1, :] = -np.arange(V, dtype=np.float32) - 1   # all negative
    x[2, :] = 0.25
    x[2, [7, 100, 4999]] = [np.inf, np.nan, -np.inf]
    x[3, :] = _round(np.random.default_rng(3).standard_normal(V), dt)
    x[3, ::2] = np.nan                               # half the row is NaN and must sort below everything
    val = torch.zeros(4, K, device="cuda")
    idx = torch.zeros(4, K, device="cuda", dtype=torch.int32)
    ob.topk(ob.F16 if dt == "f16" else ob.F32, _dev(torch, _round(x, dt), dt), 4, V, K, val, idx)
    rv, ri = orc.topk(_round(x, dt), K)
    assert np.array_equal(idx.cpu().numpy(), ri)
    assert np.array_equal(val.cpu().numpy(), rv)
    assert ri[0].tolist() == list(range(K)) and ri[2, 0] == 7


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("copies", [40, 300, 513, 3000])
def test_topk_runs_of_equal_keys_on_both_ways_through_the_kernel(ob, cuda, orc, dt, copies):
    """`copies` columns share the row's K-th largest value: up to 512 gathered keys the kernel ranks them directly, beyond
    that it bisects over all keys; both must give the lowest columns among the equals."""
    torch = cuda
    V, K = 32000, 50
    rng = np.random.default_rng(copies)
    x = _round(rng.standard_normal((3, V)), dt)
    for r in range(3):
        cols = rng.choice(V, copies, replace=False)
        x[r, cols] = 3.0 + r                       # above nearly everything else
        x[r, rng.choice(V, 10, replace=False)] = 9.0  # ten columns above the run
    val = torch.zeros(3, K, device="cuda")
    idx = torch.zeros(3, K, device="cuda", dtype=torch.int32)
    ob.topk(ob.F16 if dt == "f16" else ob.F32, _dev(torch, x, dt), 3, V, K, val, idx)
    rv, ri = orc.topk(x, K)
    assert np.array_equal(idx.cpu().numpy(), ri)
    assert np.array_equal(val.cpu().numpy(), rv)


def test_topk_reference_case(ob, cuda):
    # tests/unittests/test_beamsearch_topK.cu:12-25: probs[i] = i, V = 30000, K = 2, ids are row*V + column
    torch = cuda
    rows, V = 4, 30000
    probs = torch.arange(rows * V, device="cuda", dtype=torch.float32).reshape(rows, V)
    val = torch.zeros(rows, 2, device="cuda")
    idx = torch.zeros(rows, 2, device="cuda", dtype=torch.int32)
    ob.topk(ob.F32, probs, rows, V, 2, val, idx, global_ids=True)
    assert idx.cpu().tolist() == [[r * V + V - 1, r * V + V - 2] for r in range(rows)]


@pytest.mark.parametrize("K,temp,literal", [(3, 1.0, False), (50, 1.0, False), (50, 0.8, False), (50, 1.0, True)])
def test_sampling_matches_oracle_given_same_uniform(ob, cuda, orc, K, temp, literal):
    torch = cuda
    B, V = 16, 32000
    rng = np.random.default_rng(K)
    logits = rng.standard_normal((B, V)).astype(np.float32)
    rv, ri = orc.topk(logits, K)
    if K == 3:  # tests/unittests/test_topK_sampling.cu:6-43: values 2,1,0, step 5, end_id 10
        rv[:] = np.array([2, 1, 0], np.float32)
    for step in (5, 6, 1000):
        out = torch.zeros(B, device="cuda", dtype=torch.int32)
        sl = torch.zeros(B, device="cuda", dtype=torch.int32)
        fin = torch.zeros(B, device="cuda", dtype=torch.uint8)
        u = torch.zeros(B, device="cuda")
        ob.topk_sample(torch.from_numpy(ri).cuda(), torch.from_numpy(rv).cuda(), B, K, temp, step, V, 10, out, sl, fin, u,
                       literal_walk=literal)
        un = u.cpu().numpy()
        assert np.all((un > 0) & (un <= 1))
        want, wsl, wfin = orc.topk_sample(ri, rv, un, temperature=temp, vocab_size=V, end_id=10, literal=literal)
        assert np.array_equal(out.cpu().numpy(), want)
        assert np.array_equal(sl.cpu().numpy(), wsl) and np.array_equal(fin.cpu().numpy(), wfin)
        # same (seed, subsequence) -> same draw; a different step -> a different draw
        u2 = torch.zeros(B, device="cuda")
        ob.topk_sample(torch.from_numpy(ri).cuda(), torch.from_numpy(rv).cuda(), B, K, temp, step, V, 10, out, None, None, u2)
        assert torch.equal(u, u2)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("N,K,dual,with_x,with_bias", [
    (12288, 4096, False, True, False), (12288, 4096, False, False, False), (11008, 4096, True, True, True),
    (1376, 4096, True, True, False), (15360, 5120, False, True, True), (1728, 5120, True, True, False),
])
def test_add_residual_rmsnorm_gemm_fused(ob, cuda, orc, M, N, K, dual, with_x, with_bias):
    """One launch = fused add-bias-residual RMSNorm, then the projection (and SwiGLU)."""
    torch = cuda
    rng = np.random.default_rng(M + N)
    x = _round(rng.standard_normal((M, K)), "f16") if with_x else None
    r = _round(rng.standard_normal((M, K)), "f16")
    b = _round(0.1 * rng.standard_normal(K), "f16") if with_bias else None
    g = _round(1 + 0.1 * rng.standard_normal(K), "f16")
    W = _round(0.02 * rng.standard_normal((K, N)), "f16")
    Wu = _round(0.02 * rng.standard_normal((K, N)), "f16") if dual else None
    if with_x:
        xn, r_new = orc.add_residual_rmsnorm(r, x, b, g, 1e-5)
    else:
        xn, r_new = orc.rmsnorm(r, g, 1e-5), r
    xn = _round(xn, "f16")
    ref = orc.swiglu2(orc.gemm(xn, W), orc.gemm(xn, Wu)) if dual else orc.gemm(xn, W)
    y = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    r_out = torch.zeros(M, K, device="cuda", dtype=torch.float16)
    d_r = _dev(torch, r, "f16")
    ob.add_residual_rmsnorm_gemm(ob.F16, None if x is None else _dev(torch, x, "f16"), d_r,
                                 None if b is None else _dev(torch, b, "f16"), _dev(torch, g, "f16"), 1e-5, r_out,
                                 _dev(torch, W, "f16"), None if Wu is None else _dev(torch, Wu, "f16"), y, M, N, K)
    assert rel_err(y.float().cpu().numpy(), ref) < 2e-3  # normalised activations are rounded to fp16 in both arms
    assert np.array_equal(d_r.float().cpu().numpy(), r)  # the input residual is not touched
    if with_x:
        assert rel_err(r_out.float().cpu().numpy(), r_new) < TOL["f16"]
    with pytest.raises(ob.OnellmError):
        ob.add_residual_rmsnorm_gemm(ob.F16, d_r, d_r, None, _dev(torch, g, "f16"), 1e-5, d_r, _dev(torch, W, "f16"), None,
                                     y, M, N, K)


@pytest.mark.parametrize("M", [1, 8, 13, 40])
@pytest.mark.parametrize("N,K,dual,rms,resid,with_bias", [
    (12288, 4096, False, True, False, False),    # QKV behind the attention norm
    (4096, 4096, False, False, True, True),      # o_proj adding into the residual stream
    (11008, 4096, True, True, False, False),     # gate/up + SwiGLU behind the FFN norm
    (4096, 11008, False, False, True, False),    # down_proj adding into the residual stream
    (1376, 5120, True, True, True, True), (1000, 528, False, True, True, False),
])
def test_gemm_fused_norm_free_layer_ops(ob, cuda, orc, M, N, K, dual, rms, resid, with_bias):
    """y = [resid + bias +] f(rsqrt(mean(x^2)+eps) * x . W): RMSNorm with gamma folded into W, and the residual add."""
    torch = cuda
    rng = np.random.default_rng(7 * M + N)
    x = _round(3.0 * rng.standard_normal((M, K)), "f16")          # un-normalised residual-stream magnitudes
    g = _round(1 + 0.1 * rng.standard_normal(K), "f16")
    W = _round(0.02 * rng.standard_normal((K, N)), "f16")
    Wu = _round(0.02 * rng.standard_normal((K, N)), "f16") if dual else None
    r = _round(rng.standard_normal((M, N)), "f16") if resid else None
    b = _round(0.1 * rng.standard_normal(N), "f16") if (resid and with_bias) else None
    # the two sides of the identity the model relies on: norm kernel + projection == folded projection
    Wf = _round(W * g[:, None], "f16") if rms else W
    Wuf = (_round(Wu * g[:, None], "f16") if rms else Wu) if dual else None
    if rms:
        inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
        t0, t1 = orc.gemm(x, Wf) * inv, (orc.gemm(x, Wuf) * inv if dual else None)
    else:
        t0, t1 = orc.gemm(x, Wf), (orc.gemm(x, Wuf) if dual else None)
    ref = orc.swiglu2(t0.astype(np.float32), t1.astype(np.float32)) if dual else t0
    if resid:
        ref = ref + r + (b if b is not None else 0.0)
    y = _dev(torch, r, "f16") if resid else torch.zeros(M, N, device="cuda", dtype=torch.float16)
    ob.gemm_fused(ob.F16, _dev(torch, x, "f16"), _dev(torch, Wf, "f16"), None if Wuf is None else _dev(torch, Wuf, "f16"), y, M, N, K,
                  rms_eps=1e-5 if rms else -1.0, resid=y if resid else None, bias=None if b is None else _dev(torch, b, "f16"))
    assert rel_err(y.float().cpu().numpy(), ref) < TOL["f16"]
    if rms and not dual and not resid:
        # and against the unfused reference order: RMSNorm (gamma applied, rounded to fp16), then x . W
        xn = _round(orc.rmsnorm(x, g, 1e-5), "f16")
        assert rel_err(y.float().cpu().numpy(), orc.gemm(xn, W)) < 2e-3


@pytest.mark.parametrize("M,N,K,nk", [
    (128, 128, 64, False), (128, 128, 64, True), (256, 256, 256, False), (1024, 4096, 4096, False),
    (1000, 12288, 4096, False), (65, 1376, 4096, False), (512, 4096, 11008, False), (300, 4096, 1376, False),
    (192, 32000, 4096, True), (130, 1000, 512, True),
])
def test_gemm_f16_tensor_core_tiles(ob, cuda, orc, M, N, K, nk):
    """M > 64: the tcgen05 / TMEM / TMA kernel, both weight layouts, ragged M, N and K tails."""
    torch = cuda
    rng = np.random.default_rng(M + N + K)
    x = _round(rng.standard_normal((M, K)), "f16")
    W = _round(0.02 * rng.standard_normal((N, K) if nk else (K, N)), "f16")
    y = torch.full((M, N), 7.0, device="cuda", dtype=torch.float16)
    ob.gemm(ob.F16, _dev(torch, x, "f16"), _dev(torch, W, "f16"), y, M, N, K, ob.W_NK if nk else ob.W_KN)
    torch.cuda.synchronize()
    assert ob.lib().onellm_gemm_timeout_flag() == 0
    assert rel_err(y.float().cpu().numpy(), orc.gemm(x, W, w_is_nk=nk)) < TOL["f16"]



@pytest.mark.parametrize("M", [17, 25, 64])
@pytest.mark.parametrize("N,K,dual,rms,resid", [
    (1920, 5120, False, True, False),     # 13B QKV, one of eight ranks: 15 column tiles, the K range split eight ways
    (5120, 640, False, False, True),      # 13B o_proj slice: ten 64-row stages in all
    (1728, 5120, True, True, False),      # gate/up slice: the last column tile is half empty
    (32000, 4096, False, False, False),   # LM head: more column tiles than SMs (two blocks per SM, one wave)
    (1000, 528, True, False, True),       # ragged in N and K
    (5120, 1728, False, False, True),     # 13B down_proj slices: tuned plans with two blocks per SM
    (5120, 3456, False, False, True),
    (12288, 4096, False, True, False),    # 256-column blocks: 7B QKV behind the norm
    (4096, 11008, False, False, True),    # 7B down_proj adding into the residual stream
    (1160, 528, False, True, True),       # the last 256-column block has 128 + 8 columns, K is ragged
])
def test_gemm_tensor_core_weight_streaming_kernel(ob, cuda, orc, M, N, K, dual, rms, resid):
    """The tcgen05 kernel for 17..64 tokens (forced from 17 tokens up here) against the oracle, and bit-identical to itself."""
    torch = cuda
    before = ob.gemm_tc_min_tokens(17)
    try:
        rng = np.random.default_rng(M + N + K)
        x = _round(2.0 * rng.standard_normal((M, K)), "f16")
        W = _round(0.02 * rng.standard_normal((K, N)), "f16")
        Wu = _round(0.02 * rng.standard_normal((K, N)), "f16") if dual else None
        r = _round(rng.standard_normal((M, N)), "f16") if resid else None
        inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5) if rms else 1.0
        t0 = orc.gemm(x, W) * inv
        ref = orc.swiglu2(t0.astype(np.float32), (orc.gemm(x, Wu) * inv).astype(np.float32)) if dual else t0
        if resid:
            ref = ref + r
        outs = []
        for _ in range(2):
            y = _dev(torch, r, "f16") if resid else torch.zeros(M, N, device="cuda", dtype=torch.float16)
            ob.gemm_fused(ob.F16, _dev(torch, x, "f16"), _dev(torch, W, "f16"), None if Wu is None else _dev(torch, Wu, "f16"), y, M, N, K,
                          rms_eps=1e-5 if rms else -1.0, resid=y if resid else None, bias=None)
            outs.append(y)
        torch.cuda.synchronize()
        assert ob.lib().onellm_gemm_timeout_flag() == 0
        assert rel_err(outs[0].float().cpu().numpy(), ref) < TOL["f16"]
        assert torch.equal(outs[0], outs[1])
    finally:
        ob.gemm_tc_min_tokens(before)


@pytest.mark.parametrize("ks,nst", [(1, 3), (5, 3), (7, 4), (3, 9), (2, 6)])
def test_gemm_tensor_core_kernel_under_a_forced_plan(ob, cuda, orc, ks, nst):
    """onellm_gemm_plan_override reaches the tcgen05 kernel too: every (K split, ring depth) gives the oracle's result."""
    torch = cuda
    M, N, K = 64, 5120, 1280
    rng = np.random.default_rng(ks * 16 + nst)
    x = _round(2.0 * rng.standard_normal((M, K)), "f16")
    W = _round(0.02 * rng.standard_normal((K, N)), "f16")
    r = _round(rng.standard_normal((M, N)), "f16")
    try:
        ob.gemm_plan_override(N, K, False, ks, nst)
        assert ob.gemm_plan_query(M, N, K, False)[:2] == (ks, nst)
        y = _dev(torch, r, "f16")
        ob.gemm_fused(ob.F16, _dev(torch, x, "f16"), _dev(torch, W, "f16"), None, y, M, N, K, rms_eps=-1.0, resid=y, bias=None)
        torch.cuda.synchronize()
        assert ob.lib().onellm_gemm_timeout_flag() == 0
        assert rel_err(y.float().cpu().numpy(), orc.gemm(x, W) + r) < TOL["f16"]
    finally:
        ob.gemm_plan_override(N, K, False, 0, 3)
    assert ob.gemm_plan_query(M, N, K, False)[:2] == (5, 3)  # the tuned plan of this shape is back


def test_gemm_tensor_core_kernel_refuses_a_plan_that_leaves_a_block_without_rows(ob, cuda):
    torch = cuda
    M, N, K = 64, 5120, 1280  # twenty 64-row stages: split eight ways, three per block, the eighth block would get none
    x = torch.zeros(M, K, device="cuda", dtype=torch.float16)
    W = torch.zeros(K, N, device="cuda", dtype=torch.float16)
    y = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    try:
        ob.gemm_plan_override(N, K, False, 8, 4)
        with pytest.raises(ob.OnellmError):
            ob.gemm_fused(ob.F16, x, W, None, y, M, N, K, rms_eps=-1.0, resid=None, bias=None)
    finally:
        ob.gemm_plan_override(N, K, False, 0, 3)
    ob.gemm_fused(ob.F16, x, W, None, y, M, N, K, rms_eps=-1.0, resid=None, bias=None)
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,N,K", [(300, 512, 256), (1024, 4096, 4096), (130, 1000, 528)])
def test_gemm_rows_norm_free_context_projections(ob, cuda, orc, M, N, K):
    """onellm_gemm_rows: row scale from partial sums of squares, residual + bias in the epilogue, and the partial sums of
    squares of what was stored (the next projection's input statistics); onellm_row_sumsq."""
    torch = cuda
    rng = np.random.default_rng(M + N)
    x = _round(3.0 * rng.standard_normal((M, K)), "f16")
    W = _round(0.02 * rng.standard_normal((K, N)), "f16")
    Wu = _round(0.02 * rng.standard_normal((K, N)), "f16")
    r = _round(rng.standard_normal((M, N)), "f16")
    b = _round(0.1 * rng.standard_normal(N), "f16")
    d_x, d_W, d_Wu = _dev(torch, x, "f16"), _dev(torch, W, "f16"), _dev(torch, Wu, "f16")
    ss = torch.zeros(M, device="cuda", dtype=torch.float32)
    ob.row_sumsq(ob.F16, d_x, M, K, ss)
    want_ss = (x.astype(np.float64) ** 2).sum(axis=1)
    assert rel_err(ss.cpu().numpy(), want_ss) < 1e-5
    inv = 1.0 / np.sqrt(want_ss[:, None] / K + 1e-5)
    # (1) RMS scale; the row sums handed over as three partial sums per row
    parts = torch.stack([0.5 * ss, 0.25 * ss, 0.25 * ss], dim=1).contiguous()
    y = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    ob.gemm_rows(ob.F16, d_x, d_W, None, y, M, N, K, row_ss=parts, ss_parts=3, rms_eps=1e-5)
    assert rel_err(y.float().cpu().numpy(), orc.gemm(x, W) * inv) < TOL["f16"]
    # (2) gate/up + SwiGLU behind the same scale
    ob.gemm_rows(ob.F16, d_x, d_W, d_Wu, y, M, N, K, row_ss=ss, ss_parts=1, rms_eps=1e-5)
    ref = orc.swiglu2((orc.gemm(x, W) * inv).astype(np.float32), (orc.gemm(x, Wu) * inv).astype(np.float32))
    assert rel_err(y.float().cpu().numpy(), ref) < TOL["f16"]
    # (3) residual + bias added in place, and the statistics of the stored rows
    n_parts = ob.gemm_rows_parts(N)
    y = _dev(torch, r, "f16")
    ss_out = torch.full((M, n_parts), -1.0, device="cuda", dtype=torch.float32)
    ob.gemm_rows(ob.F16, d_x, d_W, None, y, M, N, K, resid=y, bias=_dev(torch, b, "f16"), row_ss_out=ss_out)
    got = y.float().cpu().numpy()
    assert rel_err(got, orc.gemm(x, W) + r + b) < TOL["f16"]
    assert rel_err(ss_out.sum(dim=1).cpu().numpy(), (got.astype(np.float64) ** 2).sum(axis=1)) < 1e-5   # of the ROUNDED values
    assert ob.lib().onellm_gemm_timeout_flag() == 0
