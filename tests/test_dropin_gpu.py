"""The reference's own code on this library's kernels: (1) its layer classes, compiled unchanged against
the drop-in headers and driven by tests/cpp/dropin_*.cpp, against the CPU oracle; (2) its unit-test
programs, unchanged, whose own CPU checks must agree.  The programs are prebuilt by
oracle/build_dropin.py where a oneLLM tree is present."""
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "dropin")

needs_programs = pytest.mark.skipif(not os.path.exists(os.path.join(BIN, "dropin_layers")),
                                    reason="oracle/_ref/dropin not built (needs a oneLLM source tree at build time)")


class Lcg:
    """The generator of tests/cpp/dropin_layers.cpp."""

    def __init__(self):
        self.state = 12345

    def randv(self, n, scale):
        out = np.empty(n, np.float32)
        s = self.state
        for i in range(n):
            s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
            out[i] = (s >> 8) / 16777216.0 - 0.5
        self.state = s
        return out * np.float32(scale)


def _load(d, name, shape, dtype=np.float32):
    return np.fromfile(os.path.join(d, name + ".f32"), dtype=dtype).reshape(shape)


@needs_programs
def test_reference_layer_classes_on_these_kernels(ob, cuda, orc, tmp_path):
    torch = cuda
    p = subprocess.run([os.path.join(BIN, "dropin_layers"), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "dropin_layers ok" in p.stdout
    B, H, Hkv, D, S, L, inter = 2, 4, 2, 32, 24, 2, 192
    hidden, QH = H * D, H + 2 * Hkv
    g = Lcg()
    Wqkv = g.randv(hidden * QH * D, 0.2).reshape(hidden, QH * D)
    bqkv = g.randv(QH * D, 0.2)
    Wo = g.randv(hidden * hidden, 0.2).reshape(hidden, hidden)

    # ---- context phase, layer 1; the layer uses the shipped mask (history columns off)
    lens, hist, ctx, T, max_q, max_k = [5, 3], [2, 0], [7, 3], 8, 5, 7
    X = g.randv(T * hidden, 2.0).reshape(T, hidden)
    kc = g.randv(L * B * Hkv * S * D, 2.0).reshape(L, B, Hkv, S, D)
    vc = g.randv(L * B * Hkv * S * D, 2.0).reshape(L, B, Hkv, S, D)
    po, cum, n = orc.cal_padding_offset(lens, max_q)
    mask = orc.build_causal_mask(lens, ctx, max_q, max_k, attend_history=False)
    assert np.array_equal(_load(tmp_path, "ctx_mask", (B, max_q, max_k)), mask)
    qkv = orc.gemm(X, Wqkv).reshape(T, QH, D)
    q_r, k_r, v_r = orc.qkv_bias_rope_transpose(qkv, bqkv, po, hist, B, max_q, H, Hkv, D, 10000.0)
    kc1, vc1 = np.ascontiguousarray(kc[1]), np.ascontiguousarray(vc[1])
    orc.append_kv_cache(kc1, k_r, lens, hist)
    orc.append_kv_cache(vc1, v_r, lens, hist)
    k_rep, v_rep = orc.repeat_kv(kc1, ctx, H, max_k), orc.repeat_kv(vc1, ctx, H, max_k)
    qk = np.einsum("bhqd,bhkd->bhqk", q_r.astype(np.float64), k_rep.astype(np.float64)).astype(np.float32)
    prob = orc.scale_mask_softmax(qk, mask, D ** -0.5)
    pv = np.einsum("bhqk,bhkd->bhqd", prob.astype(np.float64), v_rep.astype(np.float64)).astype(np.float32)
    attn = orc.transpose_remove_padding(pv, po, T).reshape(T, hidden)
    want = orc.gemm(attn, Wo)
    assert rel_err(_load(tmp_path, "ctx_out", (T, hidden)), want) < 2e-5
    kc_want, vc_want = kc.copy(), vc.copy()
    kc_want[1], vc_want[1] = kc1, vc1
    assert rel_err(_load(tmp_path, "ctx_k_cache", kc.shape), kc_want) < 1e-5
    assert rel_err(_load(tmp_path, "ctx_v_cache", vc.shape), vc_want) < 1e-5
    assert np.array_equal(_load(tmp_path, "ctx_k_cache", kc.shape)[0], kc[0])      # layer 0 untouched

    # ---- decode step at step 6 on layer 0 of a fresh cache, rotation at position `step`
    step = 6
    X = g.randv(B * hidden, 2.0).reshape(B, hidden)
    kc = g.randv(L * B * Hkv * S * D, 2.0).reshape(L, B, Hkv, S, D)
    vc = g.randv(L * B * Hkv * S * D, 2.0).reshape(L, B, Hkv, S, D)
    qkv = orc.gemm(X, Wqkv).reshape(B, QH, D)
    kc0, vc0 = np.ascontiguousarray(kc[0]), np.ascontiguousarray(vc[0])
    o = orc.decode_attn(qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:], kc0, vc0, step, rope_pos=step, rot_dim=D,
                        bias_q=bqkv[:H * D], bias_k=bqkv[H * D:(H + Hkv) * D], bias_v=bqkv[(H + Hkv) * D:])
    want = orc.gemm(o.reshape(B, hidden), Wo)
    assert rel_err(_load(tmp_path, "dec_out", (B, hidden)), want) < 2e-5
    assert rel_err(_load(tmp_path, "dec_k_cache", kc0.shape), kc0) < 1e-5
    assert rel_err(_load(tmp_path, "dec_v_cache", vc0.shape), vc0) < 1e-5

    # ---- FFN launch sequence and the two norms
    T = 3
    X = g.randv(T * hidden, 2.0).reshape(T, hidden)
    Wg = g.randv(hidden * inter, 0.2).reshape(hidden, inter)
    Wu = g.randv(hidden * inter, 0.2).reshape(hidden, inter)
    Wd = g.randv(inter * hidden, 0.2).reshape(inter, hidden)
    y = orc.gemm(orc.swiglu2(orc.gemm(X, Wg), orc.gemm(X, Wu)), Wd)
    assert rel_err(_load(tmp_path, "ffn_out", (T, hidden)), y) < 2e-5
    gamma = g.randv(hidden, 1.0)
    res = g.randv(T * hidden, 2.0).reshape(T, hidden)
    normed, new_res = orc.add_residual_rmsnorm(res, _load(tmp_path, "ffn_out", (T, hidden)), None, gamma, 1e-5)
    assert rel_err(_load(tmp_path, "norm_fused", (T, hidden)), normed) < 1e-5
    assert rel_err(_load(tmp_path, "norm_residual", (T, hidden)), new_res) < 1e-5
    assert rel_err(_load(tmp_path, "norm_plain", (T, hidden)), orc.rmsnorm(X, gamma, 1e-5)) < 1e-5

    # ---- embedding, beam-search top-K (2 of 2*V per item), sampling
    V, hid, rows = 1000, 64, 2
    table = g.randv(V * hid, 2.0).reshape(V, hid)
    assert np.array_equal(_load(tmp_path, "emb_out", (4, hid)), table[[7, 999, 0, 512]])
    probs = g.randv(rows * 2 * V, 20.0).reshape(rows, 2 * V)
    val, idx = orc.topk(probs, 2, global_ids=True)
    got_idx = _load(tmp_path, "topk_ids_as_float_bits", (rows, 2), np.int32)
    assert np.array_equal(got_idx, idx) and np.array_equal(_load(tmp_path, "topk_vals", (rows, 2)), val)
    # the uniform draw of (step 5, row b) from the library itself, then the oracle's walk
    u = torch.zeros(rows, device="cuda")
    scratch = torch.zeros(rows, device="cuda", dtype=torch.int32)
    ob.topk_sample(torch.from_numpy(idx).cuda(), torch.from_numpy(val).cuda(), rows, 2, 1.0, 5, V, 2, scratch, u_out=u)
    out, sl, fin = orc.topk_sample(idx, val, u.cpu().numpy(), vocab_size=V, end_id=2, seqlen=[10, 20])
    assert np.array_equal(_load(tmp_path, "sample_ids_as_float_bits", (rows,), np.int32), out)
    assert np.array_equal(_load(tmp_path, "sample_seqlen_as_float_bits", (rows,), np.int32), sl)


def _run(name):
    p = subprocess.run([os.path.join(BIN, name)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    return p.stdout


@needs_programs
@pytest.mark.parametrize("name", ["test_rmsnorm", "test_fused_addres_rms", "test_linear"])
def test_reference_unit_test_passes_its_own_check(name):
    # these print "the <i>th res is wrong" when their CPU function and the device result differ by > 1e-6
    assert "res is wrong" not in _run(name)


@needs_programs
def test_reference_unit_test_casual_mask():
    out = _run("test_casual_mask")      # prints every element as "CPU mask = a, GPU mask = b"
    pairs = re.findall(r"CPU mask = ([0-9.]+), GPU mask = ([0-9.]+)", out)
    assert len(pairs) == 25 and all(float(a) == float(b) for a, b in pairs)
    assert "test passed" in out


@needs_programs
def test_reference_unit_test_cal_paddingoffset():
    out = _run("test_cal_paddingoffset")
    po = [int(x) for x in re.findall(r"padding_offset = (-?\d+)", out)]
    cum = [int(x) for x in re.findall(r"cum_seqlens =(-?\d+)", out)]
    assert po[:9] == [0, 0, 0, 2, 2, 2, 4, 4, 4] and cum == [0, 3, 6, 9]   # tests/unittests/test_cal_paddingoffset.cu:56-58


@needs_programs
def test_reference_unit_test_activation():
    # in[i] = i: beyond the first few elements silu(x) = x exactly, so the reference's 1e-6 absolute check
    # only holds if expf agrees to the last bit with the host's on the small arguments; accept either verdict
    # on those, but nothing else may differ
    out = _run("test_activation")
    m = re.search(r"the (\d+)th res is wrong", out)
    assert "test passed" in out or (m and int(m.group(1)) < 32), out[-500:]


def _layer_weights(g, hidden, QH, D, inter):
    """The draws of the decoder drivers (tests/cpp/dropin_*_decoder.cpp), in their order."""
    w = {"g_attn": g.randv(hidden, 1.0), "g_ffn": g.randv(hidden, 1.0),
         "Wqkv": g.randv(hidden * QH * D, 0.2).reshape(hidden, QH * D), "bqkv": g.randv(QH * D, 0.2),
         "Wo": g.randv(hidden * hidden, 0.2).reshape(hidden, hidden), "bo": g.randv(hidden, 0.2)}
    for k in ("Wg", "Wu"):
        w[k] = g.randv(hidden * inter, 0.2).reshape(hidden, inter)
    w["Wd"] = g.randv(inter * hidden, 0.2).reshape(inter, hidden)
    w["g_out"] = g.randv(hidden, 1.0)
    return w


def _decoder_tail(orc, xn, attn, w):
    """What both decoder classes do behind the attention of a layer (self_decoder.cpp:50-73, context_decoder.cpp:104-128):
    add-residual RMSNorm with the attention's output bias, the FFN (whose result never leaves the layer: ffn.cpp:59-72
    writes a buffer of its own), add-residual RMSNorm with the next gamma."""
    normed1, res1 = orc.add_residual_rmsnorm(xn, attn, w["bo"], w["g_ffn"], 1e-5)
    normed2, res2 = orc.add_residual_rmsnorm(res1, normed1, None, w["g_out"], 1e-5)
    return normed2, res2


@needs_programs
def test_reference_ffn_layer_and_context_decoder_on_these_kernels(orc, tmp_path):
    p = subprocess.run([os.path.join(BIN, "dropin_context_decoder"), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "dropin_context_decoder ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
    B, H, Hkv, D, S, inter = 2, 4, 2, 32, 24, 192
    hidden, QH = H * D, H + 2 * Hkv
    g = Lcg()
    # LLaMAFFNLayer::forward: the down projection in the layer's own buffer
    T = 3
    X = g.randv(T * hidden, 2.0).reshape(T, hidden)
    Wg = g.randv(hidden * inter, 0.2).reshape(hidden, inter)
    Wu = g.randv(hidden * inter, 0.2).reshape(hidden, inter)
    Wd = g.randv(inter * hidden, 0.2).reshape(inter, hidden)
    want = orc.gemm(orc.swiglu2(orc.gemm(X, Wg), orc.gemm(X, Wu)), Wd)
    assert rel_err(_load(tmp_path, "ffn_class_down_out", (T, hidden)), want) < 2e-5
    # LlamaContextDecoder::forward, one layer
    w = _layer_weights(g, hidden, QH, D, inter)
    lens, hist, ctx, T, max_q, max_k = [5, 3], [2, 0], [7, 3], 8, 5, 7
    X = g.randv(T * hidden, 2.0).reshape(T, hidden)
    kc = g.randv(B * Hkv * S * D, 2.0).reshape(B, Hkv, S, D)
    vc = g.randv(B * Hkv * S * D, 2.0).reshape(B, Hkv, S, D)
    xn = orc.rmsnorm(X, w["g_attn"], 1e-5)
    po, cum, n = orc.cal_padding_offset(lens, max_q)
    mask = orc.build_causal_mask(lens, ctx, max_q, max_k, attend_history=False)
    qkv = orc.gemm(xn, w["Wqkv"]).reshape(T, QH, D)
    q_r, k_r, v_r = orc.qkv_bias_rope_transpose(qkv, w["bqkv"], po, hist, B, max_q, H, Hkv, D, 10000.0)
    orc.append_kv_cache(kc, k_r, lens, hist)
    orc.append_kv_cache(vc, v_r, lens, hist)
    k_rep, v_rep = orc.repeat_kv(kc, ctx, H, max_k), orc.repeat_kv(vc, ctx, H, max_k)
    qk = np.einsum("bhqd,bhkd->bhqk", q_r.astype(np.float64), k_rep.astype(np.float64)).astype(np.float32)
    prob = orc.scale_mask_softmax(qk, mask, D ** -0.5)
    pv = np.einsum("bhqk,bhkd->bhqd", prob.astype(np.float64), v_rep.astype(np.float64)).astype(np.float32)
    attn = orc.gemm(orc.transpose_remove_padding(pv, po, T).reshape(T, hidden), w["Wo"])
    out, res = _decoder_tail(orc, xn, attn, w)
    assert rel_err(_load(tmp_path, "cdec_k_cache", kc.shape), kc) < 1e-5
    assert rel_err(_load(tmp_path, "cdec_v_cache", vc.shape), vc) < 1e-5
    assert rel_err(_load(tmp_path, "cdec_residual", (T, hidden)), res) < 5e-5
    assert rel_err(_load(tmp_path, "cdec_out", (T, hidden)), out) < 5e-5


@needs_programs
def test_reference_self_decoder_on_these_kernels(orc, tmp_path):
    p = subprocess.run([os.path.join(BIN, "dropin_self_decoder"), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "dropin_self_decoder ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
    B, H, Hkv, D, S, inter, step = 2, 4, 2, 32, 24, 192, 4
    hidden, QH = H * D, H + 2 * Hkv
    g = Lcg()
    w = _layer_weights(g, hidden, QH, D, inter)
    X = g.randv(B * hidden, 2.0).reshape(B, hidden)
    kc = g.randv(B * Hkv * S * D, 2.0).reshape(B, Hkv, S, D)
    vc = g.randv(B * Hkv * S * D, 2.0).reshape(B, Hkv, S, D)
    xn = orc.rmsnorm(X, w["g_attn"], 1e-5)
    qkv = orc.gemm(xn, w["Wqkv"]).reshape(B, QH, D)
    b = w["bqkv"]
    o = orc.decode_attn(qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:], kc, vc, step, rope_pos=step, rot_dim=D,
                        bias_q=b[:H * D], bias_k=b[H * D:(H + Hkv) * D], bias_v=b[(H + Hkv) * D:])
    attn = orc.gemm(o.reshape(B, hidden), w["Wo"])
    out, res = _decoder_tail(orc, xn, attn, w)
    assert rel_err(_load(tmp_path, "sdec_k_cache", kc.shape), kc) < 1e-5
    assert rel_err(_load(tmp_path, "sdec_v_cache", vc.shape), vc) < 1e-5
    assert rel_err(_load(tmp_path, "sdec_residual", (B, hidden)), res) < 5e-5
    assert rel_err(_load(tmp_path, "sdec_out", (B, hidden)), out) < 5e-5
