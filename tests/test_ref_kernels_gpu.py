"""This library's kernels against the REFERENCE's own CUDA kernels on the same inputs (fp32).

The reference kernels come from oracle/_ref/libonellm_ref.so, compiled from the reference tree in place;
the tests are skipped where that library was not built.  Only launchers whose indexing was checked by
reading are called, inside the argument ranges noted in oracle/ref_exports.cu.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_lib
    lib = ref_lib.load()
    if lib is None:
        pytest.skip("oracle/_ref has not been built")
    return lib


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_rmsnorm_vs_reference_kernel(ob, cuda, ref):
    torch = cuda
    torch.manual_seed(0)
    x = torch.randn(16, 4096, device="cuda")
    g = 1 + 0.1 * torch.randn(4096, device="cuda")
    a, b = x.clone(), x.clone()
    assert ref.ref_gpu_rmsnorm(_p(a), _p(g), C.c_float(1e-5), 16, 4096) == 0
    ob.rmsnorm(ob.F32, b, g, 1e-5, 16, 4096)
    torch.cuda.synchronize()
    assert rel_err(b.cpu().numpy(), a.cpu().numpy()) < 1e-5


def test_swiglu_and_embedding_vs_reference_kernels(ob, cuda, ref):
    torch = cuda
    torch.manual_seed(1)
    inp = torch.randn(16, 2, 11008, device="cuda") * 3
    a, b = torch.zeros(16, 11008, device="cuda"), torch.zeros(16, 11008, device="cuda")
    assert ref.ref_gpu_swiglu(_p(inp), _p(a), 16, 11008) == 0
    ob.swiglu(ob.F32, inp, b, 16, 11008)
    torch.cuda.synchronize()
    assert rel_err(b.cpu().numpy(), a.cpu().numpy()) < 1e-5
    table = torch.randn(1000, 256, device="cuda")
    ids = torch.randint(0, 1000, (4, 9), device="cuda", dtype=torch.int32)
    a, b = torch.zeros(4, 9, 256, device="cuda"), torch.zeros(36, 256, device="cuda")
    assert ref.ref_gpu_embedding(_p(ids), _p(a), _p(table), 4, 9, 256, 1000) == 0
    ob.embedding(ob.F32, ids, b, table, 36, 256, 1000)
    torch.cuda.synchronize()
    assert torch.equal(a.reshape(36, 256), b)


def test_prefill_rope_and_cache_write_vs_reference_kernels(ob, cuda, ref, orc):
    """reference: bias+RoPE+transpose kernel, then the cache append kernel; here: one fused kernel."""
    torch = cuda
    torch.manual_seed(2)
    B, H, Hkv, D, S = 2, 8, 8, 64, 48
    lens, hist = [5, 9], [3, 0]
    max_q, T = max(lens), sum(lens)
    po, cum, _ = orc.cal_padding_offset(lens, max_q)
    QKV = torch.randn(T, H + 2 * Hkv, D, device="cuda")
    bias = 0.1 * torch.randn((H + 2 * Hkv) * D, device="cuda")
    q_ref = torch.zeros(B, H, max_q, D, device="cuda")
    k_ref, v_ref = torch.zeros(B, Hkv, max_q, D, device="cuda"), torch.zeros(B, Hkv, max_q, D, device="cuda")
    d_po = torch.from_numpy(po).cuda()
    d_hist = torch.tensor(hist, device="cuda", dtype=torch.int32)
    d_len = torch.tensor(lens, device="cuda", dtype=torch.int32)
    assert ref.ref_gpu_qkv_bias_rope(_p(q_ref), _p(k_ref), _p(v_ref), _p(QKV.clone()), _p(bias), _p(d_po), _p(d_hist), _p(d_len), B,
                                     max_q, T, H, Hkv, D, D, C.c_float(10000.0)) == 0
    kc_ref, vc_ref = torch.zeros(B, Hkv, S, D, device="cuda"), torch.zeros(B, Hkv, S, D, device="cuda")
    assert ref.ref_gpu_append_kv(_p(k_ref), _p(v_ref), _p(d_len), _p(d_hist), _p(kc_ref), _p(vc_ref), B, Hkv, max_q, S, D) == 0
    mine = QKV.clone()
    kc, vc = torch.zeros_like(kc_ref), torch.zeros_like(vc_ref)
    ob.qkv_bias_rope_kvcache(ob.F32, mine, bias, torch.from_numpy(cum).cuda(), d_hist, kc, vc, Hkv * S * D, S * D, D, T, B, H, Hkv, D,
                             D, 10000.0, S)
    torch.cuda.synchronize()
    # the two GPU paths use the same float math up to the pow / sincos implementations
    assert rel_err(kc.cpu().numpy(), kc_ref.cpu().numpy()) < 2e-5 and rel_err(vc.cpu().numpy(), vc_ref.cpu().numpy()) < 1e-6
    q_packed = torch.stack([q_ref[(t + int(po[t])) // max_q, :, (t + int(po[t])) % max_q] for t in range(T)])
    assert rel_err(mine[:, :H].cpu().numpy(), q_packed.cpu().numpy()) < 2e-5


def test_decode_attention_vs_reference_kernel(ob, cuda, ref):
    """masked_MHA_kernel with its parameters in declaration order, inside the range where it is well defined:
    one warp per block (D = 32), step <= D, Hkv == H, caches [S, B, H, D], RoPE at position `step`."""
    torch = cuda
    torch.manual_seed(3)
    B, H, D, S = 2, 4, 32, 32
    for step in (1, 7, 32):
        q, k, v = (torch.rand(B, H, D, device="cuda") * 2 - 1 for _ in range(3))
        bias = 0.1 * torch.randn(3 * H * D, device="cuda")
        kc, vc = torch.rand(S, B, H, D, device="cuda") * 2 - 1, torch.rand(S, B, H, D, device="cuda") * 2 - 1
        kc_ref, vc_ref = kc.clone(), vc.clone()
        out_ref, out = torch.zeros(B, H, D, device="cuda"), torch.zeros(B, H, D, device="cuda")
        assert ref.ref_gpu_masked_mha(_p(q), _p(k), _p(v), _p(bias), _p(kc_ref), _p(vc_ref), _p(out_ref), B, H, D, step, D,
                                      C.c_float(10000.0)) == 0
        ob.decode_attn(ob.F32, q, k, v, H * D, H * D, H * D, bias.data_ptr(), bias.data_ptr() + H * D * 4, None, kc, vc, H * D, D,
                       B * H * D, B, H, H, D, step, step, D, 10000.0, D ** -0.5, out, H * D, None, 0)
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), out_ref.cpu().numpy()) < 2e-5, step
        assert rel_err(kc[step - 1].cpu().numpy(), kc_ref[step - 1].cpu().numpy()) < 2e-5
        assert torch.equal(vc[step - 1], vc_ref[step - 1])
