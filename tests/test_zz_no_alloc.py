"""The allocation-free decode-attention entry point against the ordinary one.

onellm_decode_attn_static serves hosts that own all device memory and cannot call cudaMalloc
for a kernel's scratch: it keeps the split-KV partials in an array built into the library.  It
must give what onellm_decode_attn gives with a caller workspace, on repeated calls (the array is
shared and keeps the previous call's contents), whether this file runs alone in a fresh process
or after every other test (pytest collects it last).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(torch, seed, B, H, Hkv, D, S):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qkv = (torch.rand(B, H + 2 * Hkv, D, device="cuda", generator=g) * 2 - 1).half()
    kc = (torch.rand(B, Hkv, S, D, device="cuda", generator=g) * 2 - 1).half()
    vc = (torch.rand(B, Hkv, S, D, device="cuda", generator=g) * 2 - 1).half()
    return qkv, kc, vc


def _args(ob, qkv, kc, vc, out, B, H, Hkv, D, S, step):
    p, e = qkv.data_ptr(), 2
    ld = (H + 2 * Hkv) * D
    return (ob.F16, p, p + H * D * e, p + (H + Hkv) * D * e, ld, ld, ld, None, None, None, kc, vc, Hkv * S * D, S * D, D,
            B, H, Hkv, D, step, step - 1, D, 10000.0, D ** -0.5, out, H * D)


def test_static_scratch_matches_workspace_path_twice(ob, cuda):
    torch = cuda
    assert ob.lib().onellm_decode_attn_static_scratch_bytes() == 8 << 20
    B, H, Hkv, D, S = 8, 32, 32, 128, 2048
    wsb = ob.decode_attn_workspace_bytes(B, H, D, S)
    ws = torch.empty(wsb, device="cuda", dtype=torch.uint8)
    for call, (seed, step) in enumerate([(1, 1500), (2, 700)]):  # two calls in a row, different shapes of split
        qkv, kc, vc = _case(torch, seed, B, H, Hkv, D, S)
        kc2, vc2 = kc.clone(), vc.clone()
        want = torch.zeros(B, H, D, device="cuda", dtype=torch.float16)
        got = torch.zeros_like(want)
        ob.decode_attn(*_args(ob, qkv, kc, vc, want, B, H, Hkv, D, S, step), ws, wsb)
        ob.decode_attn_static(*_args(ob, qkv, kc2, vc2, got, B, H, Hkv, D, S, step))
        torch.cuda.synchronize()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() / np.abs(w).max() < 1e-3, f"call {call}"  # the tolerance of the fp16 parity tests
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2)  # the new row went into the cache either way


def test_static_scratch_rejects_oversized_shapes(ob, cuda):
    torch = cuda
    B, H, D, S = 64, 64, 128, 4096  # partials of 64*64*splits*(130) floats do not fit in 8 MiB
    t = torch.zeros(16, device="cuda", dtype=torch.float16)
    with pytest.raises(ob.OnellmError) as e:
        ob.decode_attn_static(ob.F16, t, t, t, 3 * H * D, 3 * H * D, 3 * H * D, None, None, None, t, t, H * S * D, S * D, D,
                              B, H, H, D, 4000, 3999, D, 10000.0, D ** -0.5, t, H * D)
    assert e.value.status == -4 and "built" in str(e.value)
