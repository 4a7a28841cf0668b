"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "onellm_b200.h")).read()
    return sorted(set(re.findall(r"ONELLM_API\s+[\w\s\*]+?\b(onellm_\w+)\s*\(", text)))


def test_header_symbols_are_exported(ob):
    names = _declared()
    assert len(names) >= 25
    lib = ob.lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert lib.onellm_abi_version() == 1


def test_argument_errors_need_no_gpu(ob):
    # validation happens before any CUDA call, so these run on a CPU-only machine
    with pytest.raises(ob.OnellmError) as e:
        ob.rmsnorm(ob.F16, 0, 0, 1e-5, 1, 64, stream=0)
    assert e.value.status == -1 and "null" in str(e.value)
    with pytest.raises(ob.OnellmError) as e:
        ob.gemm(7, 16, 16, 16, 1, 64, 64, stream=0)
    assert e.value.status == -2
    with pytest.raises(ob.OnellmError):
        ob.topk(ob.F32, 16, 1, 100, 65, 16, 16, stream=0)
    with pytest.raises(ob.OnellmError):
        ob.decode_attn(ob.F16, 16, 16, 16, 8, 8, 8, None, None, None, 16, 16, 8, 8, 8, 1, 3, 2, 128, 1, 0, 128, 1e4, 1.0,
                       16, 8, None, 0, stream=0)
    assert ob.decode_attn_workspace_bytes(8, 32, 128, 2048) > 0


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "onellm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.replace("oracle's", ""), f


def test_no_cpu_fallback_when_library_is_missing(monkeypatch):
    import onellm_b200
    monkeypatch.setattr(onellm_b200, "_lib", None)
    monkeypatch.setattr(onellm_b200, "LIB_PATH", "/nonexistent/libonellm_b200.so")
    with pytest.raises(onellm_b200.OnellmError):
        onellm_b200.lib()
