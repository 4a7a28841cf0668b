"""The command-line tools that ship with the package import on a box without a GPU, and the benchmark's per-kernel
cases are among the ones the kernel tool offers."""
import importlib
import re


def test_tools_import_without_a_gpu():
    for name in ("onellm_b200.kernel_cases", "onellm_b200.tune_plans", "onellm_b200.convert_hf"):
        importlib.import_module(name)


def test_bench_names_only_cases_the_kernel_tool_has():
    import os
    from onellm_b200 import kernel_cases as kc
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = open(os.path.join(root, "bench.py")).read()
    used = set(re.findall(r'make_case\("([a-z0-9_]+)"', src)) | set(re.findall(r'\("([a-z_0-9]+)", None\)', src)) | {"attn"}
    offered = set(kc.DECODE_CASES) | set(kc.PREFILL_CASES)
    assert used and used <= offered, sorted(used - offered)
