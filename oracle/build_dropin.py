"""Compiles the REFERENCE's own layer classes, examples and unit tests, unchanged and where they lie,
against the drop-in headers of this repository (include/onellm) and links them with libonellm_b200.so.

    python oracle/build_dropin.py /path/to/oneLLM

Test infrastructure only: it shows that a oneLLM tree builds on top of this library without edits, and
produces the programs the GPU tests run (the reference's unit tests on this library's kernels, and
tests/cpp/dropin_*.cpp, which drive the reference's layer classes).  No reference source is copied
and the reference's build system is not used.  Outputs go to oracle/_ref/dropin/ only (git-ignored).
Include order: include/onellm first, so "src/utils/..", "src/kernels/..", "src/weights/..",
"src/memory/.." and "src/models/.." resolve to the drop-in headers; the reference tree second, for the
layer classes' own headers under src/layers/.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "dropin")

LAYERS = {"ffn": "src/layers/ffn/ffn.cpp", "masked_self_attention": "src/layers/attention/masked_self_attention.cpp",
          "context_attention": "src/layers/attention/context_attention.cpp",
          "self_decoder": "src/layers/decoder/self_decoder.cpp", "context_decoder": "src/layers/decoder/context_decoder.cpp"}
# example -> layer objects it needs.  masked_attn_example.cpp does not compile against the reference's
# own headers either (it calls forward() with five arguments).
EXAMPLES = {"ffn_example": ("examples/cpp/ffn/ffn_example.cpp", ["ffn"]),
            "context_attn_example": ("examples/cpp/attention/context_attn_example.cpp", ["context_attention"]),
            "self_decoder_example": ("examples/cpp/decoder/self_decoder_example.cpp", ["self_decoder", "masked_self_attention", "ffn"]),
            "context_decoder_example": ("examples/cpp/decoder/context_decoder_example.cpp", ["context_decoder", "context_attention", "ffn"])}
# this repository's programs that drive the layer classes (tests/cpp) -> layer objects they link
DRIVERS = {"dropin_layers": ["context_attention", "masked_self_attention"],
           "dropin_self_decoder": ["self_decoder", "masked_self_attention", "ffn"],
           "dropin_context_decoder": ["context_decoder", "context_attention", "ffn"]}
# unit tests that build; test_decoder_masked_attn.cu and the empty test_layernorm.cu do not build in the
# reference tree either
UNIT_TESTS = ["test_activation", "test_append_kvcache", "test_batch_gemm", "test_beamsearch_topK", "test_cal_paddingoffset",
              "test_casual_mask", "test_fused_addres_rms", "test_fused_trans_remv_pad", "test_input_embedding", "test_linear",
              "test_qkv_bias_and_rope", "test_rmsnorm", "test_softmax", "test_topK_sampling", "test_transpose"]
# of those, the ones whose inputs are fully initialised and whose checks read host memory only: safe to
# run on a GPU as they are (tests/test_dropin_gpu.py)
RUNNABLE = ["test_rmsnorm", "test_fused_addres_rms", "test_activation", "test_linear", "test_cal_paddingoffset", "test_casual_mask"]


def _run(jobs):
    procs = [(name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)) for name, cmd in jobs]
    bad = []
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode:
            sys.stderr.write(f"--- {name}\n{out[-3000:]}\n")
            bad.append(name)
    if bad:
        raise SystemExit("did not build against the drop-in headers: " + ", ".join(bad))


def build(ref):
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "include", "onellm"), "-I" + ref,
           "-I" + os.path.join(cuda, "include")]
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cxx = [gxx, "-std=c++17", "-O1", "-w"] + inc
    obj = lambda n: os.path.join(OUT, "obj", n + ".o")
    jobs = [(n, cxx + ["-c", os.path.join(ref, src), "-o", obj(n)]) for n, src in LAYERS.items()]
    jobs += [(n, cxx + ["-c", os.path.join(ref, src), "-o", obj(n)]) for n, (src, _) in EXAMPLES.items()]
    # the unit tests use CUDA's host-side rsqrt/min: nvcc, although they hold no device code
    nvcc = ["nvcc", "-std=c++17", "-w", "-gencode", "arch=compute_100a,code=sm_100a"] + inc
    jobs += [(t, nvcc + ["-c", os.path.join(ref, "tests", "unittests", t + ".cu"), "-o", obj(t)]) for t in UNIT_TESTS]
    jobs += [(n, cxx + ["-I" + os.path.join(ROOT, "tests", "cpp"), "-c", os.path.join(ROOT, "tests", "cpp", n + ".cpp"), "-o", obj(n)])
             for n in DRIVERS]
    _run(jobs)
    link = ["-L" + os.path.join(ROOT, "onellm_b200"), "-lonellm_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-lcublas",
            "-Wl,-rpath,$ORIGIN/../../../onellm_b200"]
    jobs = [(n, [gxx, "-o", os.path.join(OUT, n), obj(n)] + [obj(d) for d in deps] + link) for n, (_, deps) in EXAMPLES.items()]
    jobs += [(t, [gxx, "-o", os.path.join(OUT, t), obj(t)] + link) for t in UNIT_TESTS]
    jobs += [(n, [gxx, "-o", os.path.join(OUT, n), obj(n)] + [obj(d) for d in deps] + link) for n, deps in DRIVERS.items()]
    _run(jobs)
    return OUT


if __name__ == "__main__":
    default = os.environ.get("ONELLM_REFERENCE_TREE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    print(build(sys.argv[1] if len(sys.argv) > 1 else default))
