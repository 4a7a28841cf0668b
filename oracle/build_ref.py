"""Compiles the REFERENCE's own sources, where they lie, into oracle/_ref/libonellm_ref.so.

    python oracle/build_ref.py /path/to/oneLLM

Test infrastructure only.  No reference source is copied: nvcc reads the files from the reference
tree (kernels under src/kernels, the unit-test sources for their CPU helper functions with `main`
renamed), plus oracle/ref_exports.cu which wraps them in C entry points.  The reference's own
build system is not used.  Outputs go to oracle/_ref/ only (git-ignored).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

KERNELS = ["rmsnorm_kernel", "fused_addresidual_norm", "activation_kernel", "input_embedding", "qkv_bias_and_RoPE",
           "append_to_kvcache", "transpose_kernel", "fused_transpose_reshape_remv_pad", "build_casual_mask", "qkv_linear"]
TESTS = ["test_fused_addres_rms", "test_activation", "test_linear", "test_input_embedding", "test_casual_mask",
         "test_qkv_bias_and_rope"]


def build(ref):
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    base = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-w", "-Xcompiler", "-fPIC", "-I" + ref,
            "-include", os.path.join(HERE, "ref_prelude.h")]
    jobs = []
    for k in KERNELS:
        jobs.append((os.path.join(ref, "src", "kernels", k + ".cu"), k, []))
    jobs.append((os.path.join(ref, "src", "kernels", "cublas_wrapper.cc"), "cublas_wrapper", ["-x", "cu"]))
    for t in TESTS:
        # every test source defines main and a CheckResult of its own: rename them per file
        jobs.append((os.path.join(ref, "tests", "unittests", t + ".cu"), t,
                     [f"-Dmain=ref_main_{t}", f"-DCheckResult=ref_check_{t}", f"-DcheckResults=ref_checks_{t}"]))
    jobs.append((os.path.join(HERE, "ref_exports.cu"), "ref_exports", []))
    objs, procs = [], []
    for src, name, extra in jobs:
        obj = os.path.join(OUT, "obj", name + ".o")
        objs.append(obj)
        procs.append((name, subprocess.Popen(base + extra + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                             stderr=subprocess.STDOUT, text=True)))
    bad = False
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode:
            sys.stderr.write(f"--- {name}\n{out}\n")
            bad = True
    if bad:
        raise SystemExit("reference sources did not compile")
    lib = os.path.join(OUT, "libonellm_ref.so")
    subprocess.check_call(["nvcc", "-shared", "-o", lib] + objs + ["-lcudart", "-lcublas"])
    return lib


if __name__ == "__main__":
    default = os.environ.get("ONELLM_REFERENCE_TREE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    print(build(sys.argv[1] if len(sys.argv) > 1 else default))
