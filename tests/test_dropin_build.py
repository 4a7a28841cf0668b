"""The drop-in C++ headers (include/onellm): they compile on their own, and, where a oneLLM tree is at
hand, the reference's layer classes, examples and unit tests compile and link against them unchanged."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the oneLLM source tree: ONELLM_REFERENCE_TREE, or a directory named "reference" beside this repository
REFERENCE_TREE = os.environ.get("ONELLM_REFERENCE_TREE", os.path.join(os.path.dirname(ROOT), "reference"))
GXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"

HEADERS = """
#include "src/utils/tensor.h"
#include "src/utils/params.h"
#include "src/utils/cuda_utils.h"
#include "src/weights/llama/llama_weights.h"
#include "src/memory/allocator/cuda_allocator.h"
#include "src/models/llama/llama_params.h"
#include "src/kernels/activation_kernel.h"
#include "src/kernels/append_to_kvcache.h"
#include "src/kernels/attn_softmax_kernel.h"
#include "src/kernels/beamsearch_topK.h"
#include "src/kernels/build_casual_mask.h"
#include "src/kernels/cal_paddingoffset.h"
#include "src/kernels/cublas_wrapper.h"
#include "src/kernels/decoder_masked_attn.h"
#include "src/kernels/fused_addresidual_norm.h"
#include "src/kernels/fused_transpose_reshape_remv_pad.h"
#include "src/kernels/input_embedding.h"
#include "src/kernels/qkv_bias_and_RoPE.h"
#include "src/kernels/qkv_linear.h"
#include "src/kernels/rmsnorm_kernel.h"
#include "src/kernels/topK_sampling.h"
#include "src/kernels/transpose_kernel.h"
"""


def test_headers_compile_alone_and_twice(tmp_path, ob):
    # two translation units including everything, linked together: every definition is inline
    body = HEADERS + """
template void launchAct<float>(const float*, float*, int, int);
template void launchAct<half>(const half*, half*, int, int);
template void launchFusedAddBiasResidualRMSNorm<float>(float*, float*, const float*, const float*, float, int, int);
template void launchBuildCausalMasks<float>(float*, const int*, const int*, int, int, int);
int NAME() { TensorMap m{{"a", Tensor(CPU, getTensorType<int>(), {1})}}; return (int)m.size() + (int)getTypeSize(FP16); }
"""
    objs = []
    for name in ("tu_one", "tu_two"):
        src = tmp_path / (name + ".cpp")
        src.write_text(body.replace("NAME", name).replace("template void", "template void" if name == "tu_one" else "extern template void"))
        obj = str(tmp_path / (name + ".o"))
        subprocess.check_call([GXX, "-std=c++17", "-Wall", "-Wno-unused-function", "-I" + os.path.join(ROOT, "include"),
                               "-I" + os.path.join(ROOT, "include", "onellm"), "-I/usr/local/cuda/include", "-c", str(src), "-o", obj])
        objs.append(obj)
    main = tmp_path / "main.cpp"
    main.write_text("int tu_one(); int tu_two(); int main() { return tu_one() + tu_two() == 4 ? 0 : 1; }\n")
    exe = str(tmp_path / "prog")
    subprocess.check_call([GXX, "-o", exe, str(main)] + objs + ["-L" + os.path.join(ROOT, "onellm_b200"), "-lonellm_b200",
                                                                "-L/usr/local/cuda/lib64", "-lcudart",
                                                                "-Wl,-rpath," + os.path.join(ROOT, "onellm_b200")])
    # an invalid tensor is dropped by the map, so each unit returns 0 + 2
    assert subprocess.call([exe]) == 0


@pytest.mark.skipif(not os.path.isdir(REFERENCE_TREE), reason="needs a oneLLM source tree")
def test_reference_layers_examples_and_unit_tests_build_unchanged(ob):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import build_dropin
    finally:
        sys.path.pop(0)
    out = build_dropin.build(REFERENCE_TREE)
    for name in list(build_dropin.EXAMPLES) + build_dropin.UNIT_TESTS + list(build_dropin.DRIVERS):
        assert os.access(os.path.join(out, name), os.X_OK), name
    assert set(build_dropin.RUNNABLE) <= set(build_dropin.UNIT_TESTS)
