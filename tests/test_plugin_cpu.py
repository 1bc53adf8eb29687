"""The compiler-side sources (``nnfusion_b200/nnfusion_plugin``) and the generated-project text, on the CPU.

* every plugin source passes ``g++ -std=c++14 -fsyntax-only`` against the reference's own headers (checkout given by
  ``NNFUSION_REFERENCE`` or found as a directory ``reference`` beside this repository; skipped where neither exists),
  with the stand-ins of ``nnfusion_plugin/stubs`` for generated and third-party headers that are not installed;
* the project generator reads its language units out of the plugin, and the function body it prints is the text the
  C++ emitter prints (checked on the literal fragments of the emitter's source);
* the generated runtime's ``para_info.json`` parses the reference's way.
"""
import glob
import json
import os
import re
import shutil
import subprocess

import numpy as np
import pytest

from nnfusion_b200 import codegen, runtime_loader, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "nnfusion_b200", "nnfusion_plugin")


def _reference_root():
    for cand in (os.environ.get("NNFUSION_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "src", "nnfusion", "core", "kernels", "kernel_emitter.hpp")):
            return cand
    return None


@pytest.mark.skipif(_reference_root() is None or shutil.which("g++") is None,
                    reason="needs the reference checkout and g++")
@pytest.mark.parametrize("source", sorted(os.path.basename(p) for p in glob.glob(os.path.join(PLUGIN, "*.cpp"))))
def test_plugin_source_passes_syntax_check_against_reference_headers(source):
    ref = _reference_root()
    inc = [os.path.join(PLUGIN, "stubs"), PLUGIN, os.path.join(ref, "src"), os.path.join(ref, "src", "nnfusion"),
           os.path.join(ref, "thirdparty"), os.path.join(ref, "thirdparty", "nlohmann"), os.path.join(ROOT, "include"),
           os.path.join(ref, "src", "nnfusion", "engine", "pass", "graph", "subgraph_fusion_optimizer"),
           os.path.join(ref, "src", "nnfusion", "core", "kernels", "cuda_gpu", "kernels")]
    cmd = ["g++", "-std=c++14", "-fsyntax-only"] + [f"-I{d}" for d in inc] + [os.path.join(PLUGIN, source)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_language_units_are_read_from_the_plugin():
    units = codegen.language_units()
    assert units["nnfusion::kernels::header::nnf_b200"] == '#include "nnf_b200.h"\n'
    assert "nnf_b200_ctx* nnf_b200_ctx_0" in units["nnfusion::kernels::declaration::nnf_b200_ctx"]
    macro = units["nnfusion::kernels::macro::NNF_B200_SAFE_CALL"]
    assert macro.startswith("#define NNF_B200_SAFE_CALL(func)") and "nnf_b200_last_error(nnf_b200_ctx_0)" in macro
    assert "compute_100a" in units["nnfusion::codegen::cmake::nnf_b200"]
    # every unit the header declares is defined, and the other way round
    declared = set()
    text = re.sub(r"//[^\n]*", "", open(os.path.join(PLUGIN, "nnf_b200_langunit.hpp")).read())
    stack = []
    for m in re.finditer(r"namespace (\w+)|LU_DECLARE\((\w+)\)|\}", text):
        if m.group(1):
            stack.append(m.group(1))
        elif m.group(2):
            declared.add("::".join(stack + [m.group(2)]))
        elif stack:
            stack.pop()
    assert declared == set(units)


def test_generated_body_is_the_emitters_text():
    rng = np.random.Generator(np.random.PCG64(5))
    node = codegen.DequantDotNode("DequantDot_0", 16, synth.make_weights(rng, 64, 256, 8, 256, np.float32, (0.001, 0.01),
                                                                        (120, 136)), x_dtype="float32")
    body = codegen.emit_function_body(node, 4096)
    emitter = open(os.path.join(PLUGIN, "dequant_dot_emitter.cpp")).read()
    # literal pieces of the C++ emitter's output statements appear verbatim in the generated body
    for piece in ("static const nnf_b200_linear_desc desc = {", "const nnf_b200_qweight w = {input1, input2, input3};",
                  "char* ws = (char*)(((uintptr_t)temp0 + 255) & ~(uintptr_t)255);",
                  "NNF_B200_SAFE_CALL(nnf_b200_linear(nnf_b200_ctx_0, stream, &desc, input0, &w, ",
                  "f, NNF_B200_KERNEL_AUTO, 0, 0, {0, 0}};"):
        assert piece in emitter.replace('\\n', ''), piece
        assert piece in body, piece
    assert "{16, 64, 256, 8, 0, NNF_B200_F32, NNF_B200_F32, NNF_B200_F32, NNF_B200_PROLOGUE_NONE, NNF_B200_EPILOGUE_NONE" in body
    assert body.rstrip().endswith("output0, ws, 4096));")


def test_para_info_parses_the_reference_way(tmp_path):
    doc = {"input": {"x": {"name": "Parameter_0_0", "id": "((float*)(inputs[1]))", "shape": [16, 4096]}},
           "weight": {"w": {"name": "Constant_1_0", "id": "((uint8_t*)(inputs[0]))", "shape": [4096, 4096]}},
           "output": {"y": {"name": "Result_5_0", "id": "((half*)(outputs[0]))", "shape": []}}}
    p = tmp_path / "para_info.json"
    p.write_text(json.dumps(doc))
    weights, inputs, outputs = runtime_loader.read_para_info(str(p))
    assert weights["w"].index == 0 and weights["w"].dtype == "uint8" and weights["w"].shape == (4096, 4096)
    assert inputs["x"].index == 1 and inputs["x"].dtype == "float32" and inputs["x"].tensor_name == "Parameter_0_0"
    assert outputs["y"].dtype == "float16" and outputs["y"].shape == (1,)     # scalars are fed as [1]
