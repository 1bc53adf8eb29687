"""Generated-project look-alike: what NNFusion's ``cuda_codegen`` writes for a graph whose only compute node is a
``DequantDot``, produced here without the compiler (which cannot be built where its third-party dependencies are
missing), from the very text the plugin's emitter and language units hold.

Output directory (the reference's ``nnfusion_rt/cuda_codegen``):

* ``nnfusion_rt.cu`` / ``nnfusion_rt.h`` -- ``extern "C"`` ``get_device_type``, ``get_workspace_size``, ``cuda_init``,
  ``kernel_entry``, ``kernel_entry_host``, ``cuda_free`` (``src/nnfusion/engine/pass/codegen/cuda_codegen_pass.cpp:117-168,
  194-211,1118-1133``; ``base_codegen_pass.cpp:206-249,326-353``), one kernel function per node named
  ``<OpType>_<dtypes...>_<kernel type>_<node name>`` (``src/nnfusion/core/kernels/kernel_emitter.cpp:90-99``) with the
  parameter list ``cudaStream_t, inputs, outputs, temps`` (``:101-143,160-181``), constants read from
  ``Constant/<tensor>.bin`` in ``cuda_init`` (``src/nnfusion/core/kernels/cuda_gpu/kernels/constant.cpp:36-59``), one
  memory pool allocated in ``cuda_init`` (``src/nnfusion/engine/memory_allocator.cpp:284-300``);
* ``para_info.json`` -- ``src/nnfusion/engine/pass/extract_graph_signature.cpp:150-236``;
* ``libnnfusion_naive_rt.so`` -- built with nvcc against ``libnnf_b200.so`` by :func:`build` (the reference builds the
  same target name with the generated CMakeLists, ``cuda_codegen_pass.cpp:1360-1437``).

The function body of the node is the text ``cuda::DequantDot::emit_function_body`` prints
(``nnfusion_plugin/dequant_dot_emitter.cpp``); header, declaration and safe-call macro are read out of the
``LU_DEFINE`` statements of ``nnfusion_plugin/codegen_units.cpp``, so the plugin stays the single source of the text.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import _lib as L
from .synth import QuantLinear

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
PLUGIN = os.path.join(PKG, "nnfusion_plugin")

_C_TYPE = {"float32": "float", "float16": "half", "uint8": "uint8_t"}
_DT_ENUM = {"float32": "NNF_B200_F32", "float16": "NNF_B200_F16"}
_EPI_ENUM = {"none": "NNF_B200_EPILOGUE_NONE", "bias": "NNF_B200_EPILOGUE_BIAS",
             "silu_mul": "NNF_B200_EPILOGUE_SILU_MUL", "add": "NNF_B200_EPILOGUE_ADD"}


def language_units() -> dict:
    """``{unit name: code}`` of every ``LU_DEFINE`` in the plugin's ``codegen_units.cpp`` (plain and raw strings)."""
    text = open(os.path.join(PLUGIN, "codegen_units.cpp")).read()
    units = {}
    for m in re.finditer(r'LU_DEFINE\(\s*([\w:]+)\s*,\s*(R"\((.*?)\)"|"((?:[^"\\]|\\.)*)")\s*\)\s*;', text, re.S):
        name = m.group(1)
        code = m.group(3) if m.group(3) is not None else bytes(m.group(4), "utf-8").decode("unicode_escape")
        units[name] = code
    return units


@dataclass
class DequantDotNode:
    """One ``DequantDot`` node of the graph: y = epilogue(x . dequant(W)^T)."""
    name: str
    M: int
    weight: QuantLinear
    x_dtype: str = "float16"          # numpy dtype names
    y_dtype: Optional[str] = None
    epilogue: str = "none"            # none | bias | add
    bias: Optional[np.ndarray] = None  # fp32 [N] with epilogue "bias"

    @property
    def desc(self) -> L.LinearDesc:
        w = self.weight
        d = L.LinearDesc()
        d.M, d.N, d.K, d.w_bits = self.M, w.N, w.K, w.bits
        d.group_size = 0 if w.group == w.K else w.group
        d.x_dtype = L.F16 if self.x_dtype == "float16" else L.F32
        d.y_dtype = L.F16 if (self.y_dtype or self.x_dtype) == "float16" else L.F32
        d.scale_dtype = L.F16 if w.scale.dtype == np.float16 else L.F32
        d.epilogue = {"none": L.EPILOGUE_NONE, "bias": L.EPILOGUE_BIAS, "add": L.EPILOGUE_ADD}[self.epilogue]
        d.rms_eps = 1e-6
        return d


def emit_function_body(node: DequantDotNode, workspace_bytes: int) -> str:
    """The text of ``cuda::DequantDot::emit_function_body`` for this node (no RMSNorm prologue, no second weight set:
    the cases this generator is used for)."""
    w = node.weight
    y_dtype = node.y_dtype or node.x_dtype
    scale_dtype = "float16" if w.scale.dtype == np.float16 else "float32"
    group = 0 if w.group == w.K else w.group
    bias = "input4" if node.epilogue in ("bias", "add") else "nullptr"
    lines = [
        f"static const nnf_b200_linear_desc desc = {{{node.M}, {w.N}, {w.K}, {w.bits}, {group}, "
        f"{_DT_ENUM[node.x_dtype]}, {_DT_ENUM[y_dtype]}, {_DT_ENUM[scale_dtype]}, NNF_B200_PROLOGUE_NONE, "
        f"{_EPI_ENUM[node.epilogue]}, 1e-06f, NNF_B200_KERNEL_AUTO, 0, 0, {{0, 0}}}};",
        "const nnf_b200_qweight w = {input1, input2, input3};",
    ]
    if workspace_bytes > 0:
        lines.append("char* ws = (char*)(((uintptr_t)temp0 + 255) & ~(uintptr_t)255);")
    lines.append(f"NNF_B200_SAFE_CALL(nnf_b200_linear(nnf_b200_ctx_0, stream, &desc, input0, &w, nullptr, nullptr, "
                 f"{bias}, output0, {'ws' if workspace_bytes > 0 else 'nullptr'}, {workspace_bytes}));")
    return "\n".join("    " + ln for ln in lines) + "\n"


def _tensor_file(name: str) -> str:
    return f"Constant/{name}.bin"


def generate(out_dir: str, node: DequantDotNode, lib=None) -> str:
    """Writes the project for a one-node graph  Parameter_0 -> DequantDot -> Result_0  into ``out_dir`` and returns the
    path of ``nnfusion_rt.cu``.  ``lib``: the loaded ``libnnf_b200.so`` (for the workspace size), default: loaded here."""
    lib = lib or L.load()
    os.makedirs(os.path.join(out_dir, "Constant"), exist_ok=True)
    w = node.weight
    d = node.desc
    import ctypes
    workspace_bytes = int(lib.nnf_b200_linear_workspace_bytes(None, ctypes.byref(d)))
    y_dtype = node.y_dtype or node.x_dtype
    scale_dtype = "float16" if w.scale.dtype == np.float16 else "float32"
    units = language_units()

    # ---- constants, dumped raw like ConstantCodegen does (packed uint4 travels as uint8)
    consts = [("Constant_1_0", "uint8", np.ascontiguousarray(w.wq)),
              ("Constant_2_0", scale_dtype, np.ascontiguousarray(w.scale)),
              ("Constant_3_0", "uint8", np.ascontiguousarray(w.zpq))]
    if node.epilogue == "bias":
        consts.append(("Constant_4_0", "float32", np.ascontiguousarray(node.bias, np.float32)))
    for name, _, arr in consts:
        arr.tofile(os.path.join(out_dir, _tensor_file(name)))

    # ---- one memory pool: constants, activations, workspace (offsets 256-byte aligned)
    offsets, cursor = {}, 0

    def place(name, nbytes):
        nonlocal cursor
        offsets[name] = cursor
        cursor += (nbytes + 255) // 256 * 256

    for name, _, arr in consts:
        place(name, arr.nbytes)
    x_bytes = node.M * w.K * (2 if node.x_dtype == "float16" else 4)
    y_bytes = node.M * w.N * (2 if y_dtype == "float16" else 4)
    place("Parameter_0_0", x_bytes)           # device copy of the input for kernel_entry_host
    place("Result_5_0", y_bytes)
    if node.epilogue == "add":
        place("Parameter_4_0", y_bytes)
    if workspace_bytes:
        place("DequantDot_0_workspace", workspace_bytes + 256)
    pool_bytes = cursor

    xt, yt, st = _C_TYPE[node.x_dtype], _C_TYPE[y_dtype], _C_TYPE[scale_dtype]
    in4 = {"bias": "float* input4, ", "add": f"{yt}* input4, ", "none": ""}[node.epilogue]
    dtypes = [xt, "uint8_t", st, "uint8_t"] + ({"bias": ["float"], "add": [yt], "none": []}[node.epilogue]) + [yt]
    fname = "DequantDot_" + "_".join(dtypes) + "_cuda_lib_" + node.name
    temp = "char* temp0" if workspace_bytes else ""
    sig = f"void {fname}(cudaStream_t stream, {xt}* input0, uint8_t* input1, {st}* input2, uint8_t* input3, {in4}" \
          f"{yt}* output0{', ' + temp if temp else ''})"

    entry_in = f"{xt}* Parameter_0_0" + (f", {yt}* Parameter_4_0" if node.epilogue == "add" else "")
    call_in4 = {"bias": "Constant_4_0, ", "add": "Parameter_4_0, ", "none": ""}[node.epilogue]
    call = f"{fname}(0, Parameter_0_0, Constant_1_0, Constant_2_0, Constant_3_0, {call_in4}Result_5_0" \
           f"{', DequantDot_0_workspace' if workspace_bytes else ''});"
    loads = "\n".join(
        f"    load_constant(group_0_CUDA_GPU0_memory_pool + {offsets[n]}, \"{_tensor_file(n)}\", {a.nbytes});"
        for n, _, a in consts)
    ptrs = "\n".join(
        f"    {n} = ({_C_TYPE[t]}*)(group_0_CUDA_GPU0_memory_pool + {offsets[n]});" for n, t, _ in consts)
    decls = "\n".join(f"{_C_TYPE[t]}* {n};" for n, t, _ in consts)
    host_add = ""
    if node.epilogue == "add":
        host_add = (f"    CUDA_SAFE_CALL(cudaMemcpyAsync(addend_dev, Parameter_4_0_host, {y_bytes}, cudaMemcpyHostToDevice, 0));\n")
    src = f"""// Generated by nnfusion_b200.codegen for the graph  Parameter_0 -> DequantDot({node.name}) -> Result_0.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <sstream>
#include <stdexcept>
#include <cuda_fp16.h>
{units['nnfusion::kernels::header::nnf_b200']}#include "nnfusion_rt.h"

#define CUDA_SAFE_CALL(x)                                                                          \\
    do                                                                                             \\
    {{                                                                                              \\
        cudaError_t result = (x);                                                                  \\
        if (result != cudaSuccess)                                                                 \\
        {{                                                                                          \\
            std::stringstream safe_call_ss;                                                        \\
            safe_call_ss << "\\nerror: " #x " failed with error"                                    \\
                         << "\\nfile: " << __FILE__ << "\\nline: " << __LINE__                       \\
                         << "\\nmsg: " << cudaGetErrorString(result);                               \\
            throw std::runtime_error(safe_call_ss.str());                                          \\
        }}                                                                                          \\
    }} while (0)
{units['nnfusion::kernels::declaration::nnf_b200_ctx']}{units['nnfusion::kernels::macro::NNF_B200_SAFE_CALL']}
char* group_0_CUDA_GPU0_memory_pool;
{decls}
{xt}* Parameter_0_0_dev;
{yt}* Result_5_0;
{(yt + '* addend_dev;') if node.epilogue == 'add' else ''}
{'char* DequantDot_0_workspace;' if workspace_bytes else ''}

static void load_constant(char* dst, const char* file, size_t bytes)
{{
    FILE* f = fopen(file, "rb");
    if (!f)
        throw std::runtime_error(std::string("cannot open ") + file);
    char* host = (char*)malloc(bytes);
    size_t got = fread(host, 1, bytes, f);
    fclose(f);
    if (got != bytes)
    {{
        free(host);
        throw std::runtime_error(std::string("short read on ") + file);
    }}
    CUDA_SAFE_CALL(cudaMemcpy(dst, host, bytes, cudaMemcpyHostToDevice));
    free(host);
}}

// Node name:	{node.name}
// Description:	DequantDot
{sig}
{{
{emit_function_body(node, workspace_bytes)}}}

extern "C" int get_device_type()
{{
    return 0;
}}

extern "C" int64_t get_workspace_size()
{{
    return 0;
}}

extern "C" void cuda_init()
{{
    CUDA_SAFE_CALL(cudaSetDevice(0));
    NNF_B200_SAFE_CALL(nnf_b200_init(0, &nnf_b200_ctx_0));
    CUDA_SAFE_CALL(cudaMalloc((void**)&group_0_CUDA_GPU0_memory_pool, {pool_bytes}));
    CUDA_SAFE_CALL(cudaMemset((void*)group_0_CUDA_GPU0_memory_pool, 0, {pool_bytes}));
{ptrs}
    Parameter_0_0_dev = ({xt}*)(group_0_CUDA_GPU0_memory_pool + {offsets['Parameter_0_0']});
    Result_5_0 = ({yt}*)(group_0_CUDA_GPU0_memory_pool + {offsets['Result_5_0']});
{('    addend_dev = (' + yt + '*)(group_0_CUDA_GPU0_memory_pool + ' + str(offsets.get('Parameter_4_0', 0)) + ');') if node.epilogue == 'add' else ''}
{('    DequantDot_0_workspace = group_0_CUDA_GPU0_memory_pool + ' + str(offsets.get('DequantDot_0_workspace', 0)) + ';') if workspace_bytes else ''}
{loads}
}}

// the output goes where the caller says (-fextern_result_memory): Result_0 is a device pointer
extern "C" int kernel_entry({entry_in}, {yt}* Result_0)
{{
    {yt}* Result_5_0 = Result_0;
    {call}
    return 0;
}}

// Device address of a pinned, mapped host buffer (nullptr for pageable memory).
static void* device_view_of_host(const void* p)
{{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess)
    {{
        (void)cudaGetLastError();
        return nullptr;
    }}
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}}

// host buffers in, host buffers out (-fhost_entry): the input is copied to the device, the node runs, the result comes
// back, the stream is synchronised.  When the result buffer is pinned (mapped into the device's address space) the
// node stores its result straight into it over PCIe, which saves the copy back; otherwise the result is copied.
extern "C" int kernel_entry_host({xt}* Parameter_0_0_host{(', ' + yt + '* Parameter_4_0_host') if node.epilogue == 'add' else ''}, {yt}* Result_0_host)
{{
    CUDA_SAFE_CALL(cudaMemcpyAsync(Parameter_0_0_dev, Parameter_0_0_host, {x_bytes}, cudaMemcpyHostToDevice, 0));
{host_add}    {yt}* mapped = ({yt}*)device_view_of_host(Result_0_host);
    if (mapped)
        kernel_entry(Parameter_0_0_dev{', addend_dev' if node.epilogue == 'add' else ''}, mapped);
    else
    {{
        kernel_entry(Parameter_0_0_dev{', addend_dev' if node.epilogue == 'add' else ''}, Result_5_0);
        CUDA_SAFE_CALL(cudaMemcpyAsync(Result_0_host, Result_5_0, {y_bytes}, cudaMemcpyDeviceToHost, 0));
    }}
    CUDA_SAFE_CALL(cudaStreamSynchronize(0));
    return 0;
}}

extern "C" void cuda_free()
{{
    CUDA_SAFE_CALL(cudaFree(group_0_CUDA_GPU0_memory_pool));
    nnf_b200_free(nnf_b200_ctx_0);
    nnf_b200_ctx_0 = nullptr;
}}
"""
    header = f"""// Generated by nnfusion_b200.codegen.
#pragma once
#include <stdint.h>
#include <cuda_fp16.h>
extern "C" int get_device_type();
extern "C" int64_t get_workspace_size();
extern "C" void cuda_init();
extern "C" int kernel_entry({entry_in}, {yt}* Result_0);
extern "C" int kernel_entry_host({xt}* Parameter_0_0_host{(', ' + yt + '* Parameter_4_0_host') if node.epilogue == 'add' else ''}, {yt}* Result_0_host);
extern "C" void cuda_free();
"""
    with open(os.path.join(out_dir, "nnfusion_rt.h"), "w") as f:
        f.write(header)
    path = os.path.join(out_dir, "nnfusion_rt.cu")
    with open(path, "w") as f:
        f.write(src)

    # ---- para_info.json, as ExtractGraphSignature writes it
    def io(name, idx, ctype, shape, side):
        return {"name": name, "id": f"(({ctype}*)({side}[{idx}]))", "shape": list(shape)}

    para = {"input": {"x": io("Parameter_0_0", 0, xt, (node.M, w.K), "inputs")},
            "output": {"y": io("Result_5_0", 0, yt, (node.M, w.N), "outputs")}}
    if node.epilogue == "add":
        para["input"]["addend"] = io("Parameter_4_0", 1, yt, (node.M, w.N), "inputs")
    with open(os.path.join(out_dir, "para_info.json"), "w") as f:
        json.dump(para, f, indent=2)
    return path


def build(out_dir: str) -> str:
    """nvcc: ``nnfusion_rt.cu`` -> ``libnnfusion_naive_rt.so`` linked against ``libnnf_b200.so`` (run-time search path set
    to the package directory).  Returns the library's path."""
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    lib = os.path.join(out_dir, "libnnfusion_naive_rt.so")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(ROOT, "include"), "-I", out_dir, os.path.join(out_dir, "nnfusion_rt.cu"), "-o", lib,
           "-L", PKG, "-lnnf_b200", "-Xlinker", f"-rpath={PKG}", "-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the generated runtime:\n" + r.stdout)
    return lib
