"""Lift the reference's own pure-torch functions out of its source tree.  TEST INFRASTRUCTURE ONLY.

The reference example modules cannot be imported (their top level imports the
reference's compiler, which needs an NPU toolchain), but the torch reference
programs inside them are plain Python.  This helper parses a module with
``ast``, selects function definitions by name and executes only those in a
namespace that holds ``torch``.  No reference source is copied into this
repository: the functions are read from the reference tree where it lies, at
run time, and only on the machine that has that tree.

Used by ``tests/golden/make_golden.py`` (to generate the committed vectors) and
by the CPU tests that compare the restatement in ``oracle/qgemm_oracle.py``
with the reference's functions whenever the tree is present.
"""
from __future__ import annotations

import ast
import importlib.util
import os

import torch

# the reference checkout: QGEMM_REFERENCE_ROOT, else a directory "reference" beside this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("QGEMM_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))


def reference_available() -> bool:
    return os.path.isfile(os.path.join(
        REFERENCE_ROOT, "examples/quant_batch_matmul/example_quant_batch_matmul.py"))


def lift(relpath: str, names, extra_globals=None) -> dict:
    """Return {name: function} for the named top-level functions of a reference file."""
    path = os.path.join(REFERENCE_ROOT, relpath)
    with open(path, "r") as f:
        tree = ast.parse(f.read(), filename=path)
    wanted = set(names)
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    for fn in body:
        fn.decorator_list = []
    missing = wanted - {n.name for n in body}
    if missing:
        raise KeyError(f"{relpath}: no top-level function(s) {sorted(missing)}")
    ns = {"torch": torch, "__name__": "lifted_reference"}
    if extra_globals:
        ns.update(extra_globals)
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return {n: ns[n] for n in names}


def load_quantize_utils():
    """tilelang/quantize/utils.py imports torch lazily and loads standalone."""
    path = os.path.join(REFERENCE_ROOT, "tilelang/quantize/utils.py")
    spec = importlib.util.spec_from_file_location("ref_quantize_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def w8a8_ref_program():
    return lift("examples/quant_batch_matmul/example_quant_batch_matmul.py", ["ref_program"])["ref_program"]


def w8a8_unbatched_ref_program():
    return lift("examples/quant_batch_matmul/example_quant_matmul.py", ["ref_program"])["ref_program"]


def dequant_fine_grained():
    return lift(
        "examples/dequantize_gemm/example_dequant_gemm_fine_grained.py",
        ["torch_unpack_uint4_to_fp16", "torch_unpack_uint4_to_int8", "ref_program_fp16",
         "ref_program_int8", "check_unpack_functions"])


def w4a8():
    return lift("examples/dequantize_gemm/example_dequant_gemm_w4a8.py",
                ["torch_convert", "ref_program", "generate_quantized_weight"])


def two_scale_golden():
    return lift("examples/deepseek_v4/int8_gemm.py", ["int8_gemm_torch_optimized"])["int8_gemm_torch_optimized"]


def act_quant_golden():
    import typing
    return lift("examples/deepseek_v4/act_quant.py", ["act_quant_torch"], {"Tuple": typing.Tuple})["act_quant_torch"]


def grouped_gemm_reference():
    return lift("examples/grouped_gemm/example_grouped_gemm_fwd.py", ["torch_gmm", "construct_inputs"])
