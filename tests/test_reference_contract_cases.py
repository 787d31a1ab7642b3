"""The reference's own contract tests, run against this library.

``tests/test_contract.py`` restates the input contract.  This file does not restate
anything: where a checkout of the reference is available (the directory named by
``B200MOE_REFERENCE_ROOT``, else the build container's default) it loads the reference's test module
``tests/test_goal_1b_edge_cases.py`` with the name ``fastpath`` bound to this package, and
runs the reference's assertions on the error table -- the cases that must fail before any
backend is chosen, so they hold for a library that has no PyTorch execution path:
wrong shapes/dtypes/ranges, mismatched ``top_k``, a compiled backend given CPU tensors, and
backend/quantisation pairs that must not change silently.  Skipped where no checkout exists.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import pytest

REFERENCE_ROOT = Path(os.environ.get("B200MOE_REFERENCE_ROOT", "/root/reference"))
REFERENCE_TESTS = REFERENCE_ROOT / "tests" / "test_goal_1b_edge_cases.py"

# the reference's test functions that only exercise the error table
ERROR_TABLE_CASES = [
    ("test_strict_shape_dtype_contiguous_and_index_validation", ()),
    ("test_top_k_and_declared_dimensions_must_match", ()),
    ("test_compiled_backend_on_cpu_is_rejected_without_fallback", ("cutlass_bf16",)),
    ("test_compiled_backend_on_cpu_is_rejected_without_fallback", ("cutlass_nvfp4",)),
    ("test_backend_and_quant_mode_cannot_silently_change", ()),
]


@pytest.fixture(scope="module")
def reference_tests():
    if not REFERENCE_TESTS.exists():
        pytest.skip(f"no reference checkout at {REFERENCE_ROOT}")
    import b200moe

    alias = types.ModuleType("fastpath")
    alias.B300MoEWorkspace = b200moe.B300MoEWorkspace
    alias.b300_moe_forward = b200moe.b300_moe_forward
    previous = sys.modules.get("fastpath")
    sys.modules["fastpath"] = alias
    try:
        spec = importlib.util.spec_from_file_location("reference_edge_cases", REFERENCE_TESTS)
        module = importlib.util.module_from_spec(spec)
        assert spec.loader is not None
        spec.loader.exec_module(module)
        assert module.b300_moe_forward is b200moe.b300_moe_forward
        yield module
    finally:
        if previous is None:
            sys.modules.pop("fastpath", None)
        else:
            sys.modules["fastpath"] = previous


@pytest.mark.parametrize("name,args", ERROR_TABLE_CASES,
                         ids=[n + ("_" + a[0] if a else "") for n, a in ERROR_TABLE_CASES])
def test_reference_error_table_holds_for_this_library(reference_tests, name, args) -> None:
    getattr(reference_tests, name)(*args)
