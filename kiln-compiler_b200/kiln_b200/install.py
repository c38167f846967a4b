"""Make ``kiln.compile(model, inputs, device="cuda")`` use this backend.

The reference reaches its GPU backend only through lazy imports inside
``kiln.api._compile_graph_gpu`` (kiln/api.py:146-147, 157, 162) and
``kiln.gpu`` (tests, benchmarks).  ``install()`` registers this package's
modules under those names before that happens, so the frontend, IR and passes
run unmodified and hand their optimised graph to ``kiln_b200.codegen.generate``.

``kiln.api.compile_graph`` imports the MLIR-based CPU backend before it looks
at ``device`` (kiln/api.py:100-103).  Where LLVM's Python bindings are absent
that import fails although the CPU backend is never used on the CUDA path; an
empty stand-in ``mlir`` package (attribute access raises at use, not at
import) is registered in that case only.
"""

from __future__ import annotations

import importlib
import importlib.util
import sys
import types


class _Missing(types.ModuleType):
    """A module whose attributes are placeholders that fail when used."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)

        class _Absent:
            def __init__(self, *a, **k):
                raise ImportError(f"mlir.{name} is not available: LLVM's MLIR Python bindings are not installed")

        _Absent.__name__ = name
        return _Absent


def register_mlir_stub():
    """Register an empty ``mlir`` package when LLVM's Python bindings are absent. True if it did."""
    if importlib.util.find_spec("mlir") is not None:
        return False
    for name in ("mlir", "mlir.ir", "mlir.passmanager", "mlir.execution_engine", "mlir.dialects",
                 "mlir.dialects.linalg"):
        mod = _Missing(name)
        mod.__path__ = []
        sys.modules[name] = mod
    sys.modules["mlir"].ir = sys.modules["mlir.ir"]
    sys.modules["mlir"].dialects = sys.modules["mlir.dialects"]
    sys.modules["mlir.dialects"].linalg = sys.modules["mlir.dialects.linalg"]
    return True


def install(stub_mlir=True):
    """Route Kiln's ``device="cuda"`` path to kiln_b200. Idempotent. Returns the ``kiln`` module."""
    from kiln_b200 import autotune, codegen, runtime

    if stub_mlir:
        register_mlir_stub()
    pkg = types.ModuleType("kiln.gpu")
    pkg.__path__ = []
    pkg.__doc__ = "Kiln's GPU backend, provided by kiln_b200 (hand-written sm_100a kernels)."
    pkg.device, pkg.interpreting = runtime.device, runtime.interpreting
    pkg.codegen, pkg.runtime, pkg.autotune = codegen, runtime, autotune
    pkg.__all__ = ["device", "interpreting"]
    sys.modules["kiln.gpu"] = pkg
    sys.modules["kiln.gpu.codegen"] = codegen
    sys.modules["kiln.gpu.runtime"] = runtime
    sys.modules["kiln.gpu.autotune"] = autotune
    kiln = importlib.import_module("kiln")
    kiln.gpu = pkg
    return kiln
