"""ctypes binding of the C ABI declared in include/kb200.h, and the nvcc build.

The shared library is built in-tree (``kiln_b200/_lib/libkb200.so``) for
sm_100a only.  There is no CPU or PyTorch fallback: if the library is
missing, ``load()`` raises and nothing above it can run.
"""

from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

ABI_VERSION = 3
MAX_RANK, MAX_OPERANDS, MAX_TAPE = 6, 12, 96

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR.parent / "csrc"
INCLUDE_DIR = PKG_DIR.parent.parent / "include"
LIB_PATH = PKG_DIR / "_lib" / "libkb200.so"

K_ELEMENTWISE, K_ROW, K_REDUCE, K_MATMUL = 0, 1, 2, 3
OPT_FUSE_ATTENTION = 1
OPT_DEPENDENT_LAUNCH = 2
OPT_FOLD_OPERAND_COPIES = 3
OPT_CONCURRENCY = 4
OPT_ABSORB_ELEMENTWISE = 5
OPT_MIRROR_ONLY = 6
OPT_FP32_ATTENTION = 7
OPT_ATTENTION_SPLIT = 8
BASE_KINDS = {"arena": 0, "const": 1, "input": 2, "output": 3}
PRECISIONS = {"fp32": 0, "tf32": 1, "bf16": 2}
OPCODES = {
    "LOAD": 0, "IMM": 1, "ACC": 2, "add": 3, "sub": 4, "mul": 5, "div": 6, "maximum": 7, "minimum": 8,
    "neg": 9, "relu": 10, "exp": 11, "tanh": 12, "sigmoid": 13, "erf": 14, "gelu_tanh": 15, "gelu_erf": 16,
    "rsqrt": 17, "sqrt": 18, "copy": 19, "reduce_sum": 20, "reduce_max": 21, "STORE": 22,
}
STATUS_EXC = {-1: ValueError, -2: NotImplementedError, -3: ValueError, -4: RuntimeError, -5: RuntimeError,
              -6: RuntimeError}


class TapeOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("level", C.c_int32),
                ("imm", C.c_float)]


class Operand(C.Structure):
    _fields_ = [("base_kind", C.c_int32), ("base_index", C.c_int32), ("elem_offset", C.c_int64),
                ("stride", C.c_int64 * MAX_RANK)]


class KernelDesc(C.Structure):
    _fields_ = [("kclass", C.c_int32), ("precision", C.c_int32), ("iter_rank", C.c_int32), ("n_kept", C.c_int32),
                ("iter_shape", C.c_int64 * MAX_RANK), ("k_extent", C.c_int64),
                ("a_slot", C.c_int32), ("b_slot", C.c_int32), ("n_operands", C.c_int32), ("n_tape", C.c_int32),
                ("operands", Operand * MAX_OPERANDS), ("tape", TapeOp * MAX_TAPE),
                ("cfg", C.c_int32 * 8), ("name", C.c_char * 32)]


EXPORTS = {
    "kb200_version": (C.c_int, []),
    "kb200_last_error": (C.c_char_p, []),
    "kb200_plan_create": (C.c_int, [C.POINTER(KernelDesc), C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "kb200_plan_bind": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64,
                                  C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_int,
                                  C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_int,
                                  C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_int]),
    "kb200_plan_set_option": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "kb200_plan_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "kb200_kernel_launch": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "kb200_plan_launch_count": (C.c_int, [C.c_void_p]),
    "kb200_kernel_impl": (C.c_char_p, [C.c_void_p, C.c_int]),
    "kb200_kernel_chain_length": (C.c_int, [C.c_void_p, C.c_int]),
    "kb200_plan_status": (C.c_int, [C.c_void_p]),
    "kb200_plan_selftest_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "kb200_plan_destroy": (None, [C.c_void_p]),
    "kb200_matmul_bf16_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                           C.c_void_p, C.c_void_p]),
    "kb200_matmul_bf16_static_status": (C.c_int, []),
}

_lib = None


def sources():
    return sorted(CSRC_DIR.glob("*.cu"))


def nvcc_command(out=LIB_PATH, verbose=False):
    cmd = ["nvcc", "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
           f"-I{INCLUDE_DIR}", f"-I{CSRC_DIR}"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    return cmd + [str(s) for s in sources()] + ["-o", str(out)]


def needs_build():
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = sources() + sorted(CSRC_DIR.glob("*.cuh")) + sorted(CSRC_DIR.glob("*.h")) + sorted(INCLUDE_DIR.glob("*.h"))
    return any(d.stat().st_mtime > built for d in deps)


def build(force=False, verbose=False):
    """Compile csrc/*.cu into libkb200.so for sm_100a (cross-compiles without a GPU)."""
    if not force and not needs_build():
        return LIB_PATH
    if shutil.which("nvcc") is None:
        raise RuntimeError("kiln_b200: nvcc not found, cannot build libkb200.so")
    LIB_PATH.parent.mkdir(parents=True, exist_ok=True)
    tmp = LIB_PATH.with_suffix(f".{os.getpid()}.tmp.so")
    proc = subprocess.run(nvcc_command(tmp, verbose), capture_output=True, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"kiln_b200: nvcc failed\n{proc.stdout}\n{proc.stderr}")
    tmp.replace(LIB_PATH)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


def load():
    """The loaded library.  Raises if it is missing or its ABI version differs."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"kiln_b200: {LIB_PATH} is missing; run kiln_b200.build() "
                           "(there is no fallback path without the CUDA library)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.kb200_version() != ABI_VERSION:
        raise RuntimeError(f"kiln_b200: libkb200.so has ABI {lib.kb200_version()}, expected {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def check(status, lib=None):
    if status == 0:
        return
    lib = lib or load()
    msg = lib.kb200_last_error().decode(errors="replace")
    raise STATUS_EXC.get(status, RuntimeError)(f"kb200: {msg} (status {status})")
