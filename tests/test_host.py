"""Host-side logic that needs no GPU: plan extraction, lowering to the C ABI, the library's
exports, the drop-in registration, and the replica sharding of the benchmark (gloo, 2 ranks)."""

import ctypes
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import GOLDEN, all_cases, load_plan
from kiln_b200 import _cabi, lowering
from kiln_b200.codegen import launches_of, program_from_plan
from kiln_b200.spec import PlanSpec

ROOT = Path(__file__).resolve().parent.parent
# the reference as installed beside this package (baseline/install_reference.py), or a checkout named by KILN_REFERENCE
REFERENCE = Path(os.environ.get("KILN_REFERENCE", ROOT / "baseline" / "_ref"))
REFERENCE_TESTS = REFERENCE / "tests" if (REFERENCE / "tests" / "models").is_dir() else REFERENCE / "kiln_tests"
needs_reference = pytest.mark.skipif(not (REFERENCE / "kiln" / "api.py").exists(),
                                     reason="the reference is neither installed under baseline/_ref nor named by KILN_REFERENCE")


@pytest.fixture(scope="session")
def lib():
    _cabi.build()
    return _cabi.load()


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "kb200.h").read_text()
    declared = set(re.findall(r"\b(kb200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_cabi.EXPORTS), declared ^ set(_cabi.EXPORTS)
    for name in declared:
        assert hasattr(lib, name)
    assert lib.kb200_version() == _cabi.ABI_VERSION
    assert lib.kb200_last_error() == b""


def test_struct_layout_matches_the_header():
    # sizes implied by include/kb200.h (natural alignment, no packing)
    assert ctypes.sizeof(_cabi.TapeOp) == 20
    assert ctypes.sizeof(_cabi.Operand) == 16 + 8 * _cabi.MAX_RANK
    expected = 16 + 8 * _cabi.MAX_RANK + 8 + 16 + 64 * _cabi.MAX_OPERANDS + 20 * _cabi.MAX_TAPE + 32 + 32
    assert ctypes.sizeof(_cabi.KernelDesc) == expected


def test_option_numbers_match_the_header():
    """The plan options the runtime sets (attention fusion ... shared attention query tiles) carry the header's numbers."""
    header = (ROOT / "include" / "kb200.h").read_text()
    declared = {name: int(value) for name, value in re.findall(r"\bKB200_(OPT_[A-Z0-9_]+)\s*=\s*(\d+)", header)}
    assert declared and sorted(declared.values()) == list(range(1, len(declared) + 1))
    ours = {name: getattr(_cabi, name) for name in dir(_cabi) if name.startswith("OPT_")}
    assert ours == declared


def test_plan_create_rejects_bad_arguments_without_a_gpu(lib):
    out = ctypes.c_void_p()
    assert lib.kb200_plan_create(None, 1, 0, ctypes.byref(out)) == -1
    assert b"descriptor" in lib.kb200_last_error()
    assert lib.kb200_plan_create(None, 0, 0, None) == -1
    assert lib.kb200_plan_launch(None, None) == -1
    assert lib.kb200_plan_launch_count(None) == 0
    lib.kb200_plan_destroy(None)


@pytest.mark.parametrize("case", all_cases())
def test_every_plan_lowers(case):
    plan = PlanSpec.from_json(load_plan(case))
    assert PlanSpec.loads(plan.dumps()).to_json() == plan.to_json()
    program = program_from_plan(plan, "fp32")
    descs = lowering.lower(plan, program.launches, "fp32", sorted(plan.const_shapes))
    assert len(program.launches) >= len(plan.kernels)
    for d, launch in zip(descs, program.launches):
        assert 1 <= d.iter_rank <= _cabi.MAX_RANK and 1 <= d.n_tape <= _cabi.MAX_TAPE
        stores = [t for t in d.tape[:d.n_tape] if t.opcode == _cabi.OPCODES["STORE"]]
        assert stores, launch.name
        for i, t in enumerate(d.tape[:d.n_tape]):
            if t.opcode >= _cabi.OPCODES["add"] and t.opcode != _cabi.OPCODES["STORE"]:
                assert t.a < i
        # every operand stays inside the buffer the plan gives it
        for o in d.operands[:d.n_operands]:
            extents = list(d.iter_shape[:d.iter_rank])
            last = o.elem_offset + sum((e - 1) * s for e, s in zip(extents, o.stride) if e > 0)
            if o.base_kind == _cabi.BASE_KINDS["arena"] and d.kclass != _cabi.K_MATMUL:
                assert (last + 1) * 4 <= plan.arena_bytes


def test_launch_list_matches_the_reference_generator():
    """Same launches, in the same order, touching the same buffers as the reference's own
    kiln.gpu.codegen.generate produced for the same graphs (recorded in reference_plans.json)."""
    ref = json.loads((GOLDEN / "reference_plans.json").read_text())
    for case in all_cases():
        plan = PlanSpec.from_json(load_plan(case))
        ours = launches_of(plan)
        theirs = ref[case]["launches"]
        assert [l.name for l in ours] == [t[0] for t in theirs], case
        kinds = {"elementwise": "elementwise", "row": "row", "reduction": "reduction", "matmul": "matmul"}
        assert [kinds[l.kind] for l in ours] == [t[1] for t in theirs], case
        for l, t in zip(ours, theirs):
            assert [list(b) for b in l.bases] == t[3], (case, l.name)
        assert plan.arena_bytes == ref[case]["arena_bytes"]
        assert len(plan.kernels) == len(ref[case]["kernels"])


def test_golden_block_plans_are_the_published_ones():
    """Kernel count and arena bytes of the GPT-2 block at every benchmark length."""
    want = {128: 2752512, 512: 29884416, 1024: 110100480, 2048: 421527552}
    offsets_128 = [1179648, 0, 1966080, 1179648, 1966080, 1179648, 0, 1572864, 1966080, 0]
    for t, arena in want.items():
        plan = PlanSpec.from_json(load_plan(f"gpt2_block_t{t}"))
        assert len(plan.kernels) == 11 and plan.arena_bytes == arena
        assert [k.kind for k in plan.kernels] == ["reduction", "matmul", "copy", "matmul", "reduction", "matmul",
                                                  "copy", "matmul", "reduction", "matmul", "matmul"]
    plan = PlanSpec.from_json(load_plan("gpt2_block_t128"))
    got = [k.outputs[0][1].offset * 4 for k in plan.kernels[:10]]
    assert got == offsets_128
    assert plan.kernels[10].outputs[0][1].base == ("output", 0)
    assert PlanSpec.from_json(load_plan("mlp_2048")).arena_bytes == 25165824


@needs_reference
def test_generate_on_a_live_reference_graph_reproduces_the_golden_plan():
    """kiln.compile's own frontend and passes, then this package's generate(): bit-identical plan."""
    code = f"""
import sys, json
sys.path[:0] = [{str(ROOT / 'kiln-compiler_b200')!r}, {str(REFERENCE)!r}, {str(REFERENCE_TESTS)!r}]
import torch, kiln_b200
kiln = kiln_b200.install()
from kiln.api import Options, build_passes
from kiln.frontend.fx_import import import_exported
from kiln.passes.manager import PassManager
from kiln.gpu.codegen import generate, default_matmul_config
from models.transformer import Block
g = import_exported(torch.export.export(Block(768, 12, 128).eval(), (torch.randn(128, 768),)).run_decompositions())
before = str(g)
PassManager(build_passes(Options(tiling=False))).run(g)
after = str(g)
prog = generate(g, allow_tf32=True)
assert str(g) == after, "generate() must not mutate the graph"
assert isinstance(prog.source, str) and len(prog.launches) == 11 and prog.precision == "tf32"
plan = prog.plan.to_json(); plan["name"] = "gpt2_block_t128"
print(json.dumps(plan, sort_keys=True))
try:
    kiln.compile(Block(32, 2, 8).eval(), (torch.randn(8, 32),), device="cuda")
except RuntimeError as e:
    assert "needs a CUDA GPU" in str(e)
"""
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = json.loads(proc.stdout.strip().splitlines()[-1])
    assert got == json.loads(json.dumps(load_plan("gpt2_block_t128"), sort_keys=True))


@needs_reference
def test_the_package_s_own_block_module_compiles_to_the_golden_plan():
    """workloads.block_module (what bench.py hands to the reference's Triton backend for the side-by-side
    run) goes through the reference's frontend and passes to the same 11-kernel plan as the reference's
    own test model, and evaluates like the functional restatement the CPU baseline times."""
    code = f"""
import sys, json
sys.path[:0] = [{str(ROOT / 'kiln-compiler_b200')!r}, {str(ROOT)!r}, {str(REFERENCE)!r}]
import numpy as np, torch, kiln_b200
from kiln_b200 import workloads as W
from oracle.torch_block import block_forward, to_torch
kiln = kiln_b200.install()
from kiln.api import Options, build_passes
from kiln.frontend.fx_import import import_exported
from kiln.passes.manager import PassManager
from kiln.gpu.codegen import generate
model = W.block_module(0, 128)
x = torch.from_numpy(W.block_input(0, 128))
with torch.no_grad():
    assert torch.allclose(model(x), block_forward(to_torch(W.block_params(0, 128)), x), rtol=1e-5, atol=1e-6)
g = import_exported(torch.export.export(model, (x,)).run_decompositions())
PassManager(build_passes(Options(tiling=False))).run(g)
plan = generate(g, allow_tf32=True).plan.to_json(); plan["name"] = "gpt2_block_t128"
print(json.dumps(plan, sort_keys=True))
"""
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = json.loads(proc.stdout.strip().splitlines()[-1])
    assert got == json.loads(json.dumps(load_plan("gpt2_block_t128"), sort_keys=True))


def test_chain_and_collapse_helpers():
    shape, strides, segs = lowering.collapse([2, 16, 8], [[16, 1, 96], [128, 8, 1]])
    assert shape == [32, 8] and strides == [[1, 96], [8, 1]] and segs == [2]
    shape, strides, _ = lowering.collapse([4, 1, 8], [[8, 0, 1], [0, 0, 1]])
    assert shape == [4, 8] and strides == [[8, 1], [0, 1]]
    shape, strides, _ = lowering.collapse([4, 8], [[8, 1], [8, 1]])
    assert shape == [32] and strides == [[1], [1]]


def test_replica_timing_reduction_with_two_gloo_ranks(tmp_path):
    """The benchmark's only cross-rank step: barrier + max over ranks of the step time."""
    script = tmp_path / "ranks.py"
    script.write_text(f"""
import os, sys
sys.path.insert(0, {str(ROOT)!r})
import bench
dist, rank, world, local = bench.dist_setup(2)
assert world == 2
bench.barrier(dist)
t = bench.max_over_ranks(dist, 10.0 + rank)
assert t == 11.0, t
first = rank * bench.SEQS
open({str(tmp_path)!r} + f"/rank{{rank}}.txt", "w").write(f"sequences {{first}} {{first + bench.SEQS - 1}}")
dist.destroy_process_group()
""")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                          capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert (tmp_path / "rank0.txt").read_text() == "sequences 0 63"
    assert (tmp_path / "rank1.txt").read_text() == "sequences 64 127"
