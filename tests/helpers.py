"""Shared test helpers: load golden plans / vectors and build the tensors of a case."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from kiln_b200 import workloads as W

GOLDEN = Path(__file__).resolve().parent / "golden"

BIG_PREFIXES = W.BENCHMARK_PREFIXES


def is_big(case):
    return W.is_benchmark_case(case)


def all_cases():
    return sorted([p.stem for p in (GOLDEN / "plans").glob("*.json")] + W.benchmark_cases())


def small_cases():
    return [c for c in all_cases() if not is_big(c)]


def big_cases():
    """The benchmark configurations the parity tests evaluate with the NumPy oracle (the batched block
    of the benchmark step is 8 x 1024 tokens: the oracle checks the batched chain on the small
    `batched_block` case, and the big one is compared with its stored eager result only)."""
    return [c for c in all_cases() if is_big(c) and not W.batched_case(c)]


def load_plan(case):
    """Plans of the benchmark configurations ship with the package (kiln_b200/plans); the rest are fixtures here."""
    if is_big(case):
        return W.stored_plan(case)
    return json.loads((GOLDEN / "plans" / f"{case}.json").read_text())


def load_vectors(case):
    with np.load(GOLDEN / "vectors" / f"{case}.npz") as z:
        return {k: z[k] for k in z.files}


def case_data(case, plan=None):
    """(inputs, consts, expected) for a case.

    Small cases: everything comes from the stored vectors; ``expected`` is
    {"out": [...eager...], "interp": [...]}.  Big cases: tensors come from the seeded
    generators in kiln_b200.workloads, ``expected`` is {"sub": [...], "step": [...]}.
    """
    plan = plan or load_plan(case)
    vec = load_vectors(case)
    if not is_big(case):
        inputs = [vec[f"in{i}"] for i in range(len(plan["input_shapes"]))]
        consts = {n: vec[f"const:{n}"] for n in plan["const_shapes"]}
        n_out = len(plan["output_shapes"])
        return inputs, consts, {"out": [vec[f"out{i}"] for i in range(n_out)],
                                "interp": [vec[f"interp{i}"] for i in range(n_out)]}
    shapes = plan["const_shapes"]
    params, x = W.case_tensors(case)
    consts = W.plan_constants(shapes, params)
    return [x], consts, {"sub": [vec["sub0"]], "step": [int(vec["step0"])]}


def subsample(out, step):
    out = np.asarray(out)
    return out.reshape(-1, out.shape[-1])[::step]
