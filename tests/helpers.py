"""Shared test helpers: load golden plans / vectors and build the tensors of a case."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from kiln_b200 import workloads as W

GOLDEN = Path(__file__).resolve().parent / "golden"

BIG_PREFIXES = ("gpt2_block_t", "mlp_2048", "linear_", "bias_gelu_", "layernorm_2048", "softmax_12x")


def is_big(case):
    return case.startswith(BIG_PREFIXES)


def all_cases():
    return sorted(p.stem for p in (GOLDEN / "plans").glob("*.json"))


def small_cases():
    return [c for c in all_cases() if not is_big(c)]


def big_cases():
    return [c for c in all_cases() if is_big(c)]


def load_plan(case):
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
    if case.startswith("gpt2_block_t"):
        t = int(case[len("gpt2_block_t"):])
        seed = 0 if t == 128 else 4
        params, x = W.block_params(seed, t), W.block_input(seed, t)
    elif case == "mlp_2048":
        params, x = W.mlp_params(), W.mlp_input()
    elif case.startswith("linear_"):
        m, n, k = (int(v) for v in case[len("linear_"):].split("x"))
        params, x = W.linear_params(m, n, k)
    elif case.startswith("bias_gelu"):
        params, x = W.bias_gelu_data()
    elif case.startswith("layernorm_2048"):
        params, x = W.layernorm_data()
    elif case.startswith("softmax_12x"):
        params, x = W.softmax_data()
    else:
        raise KeyError(case)
    consts = W.plan_constants(shapes, params)
    return [x], consts, {"sub": [vec["sub0"]], "step": [int(vec["step0"])]}


def subsample(out, step):
    out = np.asarray(out)
    return out.reshape(-1, out.shape[-1])[::step]
