"""Run a stored plan on the GPU through the package's executable (and so through the C ABI)."""

from __future__ import annotations

import numpy as np
import torch

from helpers import case_data, load_plan
from kiln_b200.codegen import program_from_plan
from kiln_b200.runtime import GPUExecutable
from kiln_b200.spec import PlanSpec


def build_executable(case, precision="fp32", cuda_graphs=True, configs=None, plan_json=None, consts=None):
    plan_json = plan_json or load_plan(case)
    plan = PlanSpec.from_json(plan_json)
    if consts is None:
        _, consts, _ = case_data(case, plan_json)
    program = program_from_plan(plan, precision, configs)
    return GPUExecutable(program, plan.arena_bytes, consts, plan.input_shapes, plan.output_shapes,
                         cuda_graphs=cuda_graphs)


def run_case(case, precision="fp32", cuda_graphs=True, configs=None):
    plan_json = load_plan(case)
    inputs, consts, expected = case_data(case, plan_json)
    exe = build_executable(case, precision, cuda_graphs, configs, plan_json, consts)
    outs = exe(*[torch.from_numpy(np.ascontiguousarray(x)) for x in inputs])
    torch.cuda.synchronize()
    exe.status()
    return exe, [o.cpu().numpy() for o in outs], (plan_json, inputs, consts, expected)
