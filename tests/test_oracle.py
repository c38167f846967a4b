"""The CPU oracle against results produced by the reference itself (tests/golden/vectors)."""

import numpy as np
import pytest

from helpers import big_cases, case_data, load_plan, small_cases, subsample
from oracle.plan_oracle import run_plan, scale_relative_error

FAST_BIG = [c for c in big_cases() if c not in ("gpt2_block_t1024", "gpt2_block_t2048")]


@pytest.mark.parametrize("case", small_cases())
def test_oracle_matches_reference_results(case):
    plan = load_plan(case)
    inputs, consts, expected = case_data(case, plan)
    got = run_plan(plan, inputs, consts, dtype=np.float32)
    for g, eager, interp in zip(got, expected["out"], expected["interp"]):
        # the reference's own tolerance against eager PyTorch (tests/test_gpu.py:37)
        np.testing.assert_allclose(g, eager, rtol=1e-4, atol=1e-5)
        # and far tighter against the reference's NumPy interpreter, whose semantics it restates
        np.testing.assert_allclose(g, interp, rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("case", small_cases())
def test_device_formulas_stay_within_tolerance(case):
    plan = load_plan(case)
    inputs, consts, expected = case_data(case, plan)
    got = run_plan(plan, inputs, consts, dtype=np.float32, device_math=True)
    for g, eager in zip(got, expected["out"]):
        np.testing.assert_allclose(g, eager, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("case", FAST_BIG)
def test_oracle_float64_matches_reference_float64(case):
    plan = load_plan(case)
    inputs, consts, expected = case_data(case, plan)
    got = run_plan(plan, inputs, consts, dtype=np.float64)
    for g, sub, step in zip(got, expected["sub"], expected["step"]):
        assert scale_relative_error(subsample(g, step), sub) < 5e-7   # stored rounded to float32


def test_torch_baseline_port_matches_the_plan_oracle():
    """The eager-PyTorch CPU baseline computes the same block as the plan oracle."""
    import torch

    from kiln_b200 import workloads as W
    from oracle.torch_block import block_forward, to_torch

    plan = load_plan("gpt2_block_t128")
    inputs, consts, _ = case_data("gpt2_block_t128", plan)
    (want,) = run_plan(plan, inputs, consts, dtype=np.float64)
    p = to_torch(W.block_params(0, 128), torch.float64)
    got = block_forward(p, torch.from_numpy(inputs[0]).double()).numpy()
    assert scale_relative_error(got, want) < 1e-7   # plan scalars (1/768, eps) are float32-rounded
