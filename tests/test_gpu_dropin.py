"""The drop-in on a GPU, end to end: the reference's own frontend and passes (`kiln.compile(model, inputs,
device="cuda")`, imported from the pip --target copy under baseline/_ref when it is there) with this
package registered as `kiln.gpu`, against eager PyTorch at the reference's own tolerances
(tests/test_gpu.py:37 of the reference: rtol 1e-4 / atol 1e-5 in FP32, 1e-2 / 1e-2 with TF32)."""

import math
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


@pytest.fixture(scope="module")
def kiln():
    if not (REF / "kiln" / "api.py").exists():
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(REF))
    import kiln_b200

    module = kiln_b200.install()
    from kiln.gpu.codegen import generate

    assert generate.__module__.startswith("kiln_b200"), "kiln.gpu must resolve to this package"
    return module


@pytest.fixture(autouse=True)
def private_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("KILN_CACHE_DIR", str(tmp_path))
    yield


def outputs(x):
    return x if isinstance(x, (tuple, list)) else (x,)


def compile_and_compare(kiln, fn, *xs, rtol=1e-4, atol=1e-5, **flags):
    compiled = kiln.compile(fn, xs, device="cuda", **flags)
    with torch.no_grad():
        want = outputs(fn(*xs))
    got = outputs(compiled(*xs))
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.is_cuda and g.dtype == torch.float32
        torch.testing.assert_close(g.cpu(), w, rtol=rtol, atol=atol)
    return compiled


torch.manual_seed(11)
SIDE = torch.randn(4, 1)
PROJ = torch.randn(41, 66)


def small_models():
    from kiln_b200 import workloads as W

    two_layer = torch.nn.Sequential(torch.nn.Linear(20, 36), torch.nn.GELU(approximate="tanh"), torch.nn.Linear(36, 12)).eval()
    return {
        "two-layer mlp": (two_layer, (torch.randn(6, 20),)),
        "layernorm": (torch.nn.LayerNorm(40).eval(), (torch.randn(9, 40),)),
        "softmax": (lambda x: F.softmax(x, -1), (torch.randn(2, 7, 29),)),
        "column sums": (lambda x: x.sum(0, keepdim=True) * x, (torch.randn(5, 12),)),
        "reduce over two dims": (lambda x: x.sum((0, 2), keepdim=True) + x.amax(0, keepdim=True), (torch.randn(3, 6, 5),)),
        "strided views": (lambda x: (x.view(5, 2, 6).transpose(0, 1) * 0.5, x.t()), (torch.randn(10, 6),)),
        "bmm with a transposed operand": (lambda a, b: torch.bmm(a, b.transpose(1, 2)), (torch.randn(2, 8, 24), torch.randn(2, 13, 24))),
        "one-row matmul": (lambda a: F.gelu(a @ PROJ, approximate="tanh"), (torch.randn(1, 41),)),
        "odd sizes": (lambda a, b: a @ b - 0.5, (torch.randn(31, 47), torch.randn(47, 21))),
        "broadcast side input": (lambda x: x / (x.sum(-1, keepdim=True) ** 2 + 1.0) + SIDE, (torch.randn(4, 44),)),
        "unary ops": (lambda x: torch.tanh(x) + torch.sigmoid(x) + torch.erf(x) + F.gelu(x) + torch.relu(-x), (torch.randn(5, 26) * 3,)),
        "small block": (W.block_module(5, 16, d=64, heads=4), (torch.randn(16, 64),)),
    }


@pytest.mark.parametrize("name", list(small_models()))
def test_compiled_module_matches_eager(kiln, name):
    fn, xs = small_models()[name]
    compile_and_compare(kiln, fn, *xs)


def test_long_rows(kiln):
    compile_and_compare(kiln, torch.nn.LayerNorm(9000).eval(), torch.randn(2, 9000))
    compile_and_compare(kiln, lambda x: F.softmax(x, -1), torch.randn(3, 6000))


def test_the_reference_s_plan_is_what_runs(kiln):
    from kiln_b200 import workloads as W

    model, x = W.block_module(0, 128), torch.from_numpy(W.block_input(0, 128))
    exact = compile_and_compare(kiln, model, x)
    assert len(exact.report.kernels) == 11 and exact.report.arena_bytes == 2752512
    fast = compile_and_compare(kiln, model, x, allow_tf32=True, rtol=1e-2, atol=1e-2)
    assert fast.report.arena_bytes == exact.report.arena_bytes


def test_autotuned_matmuls(kiln):
    model = torch.nn.Sequential(torch.nn.Linear(768, 3072), torch.nn.GELU(approximate="tanh"), torch.nn.Linear(3072, 768)).eval()
    x = torch.randn(256, 768)
    compiled = compile_and_compare(kiln, model, x, allow_tf32=True, autotune=True, rtol=1e-2, atol=1e-2)
    log = compiled.report.autotune
    assert len(log) == 2 and all(entry["source"] in ("tuned", "cache") and entry["tflops"] > 0 for entry in log)
    assert "autotuned" in str(compiled.report) or "tuned" in str(compiled.report)


def test_unfrozen_weights_are_read_at_call_time(kiln):
    model = torch.nn.Linear(24, 10).cuda()
    x = torch.randn(5, 24, device="cuda")
    compiled = kiln.compile(model, (x,), device="cuda", freeze=False)
    with torch.no_grad():
        model.weight.mul_(-1.5)
        torch.testing.assert_close(compiled(x), model(x), rtol=1e-4, atol=1e-5)


def test_wrong_shape_is_a_value_error(kiln):
    compiled = kiln.compile(torch.nn.Linear(8, 4).eval(), (torch.randn(3, 8),), device="cuda")
    with pytest.raises(ValueError):
        compiled(torch.randn(4, 8))


def test_scale_of_the_attention_matches_the_model(kiln):
    """1/sqrt(head dim) and the causal mask survive the trip through the fused attention kernel (TF32 mode)."""
    from kiln_b200 import workloads as W

    model, x = W.block_module(2, 256), torch.from_numpy(W.block_input(2, 256))
    compiled = kiln.compile(model, (x,), device="cuda", allow_tf32=True)
    with torch.no_grad():
        want = model(x).double()
    got = compiled(x).cpu().double()
    assert float((got - want).abs().max() / want.abs().max()) <= 2e-3
    assert math.isfinite(float(got.sum()))
