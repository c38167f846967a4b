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


ROW_MASK = torch.full((40, 512), float("-inf")).triu(1)


class ResidualNorm(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.norm = torch.nn.LayerNorm(256)

    def forward(self, a, b):
        s = a + b
        return s, self.norm(s)


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
        # row kernels with a chain in front of the reductions (register-resident rows, two row dims)
        "scaled masked softmax": (lambda x: F.softmax(x * 0.125 + ROW_MASK, -1), (torch.randn(6, 40, 512),)),
        "residual add, layernorm, both results": (ResidualNorm().eval(), (torch.randn(3, 50, 256), torch.randn(3, 50, 256))),
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


def test_profile_through_the_reference_api(kiln):
    """CompiledModule.profile (kiln/api.py:204-211) looks every returned name up among the graph's
    kernels: the executable must report Kiln kernel names, one entry per kernel, fused kernels included."""
    from kiln_b200 import workloads as W

    model, x = W.block_module(3, 128), torch.from_numpy(W.block_input(3, 128))
    compiled = kiln.compile(model, (x,), device="cuda", allow_tf32=True)
    rows = compiled.profile(x, iters=5)
    assert [r[0] for r in rows] == [k.name for k in compiled.graph.kernels]
    assert {r[1] for r in rows} == {k.kind for k in compiled.graph.kernels}
    assert all(ms >= 0.0 for *_, ms in rows) and sum(ms for *_, ms in rows) > 0.0
    # the fused attention is booked on the kernel that launches it; the four it covers take no time
    impls = dict(zip(compiled._exe.launch_names, compiled._exe.impls))
    covered = [launch.kernel for launch in compiled._exe.program.launches if impls[launch.name] == "fused_away"]
    assert len(covered) == 4 and all(ms == 0.0 for name, _, _, ms in rows if name in covered)
    compile_and_compare(kiln, model, x, allow_tf32=True, rtol=1e-2, atol=1e-2)


def test_attention_that_also_returns_its_weights_is_not_fused(kiln):
    """A model that returns the softmax weights beside the block output keeps them in a caller's
    output buffer: the fused attention kernel never writes the scores, so the library must run the
    planned kernels for such a graph (in the reduced-precision modes too)."""
    import torch.nn as nn

    class Attention(nn.Module):
        def __init__(self, t=128, d=128, heads=2):
            super().__init__()
            self.heads, self.qkv, self.proj = heads, nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.register_buffer("mask", torch.full((t, t), float("-inf")).triu(1))

        def forward(self, x):
            t, c = x.shape
            hd = c // self.heads
            q, k, v = (z.view(t, self.heads, hd).transpose(0, 1) for z in self.qkv(x).split(c, dim=1))
            weights = F.softmax((q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(hd)) + self.mask, dim=-1)
            return self.proj((weights @ v).transpose(0, 1).contiguous().view(t, c)), weights

    torch.manual_seed(5)
    model, x = Attention().eval(), torch.randn(128, 128)
    compiled = compile_and_compare(kiln, model, x, allow_tf32=True, rtol=1e-2, atol=1e-2)
    assert "attention_fused" not in compiled._exe.impls
    # and the same model without the second result does fuse (64-wide heads, 128 tokens)
    class Only(nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, x):
            return self.inner(x)[0]

    fused = compile_and_compare(kiln, Only(model).eval(), x, allow_tf32=True, rtol=1e-2, atol=1e-2)
    assert "attention_fused" in fused._exe.impls


def test_a_batch_of_sequences_as_one_graph(kiln):
    """[batch, tokens, d] through kiln.compile: the Linears become batch * tokens-row matmuls (256-row
    tiles on SM pairs here), attention runs on [batch, heads, tokens, head_dim] views; results match
    eager per sequence and match the single-sequence module on every sequence of the batch."""
    from kiln_b200 import workloads as W

    batch, tokens = 4, 128
    model = W.batched_block_module(6, tokens)
    x = torch.stack([torch.from_numpy(W.block_input(6, tokens, index=i)) for i in range(batch)])
    compiled = compile_and_compare(kiln, model, x, rtol=1e-3, atol=1e-3)
    assert "mm_tcgen05" in compiled._exe.impls
    fast = kiln.compile(model, (x,), device="cuda", allow_tf32=True)
    single = kiln.compile(W.block_module(6, tokens), (x[0],), device="cuda", allow_tf32=True)
    got = fast(x).cpu().double()
    with torch.no_grad():
        want = model(x).double()
    assert float((got - want).abs().max() / want.abs().max()) <= 2e-3
    for i in range(batch):
        one = single(x[i]).cpu().double()
        assert float((got[i] - one).abs().max() / want.abs().max()) <= 2e-3


class BatchedMlp(torch.nn.Module):
    """A Linear on a [batch, tokens, d] input: the reference plans matmul + bias, a reshape, then the
    activation / residual add as an elementwise kernel of its own."""

    def __init__(self, keep_hidden=False, reuse_hidden=False):
        super().__init__()
        torch.manual_seed(21)
        self.fc, self.proj = torch.nn.Linear(256, 512), torch.nn.Linear(512, 256)
        self.keep_hidden, self.reuse_hidden = keep_hidden, reuse_hidden

    def forward(self, x):
        h = self.fc(x)
        a = torch.nn.functional.gelu(h, approximate="tanh")
        y = x - self.proj(a)                     # the matmul's value is the second argument of the sub
        if self.reuse_hidden:
            y = y + h.mean(dim=-1, keepdim=True)  # a later kernel reads the first matmul's own output
        return (y, h) if self.keep_hidden else y


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
def test_elementwise_kernels_that_continue_a_matmul_run_in_its_epilogue(kiln, precision, monkeypatch):
    if precision == "bf16":
        monkeypatch.setenv("KILN_GPU_PRECISION", "bf16")
    tol = {"fp32": 1e-4, "tf32": 1e-2, "bf16": 5e-2}[precision]
    x = torch.randn(3, 128, 256, generator=torch.Generator().manual_seed(5))
    model = BatchedMlp().eval()
    fused = compile_and_compare(kiln, model, x, allow_tf32=precision != "fp32", rtol=tol, atol=tol)
    impls = fused._exe.impls
    assert impls.count("mm_tcgen05") == 2 and impls.count("fused_away") == 2, impls
    monkeypatch.setenv("KILN_GPU_ABSORB_ELEMENTWISE", "0")
    plain = compile_and_compare(kiln, model, x, allow_tf32=precision != "fp32", rtol=tol, atol=tol)
    assert "fused_away" not in plain._exe.impls and plain._exe.device_launches > fused._exe.device_launches
    a, b = fused(x).cpu(), plain(x).cpu()
    torch.testing.assert_close(a, b, rtol=tol, atol=tol)


@pytest.mark.parametrize("variant", ["output", "read again"])
def test_a_matmul_whose_own_value_is_needed_keeps_its_output(kiln, variant):
    """Not absorbed: the matmul's result is a plan output, or a later kernel reads it."""
    x = torch.randn(3, 128, 256, generator=torch.Generator().manual_seed(6))
    model = BatchedMlp(keep_hidden=variant == "output", reuse_hidden=variant == "read again").eval()
    compiled = compile_and_compare(kiln, model, x, allow_tf32=True, rtol=1e-2, atol=1e-2)
    names = dict(zip(compiled._exe.launch_names, compiled._exe.impls))
    gelu = [n for n, impl in names.items() if "ew" in n][0]
    assert names[gelu] != "fused_away", names


class ProjectAddNorm(torch.nn.Module):
    """LayerNorm(x + Linear(a)) on a [batch, tokens, d] input: the reference plans the add in front of the
    LayerNorm's reductions; here it runs in the matmul's epilogue and the row kernel reads the sum."""

    def __init__(self, keep_sum):
        super().__init__()
        torch.manual_seed(23)
        self.proj, self.ln = torch.nn.Linear(512, 256), torch.nn.LayerNorm(256)
        self.keep_sum = keep_sum

    def forward(self, x, a):
        s = x + self.proj(a)
        y = self.ln(s)
        return (y, s) if self.keep_sum else y


@pytest.mark.parametrize("keep_sum", [False, True], ids=["value only", "value and sum"])
@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
def test_the_add_in_front_of_a_layernorm_runs_in_the_matmul_before_it(kiln, precision, keep_sum, monkeypatch):
    if precision == "bf16":
        monkeypatch.setenv("KILN_GPU_PRECISION", "bf16")
    tol = {"fp32": 1e-4, "tf32": 1e-2, "bf16": 5e-2}[precision]
    gen = torch.Generator().manual_seed(7)
    x, a = torch.randn(3, 128, 256, generator=gen), torch.randn(3, 128, 512, generator=gen)
    model = ProjectAddNorm(keep_sum).eval()
    fused = compile_and_compare(kiln, model, x, a, allow_tf32=precision != "fp32", rtol=tol, atol=tol)
    assert "mm_tcgen05" in fused._exe.impls and "row_layernorm" in fused._exe.impls, fused._exe.impls
    steps = dict(zip(fused._exe.impls, fused._exe.chain_lengths))
    assert steps["mm_tcgen05"] == 2 and steps["row_layernorm"] == 0, steps        # bias and the add; no chain left in front of the row
    monkeypatch.setenv("KILN_GPU_ABSORB_ELEMENTWISE", "0")
    plain = compile_and_compare(kiln, model, x, a, allow_tf32=precision != "fp32", rtol=tol, atol=tol)
    steps = dict(zip(plain._exe.impls, plain._exe.chain_lengths))
    assert steps["mm_tcgen05"] == 1 and steps["row_layernorm"] == 1, steps
    for got, want in zip(outputs(fused(x, a)), outputs(plain(x, a))):
        torch.testing.assert_close(got.cpu(), want.cpu(), rtol=tol, atol=tol)


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
