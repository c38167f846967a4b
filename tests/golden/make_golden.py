"""Regenerate the golden fixtures from the reference implementation.

    python tests/golden/make_golden.py [--reference /path/to/kiln-compiler]

Needs the reference checkout (default: $KILN_REFERENCE, else ../reference next
to this repository root's parent).  It imports the reference's frontend, passes,
NumPy interpreter and its test models, runs them on seeded inputs, and writes:

  plans/<case>.json      the launch plan kiln_b200.codegen.plan_of derives from the
                         reference's optimised graph (kernels, layouts, arena offsets); the
                         benchmark configurations' plans go to kiln_b200/plans/ in the package
  vectors/<case>.npz     inputs, constants and the reference's own results:
                         out<i>  eager PyTorch (what tests/test_gpu.py of the reference
                                 compares against), interp<i>  kiln.ir.interpret
  reference_plans.json   per case: the reference's kernel list, arena / naive /
                         lower-bound bytes and the launch list its own
                         kiln.gpu.codegen.generate produces (names, kinds, grids, bases)

Large cases (the GPT-2-small block, the 2048-token MLP, the Linear sweep, the
[2048, 3072] fused ops) take their tensors from kiln_b200.workloads, so only a
strided subsample of the reference's float64 result is stored (key sub<i>, rounded to
float32, with the row step in step<i>).
"""

from __future__ import annotations

import argparse
import json
import os
import random
import sys
from dataclasses import replace
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT / "kiln-compiler_b200"))


def slug(name):
    return "".join(c if c.isalnum() else "_" for c in name).strip("_").lower()


class FnModule(torch.nn.Module):
    def __init__(self, fn):
        super().__init__()
        self.fn = fn

    def forward(self, *args):
        return self.fn(*args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KILN_REFERENCE", str(ROOT.parent / "reference")))
    ap.add_argument("--only", default=None, help="regenerate just this case (its slug), keeping every other fixture as it is")
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "tests"))

    from kiln.api import Options, build_passes
    from kiln.frontend.fx_import import import_exported
    from kiln.gpu.codegen import generate as reference_generate
    from kiln.ir import interpret
    from kiln.passes.manager import PassManager
    from models.transformer import Block
    from test_memory_plan import random_graph

    from kiln_b200 import workloads as W
    from kiln_b200.codegen import plan_of

    (HERE / "plans").mkdir(exist_ok=True)
    (HERE / "vectors").mkdir(exist_ok=True)
    summary = {}

    def optimise(graph, options):
        pm = PassManager(build_passes(replace(options, tiling=False)))
        pm.run(graph)
        return pm

    def record(case, graph, pm):
        plan = plan_of(graph)
        plan.name = case
        # the benchmark configurations' plans ship with the package (the benchmark runs them where the
        # reference is not installed); every other plan is a test fixture
        plan_dir = W.PLAN_DIR if W.is_benchmark_case(case) else HERE / "plans"
        (plan_dir / f"{case}.json").write_text(plan.dumps() + "\n")
        program = reference_generate(graph)
        stats = pm.stats.get("memory-plan", {})
        summary[case] = {
            "kernels": [f"{k.name} {k.kind} {' '.join(n.op for n in k.nodes)}" for k in graph.kernels],
            "arena_bytes": graph.attrs.get("arena_bytes", 0),
            "naive_bytes": stats.get("naive_bytes", 0),
            "lower_bound_bytes": stats.get("lower_bound_bytes", 0),
            "launches": [[l.name, l.kind, list(l.grid), [list(b) for b in l.bases]] for l in program.launches],
        }
        return plan

    def export(fn, xs):
        module = fn if isinstance(fn, torch.nn.Module) else FnModule(fn)
        module.eval()
        with torch.no_grad():
            ep = torch.export.export(module, tuple(xs)).run_decompositions()
            expected = module(*xs)
        expected = list(expected) if isinstance(expected, (tuple, list)) else [expected]
        return import_exported(ep), expected, module

    def wanted(case):
        return args.only is None or args.only == case

    def small_case(name, fn, xs, **flags):
        case = slug(name)
        if not wanted(case):
            return
        torch.manual_seed(0)
        graph, expected, module = export(fn, xs)
        options = Options(device="cuda", **flags)
        pm = optimise(graph, options)
        plan = record(case, graph, pm)
        live = dict(module.named_parameters()) | dict(module.named_buffers())
        it = iter(xs)
        inputs = []
        for a, attrs in zip(graph.args, graph.arg_attrs):
            inputs.append(live[attrs["param"]].detach().numpy() if "param" in attrs else next(it).numpy())
        user = [x.numpy() for x in xs]
        interp = interpret(graph, *user)
        data = {f"in{i}": np.ascontiguousarray(x, np.float32) for i, x in enumerate(inputs)}
        data.update({f"const:{n}": graph.constants[n] for n in plan.const_shapes})
        data.update({f"out{i}": e.detach().numpy() for i, e in enumerate(expected)})
        data.update({f"interp{i}": e for i, e in enumerate(interp)})
        np.savez_compressed(HERE / "vectors" / f"{case}.npz", **data)

    # ---- the reference's own GPU test cases (tests/test_gpu.py:47-66, 79-122, 143-169) ----
    torch.manual_seed(0)
    Wm = torch.randn(37, 70)
    Y = torch.randn(3, 1)
    MASK = torch.full((2, 5000), float("-inf")).triu(1)
    cases = {
        "mlp": (torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(approximate="tanh"),
                                    torch.nn.Linear(40, 8)), (torch.randn(5, 24),)),
        "layernorm": (torch.nn.LayerNorm(48), (torch.randn(7, 48),)),
        "softmax": (lambda x: F.softmax(x, -1), (torch.randn(3, 5, 33),)),
        "column sum": (lambda x: x.sum(0, keepdim=True) * x, (torch.randn(6, 10),)),
        "full reduction": (lambda x: x.sum((0, 1), keepdim=True) * 2.0, (torch.randn(3, 4),)),
        "reduce dims 0 2": (lambda x: x.sum((0, 2), keepdim=True) + x.amax(0, keepdim=True),
                            (torch.randn(4, 5, 6),)),
        "views": (lambda x: (x.view(4, 3, 5).transpose(0, 1) * 2.0, x.t()), (torch.randn(12, 5),)),
        "bmm transposed operand": (lambda a, b: torch.bmm(a, b.transpose(1, 2)),
                                   (torch.randn(3, 9, 20), torch.randn(3, 17, 20))),
        "decode m1": (lambda a: F.gelu(a @ Wm, approximate="tanh"), (torch.randn(1, 37),)),
        "odd k": (lambda a, b: a @ b + 1.0, (torch.randn(33, 45), torch.randn(45, 19))),
        "per row scalar input": (lambda x: x / (x.sum(-1, keepdim=True) ** 2 + 1.0) + Y, (torch.randn(3, 50),)),
        "multi shape outputs": (lambda x: (x.exp() * 2, (x.exp() + Y[:2]).sum(-1, keepdim=True)),
                                (torch.randn(2, 9),)),
        "unary ops": (lambda x: torch.tanh(x) + torch.sigmoid(x) + torch.erf(x) + F.gelu(x) + torch.relu(-x),
                      (torch.randn(4, 30) * 3,)),
        "transformer block": (Block(d=32, nh=2, T=8), (torch.randn(8, 32),)),
        "long layernorm": (torch.nn.LayerNorm(10000), (torch.randn(2, 10000),)),
        "long softmax": (lambda x: F.softmax(x, -1), (torch.randn(2, 5000),)),
        "long masked softmax": (lambda x: F.softmax(x + MASK, -1), (torch.randn(2, 5000),)),
        "sliced views": (lambda x: x.view(4, 3, 5).transpose(0, 1)[:, 1:3, :] * 2.0, (torch.randn(12, 5),)),
        "tf32 linear": (torch.nn.Linear(64, 32), (torch.randn(16, 64),)),
        "autotune mlp": (torch.nn.Sequential(torch.nn.Linear(48, 64), torch.nn.GELU(approximate="tanh")),
                         (torch.randn(20, 48),)),
        "block d64": (Block(d=64, nh=4, T=16), (torch.randn(16, 64),)),
        "erf gelu mlp": (torch.nn.Sequential(torch.nn.Linear(40, 72), torch.nn.GELU(), torch.nn.Linear(72, 24)),
                         (torch.randn(130, 40),)),
        "wide bmm": (lambda a, b: torch.bmm(a, b) * 0.5, (torch.randn(3, 70, 130), torch.randn(3, 130, 96))),
        # a whole batch of sequences as ONE graph: Linear flattens the leading dims, attention runs on
        # [batch, heads, tokens, head_dim] views (the "batched models" row of the scope)
        "batched block": (W.batched_block_module(7, 16, d=64, heads=4), (torch.randn(3, 16, 64),)),
    }
    for name, (fn, xs) in cases.items():
        small_case(name, fn, xs)
    small_case("transformer block unfused", Block(d=32, nh=2, T=8), (torch.randn(8, 32),),
               fusion=False, memory_plan=False)
    small_case("unfrozen linear", torch.nn.Linear(16, 8), (torch.randn(4, 16),), freeze=False)

    # ---- random graphs (tests/test_gpu.py:125-134, generator tests/test_memory_plan.py:114-137) ----
    for seed in range(6):
        for fusion in (False, True):
            case = f"random_s{seed}_{'fused' if fusion else 'unfused'}"
            if not wanted(case):
                continue
            rng = random.Random(seed)
            g = random_graph(rng, n_ops=rng.randint(6, 22))
            x = np.random.default_rng(seed).standard_normal(g.args[0].shape).astype(np.float32) * 0.5
            expected = interpret(g, x)
            pm = optimise(g, Options(fusion=fusion, device="cuda"))
            record(case, g, pm)
            data = {"in0": x}
            data.update({f"out{i}": e for i, e in enumerate(expected)})
            data.update({f"interp{i}": e for i, e in enumerate(expected)})
            np.savez_compressed(HERE / "vectors" / f"{case}.npz", **data)

    # ---- the benchmark configurations: plans + subsampled float64 results ----
    def big_case(case, module, x, step):
        if not wanted(case):
            return
        graph, _, _ = export(module, (torch.from_numpy(x),))
        pm = optimise(graph, Options(device="cuda"))
        record(case, graph, pm)
        with torch.no_grad():
            out = module.double()(torch.from_numpy(x).double())
        out2d = out.reshape(-1, out.shape[-1]).numpy()
        np.savez_compressed(HERE / "vectors" / f"{case}.npz", sub0=out2d[::step].astype(np.float32),
                            step0=np.int64(step))

    for t, step in ((128, 8), (512, 32), (1024, 64), (2048, 128)):
        params = W.block_params(0 if t == 128 else 4, t)
        model = Block(768, 12, t).eval()
        model.load_state_dict({k: torch.from_numpy(v) for k, v in params.items()})
        big_case(f"gpt2_block_t{t}", model, W.block_input(0 if t == 128 else 4, t), step)

    # the benchmark's step: eight 1024-token sequences as one [8, 1024, 768] graph
    _, xb = W.case_tensors("gpt2_block_b8_t1024")
    big_case("gpt2_block_b8_t1024", W.batched_block_module(4, 1024), xb, 512)

    mp = W.mlp_params()
    mlp = torch.nn.Sequential(torch.nn.Linear(768, 3072), torch.nn.GELU(approximate="tanh"),
                              torch.nn.Linear(3072, 768)).eval()
    mlp.load_state_dict({k: torch.from_numpy(v) for k, v in mp.items()})
    big_case("mlp_2048", mlp, W.mlp_input(), 64)

    for m, n, k in W.LINEAR_SHAPES:
        p, a = W.linear_params(m, n, k)
        lin = torch.nn.Linear(k, n).eval()
        lin.load_state_dict({k_: torch.from_numpy(v) for k_, v in p.items()})
        big_case(f"linear_{m}x{n}x{k}", lin, a, max(1, m // 16))

    p, x = W.bias_gelu_data()
    bias = torch.from_numpy(p["bias"])

    class BiasGelu(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("bias", bias)

        def forward(self, t):
            return F.gelu(t + self.bias, approximate="tanh")

    big_case("bias_gelu_2048x3072", BiasGelu().eval(), x, 128)
    p, x = W.layernorm_data()
    ln = torch.nn.LayerNorm(768, eps=1e-5).eval()
    ln.load_state_dict({k_: torch.from_numpy(v) for k_, v in p.items()})
    big_case("layernorm_2048x768", ln, x, 64)
    _, x = W.softmax_data()
    big_case("softmax_12x512x512", FnModule(lambda t: F.softmax(t, -1)).eval(), x, 192)

    if args.only is not None:
        summary = {**json.loads((HERE / "reference_plans.json").read_text()), **summary}
    (HERE / "reference_plans.json").write_text(json.dumps(summary, indent=1, sort_keys=True) + "\n")
    print(f"wrote {len(summary)} cases")


if __name__ == "__main__":
    main()
