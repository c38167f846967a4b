"""Seeded synthetic workloads: the shapes, value distributions and seeds the benchmark is quoted on.

No dataset is involved anywhere on this path; every tensor is drawn from a
NumPy ``default_rng(seed)`` stream so that the machine that wrote the golden
fixtures and the machine that runs the GPU tests produce identical bytes.

Parameter names are the module paths the Kiln frontend gives constants
(``fc.weight``; ``fc.weight.transpose`` after constant folding stores the
weight as [K, N], kiln/passes/freeze.py:62-68).
"""

from __future__ import annotations

import numpy as np

GPT2_SMALL = {"d": 768, "heads": 12}


def _normal(rng, shape, std=1.0, mean=0.0):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def causal_mask(t):
    """[T, T] additive mask: 0 on and below the diagonal, -inf above."""
    m = np.zeros((t, t), dtype=np.float32)
    m[np.triu_indices(t, 1)] = -np.inf
    return m


def block_params(seed, t, d=768, heads=12, weight_std=0.02):
    """GPT-2 style pre-LN block: weights N(0, 0.02), biases 0, LayerNorm gamma 1 / beta 0."""
    del heads
    rng = np.random.default_rng(seed)
    p = {
        "ln1.weight": np.ones(d, np.float32), "ln1.bias": np.zeros(d, np.float32),
        "ln2.weight": np.ones(d, np.float32), "ln2.bias": np.zeros(d, np.float32),
        "c_attn.weight": _normal(rng, (3 * d, d), weight_std), "c_attn.bias": np.zeros(3 * d, np.float32),
        "c_proj.weight": _normal(rng, (d, d), weight_std), "c_proj.bias": np.zeros(d, np.float32),
        "fc.weight": _normal(rng, (4 * d, d), weight_std), "fc.bias": np.zeros(4 * d, np.float32),
        "proj.weight": _normal(rng, (d, 4 * d), weight_std), "proj.bias": np.zeros(d, np.float32),
        "mask": causal_mask(t),
    }
    return p


def block_input(seed, t, d=768, index=0):
    """Input sequence number ``index`` of the seeded stream: [T, d] ~ N(0, 1)."""
    rng = np.random.default_rng([seed, 1000 + index])
    return _normal(rng, (t, d))


def mlp_params(seed=1, d=768, hidden=3072):
    """Linear(d, hidden) -> tanh-GELU -> Linear(hidden, d); W ~ N(0, 0.02), b ~ U(-0.01, 0.01)."""
    rng = np.random.default_rng(seed)
    u = lambda n: rng.uniform(-0.01, 0.01, n).astype(np.float32)
    return {"0.weight": _normal(rng, (hidden, d), 0.02), "0.bias": u(hidden),
            "2.weight": _normal(rng, (d, hidden), 0.02), "2.bias": u(d)}


def mlp_input(seed=1, tokens=2048, d=768):
    return _normal(np.random.default_rng([seed, 1000]), (tokens, d))


LINEAR_SHAPES = [(2048, 3072, 768), (128, 2304, 768), (128, 768, 768), (128, 3072, 768), (128, 768, 3072),
                 (1, 3072, 768)]      # M x N x K


def linear_params(m, n, k, seed=2):
    """A, W ~ N(0, 1/sqrt(K)); bias ~ N(0, 0.01)."""
    rng = np.random.default_rng([seed, m, n, k])
    std = 1.0 / np.sqrt(k)
    return {"weight": _normal(rng, (n, k), std), "bias": _normal(rng, (n,), 0.01)}, _normal(rng, (m, k), std)


def bias_gelu_data(seed=3, rows=2048, cols=3072):
    rng = np.random.default_rng([seed, 0])
    return {"bias": _normal(rng, (cols,), 0.1)}, _normal(rng, (rows, cols))


def layernorm_data(seed=3, rows=2048, d=768):
    rng = np.random.default_rng([seed, 1])
    return {"weight": _normal(rng, (d,), 0.1, 1.0), "bias": _normal(rng, (d,), 0.1)}, _normal(rng, (rows, d))


def softmax_data(seed=3, shape=(12, 512, 512)):
    return {}, _normal(np.random.default_rng([seed, 2]), shape, 3.0)


def plan_constants(const_shapes, params):
    """Constant arrays for a plan from module-style parameters.

    ``name.transpose`` is the folded [K, N] copy of ``name`` (constant folding
    evaluates the transpose at compile time, kiln/passes/freeze.py:57-71).
    """
    out = {}
    for name, shape in const_shapes.items():
        if name in params:
            arr = params[name]
        elif name.endswith(".transpose") and name[:-len(".transpose")] in params:
            arr = np.ascontiguousarray(params[name[:-len(".transpose")]].T)
        else:
            raise KeyError(f"no data for constant {name!r}")
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        if tuple(arr.shape) != tuple(shape):
            raise ValueError(f"constant {name!r}: expected {tuple(shape)}, got {arr.shape}")
        out[name] = arr
    return out


def block_flops(t, d=768, heads=12):
    """Algorithmic FLOPs of one block call as the reference computes it (full T x T attention)."""
    del heads
    return 2 * t * d * (3 * d) + 2 * t * d * d + 2 * 2 * t * d * (4 * d) + 2 * 2 * t * t * d


def block_module(seed, t, d=768, heads=12):
    """The same block as a ``torch.nn.Module`` holding ``block_params(seed, t)``: what a user hands to
    ``kiln.compile``.  Written with the operations the Kiln frontend imports (Linear, LayerNorm,
    view / transpose / split, matmul, softmax, tanh-GELU; architecture of the reference's test model,
    tests/models/transformer.py:5-29) and with its parameter names, so that the compiled plan is the
    11-kernel plan stored under tests/golden/plans."""
    import math

    import torch
    from torch import nn
    from torch.nn import functional as F

    class PreLNBlock(nn.Module):
        def __init__(self):
            super().__init__()
            self.heads = heads
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.c_attn, self.c_proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.fc, self.proj = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
            self.register_buffer("mask", torch.zeros(t, t))

        def attention(self, h):
            tokens, width = h.shape
            hd = width // self.heads
            q, k, v = (z.view(tokens, self.heads, hd).transpose(0, 1) for z in self.c_attn(h).split(width, dim=1))
            scores = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(hd)) + self.mask[:tokens, :tokens]
            merged = (F.softmax(scores, dim=-1) @ v).transpose(0, 1).contiguous().view(tokens, width)
            return self.c_proj(merged)

        def forward(self, x):
            x = x + self.attention(self.ln1(x))
            return x + self.proj(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))

    model = PreLNBlock().eval()
    state = {k: torch.from_numpy(v.copy()) for k, v in block_params(seed, t, d, heads).items()}
    model.load_state_dict(state)
    return model


def batched_block_module(seed, t, d=768, heads=12):
    """The block of ``block_module`` taking ``[batch, tokens, d]``: every sequence of the batch in ONE
    compiled graph.  The frontend flattens the leading dims of every Linear (kiln/frontend/
    fx_import.py:150-153), so the projections become ``batch * tokens``-row matmuls; attention stays
    per sequence and head through ``[batch, heads, tokens, head_dim]`` views."""
    import math

    import torch
    from torch import nn
    from torch.nn import functional as F

    class BatchedPreLNBlock(nn.Module):
        def __init__(self):
            super().__init__()
            self.heads = heads
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.c_attn, self.c_proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.fc, self.proj = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
            self.register_buffer("mask", torch.zeros(t, t))

        def attention(self, h):
            batch, tokens, width = h.shape
            hd = width // self.heads
            q, k, v = (z.view(batch, tokens, self.heads, hd).transpose(1, 2) for z in self.c_attn(h).split(width, dim=2))
            scores = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(hd)) + self.mask[:tokens, :tokens]
            merged = (F.softmax(scores, dim=-1) @ v).transpose(1, 2).contiguous().view(batch, tokens, width)
            return self.c_proj(merged)

        def forward(self, x):
            x = x + self.attention(self.ln1(x))
            return x + self.proj(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))

    model = BatchedPreLNBlock().eval()
    model.load_state_dict({k: torch.from_numpy(v.copy()) for k, v in block_params(seed, t, d, heads).items()})
    return model


# ---------------------------------------------------------------------------------------------
# The benchmark configurations by name: tensors, modules, stored launch plans
# ---------------------------------------------------------------------------------------------

BENCHMARK_PREFIXES = ("gpt2_block_t", "gpt2_block_b", "mlp_2048", "linear_", "bias_gelu_", "layernorm_2048", "softmax_12x")
PLAN_DIR = __import__("pathlib").Path(__file__).resolve().parent / "plans"


def is_benchmark_case(case):
    return case.startswith(BENCHMARK_PREFIXES)


def benchmark_cases():
    return sorted(p.stem for p in PLAN_DIR.glob("*.json"))


def stored_plan(case):
    """The launch plan of a benchmark configuration as the reference's passes produce it (written by
    tests/golden/make_golden.py from the imported reference; a test compares it with a live compile
    where the reference is importable).  Lets the backend run a configuration on a machine that has
    no copy of the reference's frontend."""
    import json

    return json.loads((PLAN_DIR / f"{case}.json").read_text())


def batched_case(case):
    """(batch, tokens) of a ``gpt2_block_b<batch>_t<tokens>`` case name, or None."""
    import re

    m = re.fullmatch(r"gpt2_block_b(\d+)_t(\d+)", case)
    return (int(m.group(1)), int(m.group(2))) if m else None


def case_tensors(case):
    """(parameters by module path, input array) of a benchmark configuration."""
    if batched_case(case):
        batch, t = batched_case(case)
        return block_params(4, t), np.stack([block_input(4, t, index=i) for i in range(batch)])
    if case.startswith("gpt2_block_t"):
        t = int(case[len("gpt2_block_t"):])
        seed = 0 if t == 128 else 4
        return block_params(seed, t), block_input(seed, t)
    if case == "mlp_2048":
        return mlp_params(), mlp_input()
    if case.startswith("linear_"):
        m, n, k = (int(v) for v in case[len("linear_"):].split("x"))
        return linear_params(m, n, k)
    if case.startswith("bias_gelu"):
        return bias_gelu_data()
    if case.startswith("layernorm_2048"):
        return layernorm_data()
    if case.startswith("softmax_12x"):
        return softmax_data()
    raise KeyError(case)


def case_module(case):
    """(torch.nn.Module, input tensor) of a benchmark configuration: what a user hands to
    ``kiln.compile``.  Parameter names match ``case_tensors`` and the stored plans' constants."""
    import torch
    from torch import nn
    from torch.nn import functional as F

    params, x = case_tensors(case)
    state = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in params.items()}
    if batched_case(case):
        return batched_block_module(4, batched_case(case)[1]), torch.from_numpy(x)
    if case.startswith("gpt2_block_t"):
        t = int(case[len("gpt2_block_t"):])
        return block_module(0 if t == 128 else 4, t), torch.from_numpy(x)
    if case == "mlp_2048":
        module = nn.Sequential(nn.Linear(768, 3072), nn.GELU(approximate="tanh"), nn.Linear(3072, 768))
    elif case.startswith("linear_"):
        module = nn.Linear(x.shape[1], params["weight"].shape[0])
    elif case.startswith("bias_gelu"):
        class BiasGelu(nn.Module):
            def __init__(self):
                super().__init__()
                self.register_buffer("bias", torch.zeros(x.shape[1]))

            def forward(self, t):
                return F.gelu(t + self.bias, approximate="tanh")

        module = BiasGelu()
    elif case.startswith("layernorm_2048"):
        module = nn.LayerNorm(x.shape[1], eps=1e-5)
    else:
        class Softmax(nn.Module):
            def forward(self, t):
                return F.softmax(t, -1)

        module = Softmax()
    module.load_state_dict(state)
    return module.eval(), torch.from_numpy(x)
