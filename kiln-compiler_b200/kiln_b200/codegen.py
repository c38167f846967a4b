"""Turn an optimised Kiln graph into a launch plan (stands in for kiln.gpu.codegen).

The reference writes one Triton kernel per Kiln kernel, with every shape,
stride and arena offset as a literal in the source (kiln/gpu/codegen.py:8-12,
601-614).  Here ``generate`` collects exactly the same facts into a
``PlanSpec`` instead of source text; hand-written sm_100a kernels behind the C
ABI then run it.  The graph itself (fusion groups, layouts, arena offsets) is
the reference's and is only read, never changed.

Public names match the reference module: ``generate``, ``default_matmul_config``,
``Launch``, ``Program``, ``next_pow2``, ``sm_count``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

from kiln_b200.spec import ELEMENTWISE_OPS, REDUCTION_OPS, KernelSpec, NodeSpec, OperandSpec, PlanSpec

PRECISIONS = ("fp32", "tf32", "bf16")
GRID_LIMIT = 65535


def next_pow2(n):
    p = 1
    while p < n:
        p *= 2
    return p


def resolve_precision(allow_tf32: bool) -> str:
    """FP32 / TF32 follow ``allow_tf32`` as in the reference (codegen.py:515-516).

    The Kiln IR has no bf16 type (kiln/ir/core.py:41-43), so BF16 operands are
    a backend-internal mode selected with KILN_GPU_PRECISION=bf16; the arena
    plan stays the float32 one.
    """
    env = os.environ.get("KILN_GPU_PRECISION", "").strip().lower()
    if env:
        if env not in PRECISIONS:
            raise ValueError(f"KILN_GPU_PRECISION must be one of {PRECISIONS}, got {env!r}")
        return env
    return "tf32" if allow_tf32 else "fp32"


@dataclass
class Launch:
    """One device launch of the plan (same role as codegen.py:106-116)."""

    name: str
    kind: str                   # elementwise | row | reduction | matmul
    kernel: str                 # the Kiln kernel it comes from
    bases: list                 # ("input", i) | ("output", i) | ("const", name) | ("arena",)
    kernel_index: int = 0       # position in plan.kernels
    output_index: int | None = None   # elementwise: which kernel output this launch writes
    config: dict = field(default_factory=dict)
    grid: tuple = ()


@dataclass
class Program:
    """``source`` is a readable dump of the plan (the reference prints its
    Triton source at the same place, kiln/api.py:167-168)."""

    source: str
    launches: list = field(default_factory=list)
    plan: PlanSpec | None = None
    precision: str = "fp32"


def sm_count():
    """SMs of the current CUDA device; 148 (a B200) when there is none to ask."""
    import torch

    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return 148


def _matmul_dims(kernel):
    mm = next(n for n in kernel.nodes if n.op == "matmul")
    a, b = mm.inputs
    batch = 1
    for d in a.shape[:-2]:
        batch *= d
    return batch, a.shape[-2], b.shape[-1], a.shape[-1]


def default_matmul_config(graph, kernel):
    """The configuration used without measuring (role of codegen.py:563-598).

    All zeros: the library then applies its own rule when buffers are bound -- with more than 128
    rows, 256-row tiles on SM pairs (256 or 128 columns by a cost model of rounds, issue and
    tensor time); otherwise the widest 128-row tile that still gives every SM a tile, and, when
    even that leaves SMs idle (128-token projections, 768-wide layers), a split of K so that every
    SM streams a share of the operands.  The autotuner searches around this default.
    """
    del graph, kernel
    return {"BM": 0, "BN": 0, "BK": 0, "stages": 0, "split_k": 0, "impl": "auto"}


def _operand(layout, graph):
    base = layout.base
    if base[0] == "arena":
        byte_offset = base[1].node.attrs.get("offset", 0)
        if byte_offset % 4:
            raise NotImplementedError("GPU backend: arena offset is not a multiple of 4 bytes")
        return OperandSpec(("arena",), byte_offset // 4 + layout.offset, tuple(layout.shape), tuple(layout.strides))
    return OperandSpec(tuple(base), layout.offset, tuple(layout.shape), tuple(layout.strides))


def kernel_spec(graph, kernel, layouts) -> KernelSpec:
    from kiln.passes.buffers import kernel_inputs, kernel_outputs

    inputs = kernel_inputs(graph, kernel)
    outputs = kernel_outputs(graph, kernel)
    index_of = {n: i for i, n in enumerate(kernel.nodes)}
    nodes = []
    for n in kernel.nodes:
        refs = []
        for v in n.inputs:
            if v.node is not None and v.node in index_of:
                refs.append(("node", index_of[v.node]))
            elif graph.is_scalar_const(v):
                refs.append(("scalar", float(graph.const_data(v))))
            else:
                refs.append(("operand", inputs.index(v)))
        attrs = {}
        if n.op in REDUCTION_OPS:
            attrs["dims"] = [int(d) for d in n.attrs["dims"]]
        if n.op == "gelu":
            attrs["approximate"] = n.attrs.get("approximate", "none")
        nodes.append(NodeSpec(n.op, refs, tuple(n.out.shape), attrs))
    return KernelSpec(kernel.name, kernel.kind, nodes, [_operand(layouts[v], graph) for v in inputs],
                      [(index_of[v.node], _operand(layouts[v], graph)) for v in outputs])


def plan_of(graph) -> PlanSpec:
    """The plan of a graph that has been through fusion, buffer assignment and memory planning."""
    from kiln.ir import ops
    from kiln.passes.buffers import compute_layouts

    layouts = compute_layouts(graph)
    for k in graph.kernels:
        for n in k.nodes:
            if ops.kind(n.op) not in ("elementwise", "reduction", "matmul"):
                raise NotImplementedError(f"GPU backend: unexpected op '{n.op}' in a kernel")
    kernels = [kernel_spec(graph, k, layouts) for k in graph.kernels]
    used = {}
    for k in kernels:
        for o in k.inputs:
            if o.base[0] == "const":
                used[o.base[1]] = tuple(graph.constants[o.base[1]].shape)
    return PlanSpec(graph.name, [tuple(a.shape) for a in graph.args], [tuple(r.shape) for r in graph.results],
                    int(graph.attrs.get("arena_bytes", 0)), used, kernels)


def launch_kind(k: KernelSpec) -> str:
    """Which of the four kernel classes runs a Kiln kernel (codegen.py:532-542)."""
    if k.kind == "matmul":
        return "matmul"
    if k.kind == "reduction":
        reds = [n for n in k.nodes if n.op in REDUCTION_OPS]
        from kiln_b200.spec import input_shape_of, is_row_reduction

        if all(is_row_reduction(n, input_shape_of(k, n)) for n in reds):
            return "row"
        if len(k.nodes) != 1:
            raise NotImplementedError("GPU backend: a non-row reduction fused with other ops")
        return "reduction"
    return "elementwise"


def _bases(k: KernelSpec, outputs):
    keys = []
    for o in list(k.inputs) + [o for _, o in outputs]:
        if o.base not in keys:
            keys.append(o.base)
    return keys


def launches_of(plan: PlanSpec, configs=None):
    """One Launch per device kernel class instance.  An elementwise Kiln kernel
    gets one launch per output, as in the reference (codegen.py:541-542)."""
    configs = configs or {}
    out = []
    for ki, k in enumerate(plan.kernels):
        for n in k.nodes:
            if n.op not in ELEMENTWISE_OPS and n.op not in REDUCTION_OPS and n.op != "matmul":
                raise NotImplementedError(f"GPU backend: no lowering for '{n.op}'")
        kind = launch_kind(k)
        if kind == "elementwise":
            for oi in range(len(k.outputs)):
                out.append(Launch(f"{k.name}_ew{oi}", kind, k.name, _bases(k, k.outputs), ki, oi))
        else:
            suffix = {"row": "row", "reduction": "reduce", "matmul": "matmul"}[kind]
            launch = Launch(f"{k.name}_{suffix}", kind, k.name, _bases(k, k.outputs), ki, None,
                            dict(configs.get(k.name, {})))
            if kind == "matmul":
                mm = next(n for n in k.nodes if n.op == "matmul")
                batch = 1
                for d in mm.shape[:-2]:
                    batch *= d
                if batch > GRID_LIMIT:
                    raise NotImplementedError(f"GPU backend: matmul batch {batch} exceeds CUDA grid limits")
            out.append(launch)
    return out


def describe(plan: PlanSpec, launches, precision) -> str:
    """Readable text for Program.source / dump_mlir."""
    lines = [f"# kiln-b200 launch plan for graph '{plan.name}': {len(plan.kernels)} kernels, "
             f"{len(launches)} launches, arena {plan.arena_bytes} bytes, matmul precision {precision}"]
    for l in launches:
        k = plan.kernels[l.kernel_index]
        lines.append(f"launch {l.name} [{l.kind}] ops: {' '.join(k.ops)}")
        for j, o in enumerate(k.inputs):
            lines.append(f"  in{j}  {list(o.shape)} @ {'/'.join(map(str, o.base))} + {o.offset} strides {list(o.strides)}")
        outs = k.outputs if l.output_index is None else [k.outputs[l.output_index]]
        for i, o in outs:
            lines.append(f"  out  node{i} {list(o.shape)} @ {'/'.join(map(str, o.base))} + {o.offset} "
                         f"strides {list(o.strides)}")
        if l.config:
            lines.append(f"  config {l.config}")
    lines.append("# plan json")
    lines.append(plan.dumps())
    return "\n".join(lines) + "\n"


def generate(graph, allow_tf32=False, matmul_config=default_matmul_config) -> Program:
    """Same signature and error behaviour as kiln.gpu.codegen.generate (codegen.py:601-614):
    raises NotImplementedError for graphs the backend cannot run, never mutates ``graph``."""
    plan = plan_of(graph)
    configs = {}
    for k, spec in zip(graph.kernels, plan.kernels):
        if spec.kind == "matmul":
            configs[spec.name] = dict(matmul_config(graph, k))
    precision = resolve_precision(allow_tf32)
    launches = launches_of(plan, configs)
    return Program(describe(plan, launches, precision), launches, plan, precision)


def program_from_plan(plan: PlanSpec, precision="fp32", configs=None) -> Program:
    """A Program from a stored plan, for running without the Kiln frontend."""
    if precision not in PRECISIONS:
        raise ValueError(f"precision must be one of {PRECISIONS}")
    launches = launches_of(plan, configs)
    return Program(describe(plan, launches, precision), launches, plan, precision)
