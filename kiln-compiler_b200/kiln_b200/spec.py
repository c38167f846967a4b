"""Launch-plan data model: what the GPU backend needs to know about one Kiln graph.

The reference's code generator walks the optimised graph and writes Triton
source in which every size, stride and arena offset is a literal
(kiln/gpu/codegen.py:8-12).  This backend keeps the same facts as data: one
``KernelSpec`` per Kiln kernel (fusion group) holding its scalar-op DAG, the
resolved layout of every tensor it touches, and which values it writes.  The
structures are plain Python and JSON-serialisable, so a plan can be stored,
diffed against a golden copy, evaluated on the CPU by the test oracle, and
lowered to the C ABI without the Kiln frontend being importable.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from math import prod

SCHEMA = 1

ELEMENTWISE_OPS = ("add", "sub", "mul", "div", "maximum", "minimum", "neg", "relu", "exp", "tanh",
                   "sigmoid", "erf", "gelu", "rsqrt", "sqrt", "copy")
REDUCTION_OPS = ("reduce_sum", "reduce_max")


@dataclass(frozen=True)
class OperandSpec:
    """A tensor in device memory: base buffer, element offset, shape, element strides.

    ``base`` is ("arena",), ("const", name), ("input", i) or ("output", i), the
    same keys as the reference's Launch.bases (kiln/gpu/codegen.py:106-116).
    ``offset`` counts float32 elements from the start of that buffer and, for
    the arena, already includes the planned byte offset divided by four
    (kiln/gpu/codegen.py:545-549).
    """

    base: tuple
    offset: int
    shape: tuple
    strides: tuple

    @property
    def numel(self):
        return prod(self.shape) if self.shape else 1

    @property
    def span(self):
        """Largest element index reached, relative to ``offset``."""
        return sum((s - 1) * st for s, st in zip(self.shape, self.strides) if s > 0)

    def to_json(self):
        return {"base": list(self.base), "offset": self.offset, "shape": list(self.shape),
                "strides": list(self.strides)}

    @classmethod
    def from_json(cls, d):
        return cls(tuple(d["base"]), int(d["offset"]), tuple(d["shape"]), tuple(d["strides"]))


@dataclass
class NodeSpec:
    """One scalar op of a kernel.  ``inputs`` entries are ("node", i) for the
    i-th node of the same kernel, ("operand", j) for the kernel's j-th input
    tensor, or ("scalar", x) for a float32 literal."""

    op: str
    inputs: list
    shape: tuple
    attrs: dict = field(default_factory=dict)

    def to_json(self):
        return {"op": self.op, "inputs": [list(i) for i in self.inputs], "shape": list(self.shape),
                "attrs": self.attrs}

    @classmethod
    def from_json(cls, d):
        return cls(d["op"], [tuple(i) for i in d["inputs"]], tuple(d["shape"]), dict(d.get("attrs", {})))


@dataclass
class KernelSpec:
    """One fusion group with every layout resolved.

    ``inputs``   tensors read from outside the kernel (scalars excluded), in
                 the order kiln.passes.buffers.kernel_inputs returns them;
    ``outputs``  (node index, where it is written) for every value needed
                 outside the kernel, in kernel_outputs order.
    """

    name: str
    kind: str                      # elementwise | reduction | matmul | copy
    nodes: list
    inputs: list
    outputs: list

    @property
    def ops(self):
        return [n.op for n in self.nodes]

    def to_json(self):
        return {"name": self.name, "kind": self.kind, "nodes": [n.to_json() for n in self.nodes],
                "inputs": [o.to_json() for o in self.inputs],
                "outputs": [[i, o.to_json()] for i, o in self.outputs]}

    @classmethod
    def from_json(cls, d):
        return cls(d["name"], d["kind"], [NodeSpec.from_json(n) for n in d["nodes"]],
                   [OperandSpec.from_json(o) for o in d["inputs"]],
                   [(int(i), OperandSpec.from_json(o)) for i, o in d["outputs"]])


@dataclass
class PlanSpec:
    """Everything static about one compiled graph."""

    name: str
    input_shapes: list
    output_shapes: list
    arena_bytes: int
    const_shapes: dict             # name -> shape, for every constant some kernel reads
    kernels: list

    def to_json(self):
        return {"schema": SCHEMA, "name": self.name, "input_shapes": [list(s) for s in self.input_shapes],
                "output_shapes": [list(s) for s in self.output_shapes], "arena_bytes": self.arena_bytes,
                "const_shapes": {k: list(v) for k, v in self.const_shapes.items()},
                "kernels": [k.to_json() for k in self.kernels]}

    def dumps(self):
        return json.dumps(self.to_json(), indent=1, sort_keys=True)

    @classmethod
    def from_json(cls, d):
        if d.get("schema") != SCHEMA:
            raise ValueError(f"plan schema {d.get('schema')!r} is not {SCHEMA}")
        return cls(d["name"], [tuple(s) for s in d["input_shapes"]], [tuple(s) for s in d["output_shapes"]],
                   int(d["arena_bytes"]), {k: tuple(v) for k, v in d["const_shapes"].items()},
                   [KernelSpec.from_json(k) for k in d["kernels"]])

    @classmethod
    def loads(cls, text):
        return cls.from_json(json.loads(text))


def is_row_reduction(node: NodeSpec, in_shape) -> bool:
    """A keepdim reduction over exactly the innermost dim (kiln/passes/fusion.py:54-57)."""
    rank = len(in_shape)
    return rank >= 1 and list(node.attrs["dims"]) == [rank - 1]


def input_shape_of(kernel: KernelSpec, node: NodeSpec, which=0):
    ref = node.inputs[which]
    if ref[0] == "node":
        return kernel.nodes[ref[1]].shape
    if ref[0] == "operand":
        return kernel.inputs[ref[1]].shape
    return ()
