"""Lower a PlanSpec to the POD descriptors of the C ABI (include/kb200.h).

Purely mechanical: align every tensor's strides to the kernel's iteration
space (broadcast dims get stride 0, as the reference skips them when it
writes an address, kiln/gpu/codegen.py:212-216), merge iteration dims that
are contiguous for every tensor, and flatten the scalar-op DAG into a tape.
Which hand-written kernel runs a descriptor is decided inside the library.
"""

from __future__ import annotations

import os

from kiln_b200 import _cabi
from kiln_b200.codegen import Launch
from kiln_b200.spec import REDUCTION_OPS, KernelSpec, OperandSpec, PlanSpec, input_shape_of

IMPL_CODES = {"auto": 0, "simt": 1, "tc": 2, "gemv": 3}


def align_strides(op: OperandSpec, iter_shape):
    """Strides of ``op`` right-aligned to ``iter_shape``; 0 where it broadcasts."""
    rank = len(iter_shape)
    if len(op.shape) > rank:
        lead = len(op.shape) - rank
        if any(s != 1 for s in op.shape[:lead]):
            raise NotImplementedError(f"GPU backend: operand {op.shape} does not broadcast to {tuple(iter_shape)}")
        shape, strides = op.shape[lead:], op.strides[lead:]
    else:
        shape, strides = op.shape, op.strides
    out = [0] * rank
    for i, (size, stride) in enumerate(zip(shape, strides)):
        j = rank - len(shape) + i
        if size == 1 or stride == 0:
            continue
        if size != iter_shape[j]:
            raise NotImplementedError(f"GPU backend: operand {op.shape} does not broadcast to {tuple(iter_shape)}")
        out[j] = stride
    return out


def collapse(shape, stride_lists, segments=None):
    """Drop size-1 dims and merge neighbours that are contiguous in every tensor.

    ``segments`` (list of dim counts summing to the rank) marks groups that must
    not be merged with each other, e.g. row dims | inner.  Returns the new shape,
    the new stride lists and the new segment sizes.
    """
    segments = segments or [len(shape)]
    new_shape, new_strides, new_segments = [], [[] for _ in stride_lists], []
    d = 0
    for seg in segments:
        count = 0
        for _ in range(seg):
            size = shape[d]
            if size != 1:
                if count and all(sl[-1] == st[d] * size for sl, st in zip(new_strides, stride_lists)):
                    new_shape[-1] *= size
                    for sl, st in zip(new_strides, stride_lists):
                        sl[-1] = st[d]
                else:
                    new_shape.append(size)
                    for sl, st in zip(new_strides, stride_lists):
                        sl.append(st[d])
                    count += 1
            d += 1
        new_segments.append(count)
    return new_shape, new_strides, new_segments


class _Tape:
    def __init__(self):
        self.entries = []      # [opcode, a, b, level, imm]
        self.node_value = {}
        self.loads = {}
        self.imms = {}

    def emit(self, opcode, a=0, b=0, level=0, imm=0.0):
        self.entries.append([_cabi.OPCODES[opcode], a, b, level, float(imm)])
        return len(self.entries) - 1

    def level(self, i):
        return self.entries[i][3]


def _opcode_of(node):
    if node.op == "gelu":
        return "gelu_tanh" if node.attrs.get("approximate", "none") == "tanh" else "gelu_erf"
    return node.op


def build_tape(kernel: KernelSpec, wanted, slot_of_input, slot_of_output):
    """Flatten the nodes needed for the ``wanted`` outputs (indices into kernel.outputs)."""
    needed, stack = set(), [kernel.outputs[oi][0] for oi in wanted]
    while stack:
        i = stack.pop()
        if i in needed:
            continue
        needed.add(i)
        stack.extend(ref[1] for ref in kernel.nodes[i].inputs if ref[0] == "node")
    tape = _Tape()

    def value(ref):
        if ref[0] == "node":
            return tape.node_value[ref[1]]
        if ref[0] == "scalar":
            key = float(ref[1])
            if key not in tape.imms:
                tape.imms[key] = tape.emit("IMM", imm=key)
            return tape.imms[key]
        j = ref[1]
        if j not in tape.loads:
            tape.loads[j] = tape.emit("LOAD", a=slot_of_input(j))
        return tape.loads[j]

    for i, node in enumerate(kernel.nodes):
        if i not in needed:
            continue
        if node.op == "matmul":
            tape.node_value[i] = tape.emit("ACC")
            continue
        args = [value(ref) for ref in node.inputs]
        lvl = max(tape.level(a) for a in args)
        if node.op in REDUCTION_OPS:
            tape.node_value[i] = tape.emit(node.op, a=args[0], level=lvl + 1)
        else:
            tape.node_value[i] = tape.emit(_opcode_of(node), a=args[0], b=args[1] if len(args) > 1 else 0, level=lvl)
    for oi in wanted:
        v = tape.node_value[kernel.outputs[oi][0]]
        tape.emit("STORE", a=v, b=slot_of_output(oi), level=tape.level(v))
    return tape.entries


def _fill(desc, kclass, precision, iter_shape, operands, tape, name, n_kept=0, k_extent=0, a_slot=-1, b_slot=-1,
          config=None):
    if len(iter_shape) > _cabi.MAX_RANK:
        raise NotImplementedError(f"GPU backend: {name} needs {len(iter_shape)} iteration dims (max {_cabi.MAX_RANK})")
    if len(operands) > _cabi.MAX_OPERANDS:
        raise NotImplementedError(f"GPU backend: {name} touches {len(operands)} tensors (max {_cabi.MAX_OPERANDS})")
    if len(tape) > _cabi.MAX_TAPE:
        raise NotImplementedError(f"GPU backend: {name} has {len(tape)} scalar ops (max {_cabi.MAX_TAPE})")
    desc.kclass, desc.precision = kclass, _cabi.PRECISIONS[precision]
    desc.iter_rank, desc.n_kept = len(iter_shape), n_kept
    for d, s in enumerate(iter_shape):
        desc.iter_shape[d] = s
    desc.k_extent, desc.a_slot, desc.b_slot = k_extent, a_slot, b_slot
    desc.n_operands, desc.n_tape = len(operands), len(tape)
    for slot, (op, strides) in enumerate(operands):
        o = desc.operands[slot]
        o.base_kind = _cabi.BASE_KINDS[op.base[0]]
        o.base_index = 0 if op.base[0] == "arena" else op.base[1]
        o.elem_offset = op.offset
        for d, st in enumerate(strides):
            o.stride[d] = st
    for i, (opcode, a, b, level, imm) in enumerate(tape):
        t = desc.tape[i]
        t.opcode, t.a, t.b, t.level, t.imm = opcode, a, b, level, imm
    config = config or {}
    cfg = [config.get("BM", 0), config.get("BN", 0), config.get("BK", 0), config.get("stages", 0),
           config.get("split_k", 0), IMPL_CODES.get(config.get("impl", "auto"), 0), config.get("debug", 0),
           {"auto": 0, "plain": 1, "bulk_columns": 2}[config.get("stores", "auto")]]
    if precision == "fp32" and os.environ.get("KILN_GPU_FP32_MATMUL", "").lower() == "ieee":
        cfg[6] = int(cfg[6]) | 1024     # CUDA-core FP32 matmul: IEEE results also for infinite operand elements
    for i, c in enumerate(cfg):
        desc.cfg[i] = int(c)
    desc.name = name.encode()[:31]
    return desc


def _lower_elementwise(kernel, launch, const_index, desc):
    node_i, out = kernel.outputs[launch.output_index]
    shape = list(out.shape) or [1]
    n_in = len(kernel.inputs)
    tape = build_tape(kernel, [launch.output_index], lambda j: j, lambda oi: n_in)
    ops = list(kernel.inputs) + [out]
    strides = [align_strides(o, shape) for o in ops]
    new_shape, new_strides, _ = collapse(shape, strides)
    if not new_shape:
        new_shape, new_strides = [1], [[0] for _ in ops]
    return _fill(desc, _cabi.K_ELEMENTWISE, "fp32", new_shape, list(zip(_rebase(ops, const_index), new_strides)),
                 tape, launch.name)


def _lower_row(kernel, launch, const_index, desc):
    red = next(n for n in kernel.nodes if n.op in REDUCTION_OPS)
    shape = list(input_shape_of(kernel, red))
    n_in = len(kernel.inputs)
    tape = build_tape(kernel, range(len(kernel.outputs)), lambda j: j, lambda oi: n_in + oi)
    ops = list(kernel.inputs) + [o for _, o in kernel.outputs]
    strides = [align_strides(o, shape) for o in ops]
    rows, row_strides, _ = collapse(shape[:-1], [s[:-1] for s in strides])
    if not rows:
        rows, row_strides = [1], [[0] for _ in ops]
    new_shape = rows + [shape[-1]]
    new_strides = [rs + [s[-1]] for rs, s in zip(row_strides, strides)]
    return _fill(desc, _cabi.K_ROW, "fp32", new_shape, list(zip(_rebase(ops, const_index), new_strides)), tape,
                 launch.name)


def _lower_reduce(kernel, launch, const_index, desc):
    (node,) = kernel.nodes
    x = kernel.inputs[0] if node.inputs[0][0] == "operand" else None
    if x is None:
        raise NotImplementedError("GPU backend: reduction of a scalar")
    (_, out), = kernel.outputs
    dims = {d % len(x.shape) for d in node.attrs["dims"]}
    kept = [d for d in range(len(x.shape)) if d not in dims and x.shape[d] != 1]
    red = [d for d in sorted(dims) if x.shape[d] != 1]
    out_strides_full = align_strides(out, [1 if d in dims else s for d, s in enumerate(x.shape)])
    shape = [x.shape[d] for d in kept + red]
    xs = [x.strides[d] for d in kept + red]
    os_ = [out_strides_full[d] for d in kept] + [0] * len(red)
    new_shape, (xs, os_), segs = collapse(shape, [xs, os_], [len(kept), len(red)])
    tape = build_tape(kernel, [0], lambda j: 0, lambda oi: 1)
    return _fill(desc, _cabi.K_REDUCE, "fp32", new_shape, list(zip(_rebase([x, out], const_index), [xs, os_])), tape,
                 launch.name, n_kept=segs[0])


def _lower_matmul(kernel, launch, const_index, desc, precision):
    mm_i = next(i for i, n in enumerate(kernel.nodes) if n.op == "matmul")
    mm = kernel.nodes[mm_i]
    if any(ref[0] != "operand" for ref in mm.inputs):
        raise NotImplementedError("GPU backend: matmul operand computed inside its own kernel")
    a, b = kernel.inputs[mm.inputs[0][1]], kernel.inputs[mm.inputs[1][1]]
    if len(a.shape) != len(b.shape) or len(a.shape) not in (2, 3):
        raise NotImplementedError(f"GPU backend: matmul of shapes {a.shape} x {b.shape}")
    batch = a.shape[0] if len(a.shape) == 3 else 1
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    iter_shape = [batch, m, n]

    def mm_strides(o):
        sb = o.strides[0] if len(o.shape) == 3 and o.shape[0] != 1 else 0
        return [sb, o.strides[-2] if o.shape[-2] != 1 else 0, o.strides[-1] if o.shape[-1] != 1 else 0]

    slots = [(a, mm_strides(a)), (b, mm_strides(b))]
    epi_slot = {}

    def slot_of_input(j):
        if j not in epi_slot:
            epi_slot[j] = len(slots)
            slots.append((kernel.inputs[j], align_strides(kernel.inputs[j], iter_shape)))
        return epi_slot[j]

    out_slot = {}

    def slot_of_output(oi):
        if oi not in out_slot:
            out_slot[oi] = len(slots)
            slots.append((kernel.outputs[oi][1], align_strides(kernel.outputs[oi][1], iter_shape)))
        return out_slot[oi]

    tape = build_tape(kernel, range(len(kernel.outputs)), slot_of_input, slot_of_output)
    ops = _rebase([o for o, _ in slots], const_index)
    return _fill(desc, _cabi.K_MATMUL, precision, iter_shape, list(zip(ops, [s for _, s in slots])), tape, launch.name,
                 k_extent=k, a_slot=0, b_slot=1, config=launch.config)


def _rebase(ops, const_index):
    """Constants are addressed by position in the bind call, not by name."""
    out = []
    for o in ops:
        if o.base[0] == "const":
            o = OperandSpec(("const", const_index[o.base[1]]), o.offset, o.shape, o.strides)
        out.append(o)
    return out


def lower(plan: PlanSpec, launches: list[Launch], precision: str, const_order: list[str]):
    """ctypes array of kb200_kernel_desc, one per launch, in launch order."""
    const_index = {name: i for i, name in enumerate(const_order)}
    descs = (_cabi.KernelDesc * max(len(launches), 1))()
    for i, launch in enumerate(launches):
        kernel = plan.kernels[launch.kernel_index]
        d = descs[i]
        if launch.kind == "elementwise":
            _lower_elementwise(kernel, launch, const_index, d)
        elif launch.kind == "row":
            _lower_row(kernel, launch, const_index, d)
        elif launch.kind == "reduction":
            _lower_reduce(kernel, launch, const_index, d)
        elif launch.kind == "matmul":
            _lower_matmul(kernel, launch, const_index, d, precision)
        else:
            raise NotImplementedError(f"GPU backend: launch kind {launch.kind!r}")
    return descs
