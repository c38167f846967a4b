"""GPU matmul autotuning by measurement (stands in for kiln.gpu.autotune).

Contract shared with the reference's tuner (kiln/gpu/autotune.py:113-193), because
``kiln.api`` and the reference's tests rely on it: ``GPUAutotuner(allow_tf32).config_for(graph,
kernel)`` returns the configuration dict handed to ``generate``; every lookup appends an entry
to ``log`` (keys shape, source = "tuned" | "cache", config, default_config, tflops,
default_tflops, candidates, seconds); results persist in ``$KILN_CACHE_DIR/b200_autotune.json``
keyed by GPU name, precision and shape, written atomically, a damaged file being ignored; a
candidate counts only if its result matches a float64 product relative to the output's scale;
and the default configuration is kept unless something beats it by MIN_GAIN.

How a shape is tuned here: every candidate becomes a ``Trial`` (a compiled one-matmul plan on
shared operands) that first has to pass ``check`` and is then timed as GPU time only (many
launches in one CUDA graph); the fastest few and the default go through alternating timing
rounds so that clock drift hits all of them alike; ``Verdict`` turns the timings into the
cached entry.

What is searched is this backend's own space, not Triton's: which tensor-core kernel (256-row
tiles on SM pairs, BM = 256, or single-CTA 128-row tiles, BM = 128), the tile width BN, K
slabs per pipeline step (BK: 1 or 2, pair kernel), pipeline stages and the cluster split-K
factor of the single-CTA kernel; plus the CUDA-core FP32 kernel.
"""

from __future__ import annotations

import json
import os
import time
import warnings
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch

from kiln_b200.codegen import default_matmul_config, next_pow2, program_from_plan, resolve_precision
from kiln_b200.runtime import GPUExecutable, GraphTimer, device
from kiln_b200.spec import KernelSpec, NodeSpec, OperandSpec, PlanSpec

MIN_GAIN = 1.03
FINALISTS = 3
TIMING_ROUNDS = 3
SHARED_MEMORY_BYTES = 227 * 1024     # per CTA on B200
ERROR_BOUND = {"fp32": 1e-4, "tf32": 2e-2, "bf16": 5e-2}     # relative to the output's scale (autotune.py:147-151)

# single-CTA kernel: (BN, stages, split_k)
SINGLE_CTA_TILES = [(256, 4, 1), (256, 3, 1), (128, 4, 1), (128, 6, 1), (64, 6, 1), (128, 4, 2), (128, 4, 4), (64, 6, 2),
                    (64, 6, 4), (64, 6, 8), (256, 3, 2)]
# CTA-pair kernel (256 rows over a cluster of two SMs): (BN, K slabs per step)
PAIR_TILES = [(256, 1), (128, 1), (128, 2)]
SINGLE_CTA_EPILOGUE_BYTES = 8 * 7168     # transpose / staging buffers of its eight epilogue warps
TC_CANDIDATES = SINGLE_CTA_TILES          # older name


def cache_path() -> Path:
    return Path(os.environ.get("KILN_CACHE_DIR") or Path.home() / ".cache" / "kiln") / "b200_autotune.json"


def device_name():
    return torch.cuda.get_device_name(device())


def stage_bytes(cfg):
    """Shared memory of one pipeline stage: 128 A rows and the CTA's B rows, 128 bytes of K each
    (a CTA of a pair holds half the tile's columns), times the K slabs per step."""
    b_rows = cfg["BN"] // 2 if cfg["BM"] == 256 else cfg["BN"]
    return (128 + b_rows) * 128 * max(1, cfg.get("BK", 0))


def candidates(m, n, k):
    """Every configuration worth measuring for an m x n x k matmul on this backend."""
    widest = max(64, next_pow2(n))          # a tile much wider than the problem only adds masked-off work
    found = []
    if m > 128 and n >= 128:
        for bn, slabs in PAIR_TILES:
            if bn <= widest:
                found.append({"BM": 256, "BN": bn, "BK": slabs, "stages": 0, "split_k": 1, "impl": "tc"})
    for bn, stages, split in SINGLE_CTA_TILES:
        cfg = {"BM": 128, "BN": bn, "stages": stages, "split_k": split, "impl": "tc"}
        fits = stage_bytes(cfg) * stages + SINGLE_CTA_EPILOGUE_BYTES + 1024 <= SHARED_MEMORY_BYTES
        if bn <= widest and fits and (split == 1 or k // split >= 128):
            found.append(cfg)
    found.append({"BM": 64, "BN": 64, "stages": 1, "split_k": 1, "impl": "simt"})
    return found


def matmul_plan(batch, m, n, k, b_kmajor=False) -> PlanSpec:
    """A bare [batch,] M x K by K x N matmul reading two inputs and writing one output.
    With ``b_kmajor`` the second input is stored as [N, K] and read through a transposed view."""
    lead = (batch,) if batch > 1 else ()

    def contiguous(shape):
        strides, acc = [], 1
        for s in reversed(shape):
            strides.append(acc)
            acc *= s
        return tuple(reversed(strides))

    a_shape, b_shape, c_shape = (*lead, m, k), (*lead, k, n), (*lead, m, n)
    b_stored = (*lead, n, k) if b_kmajor else b_shape
    b_strides = contiguous(b_shape)
    if b_kmajor:
        st = contiguous(b_stored)
        b_strides = (*st[:-2], st[-1], st[-2])
    kernel = KernelSpec("k0", "matmul", [NodeSpec("matmul", [("operand", 0), ("operand", 1)], c_shape)],
                        [OperandSpec(("input", 0), 0, a_shape, contiguous(a_shape)),
                         OperandSpec(("input", 1), 0, b_shape, b_strides)],
                        [(0, OperandSpec(("output", 0), 0, c_shape, contiguous(c_shape)))])
    return PlanSpec("matmul", [a_shape, b_stored], [c_shape], 0, {}, [kernel])


def frozen(config):
    return tuple(sorted(config.items()))


class TuningCache:
    """The on-disk table of tuned shapes.  Reading never fails (a missing or damaged file is an
    empty table); writing goes through a scratch file and a rename, and a failure to write is a
    warning, not an error."""

    def __init__(self, enabled=True):
        self.enabled = enabled
        self.table = self._read() if enabled else {}

    @staticmethod
    def _read():
        try:
            table = json.loads(cache_path().read_text())
        except (OSError, ValueError):
            return {}
        return table if isinstance(table, dict) else {}

    def get(self, key):
        return self.table.get(key)

    def put(self, key, entry):
        self.table[key] = entry
        if not self.enabled:
            return
        target = cache_path()
        try:
            target.parent.mkdir(parents=True, exist_ok=True)
            scratch = target.with_name(f"{target.name}.{os.getpid()}.part")
            scratch.write_text(json.dumps(self.table, indent=1, sort_keys=True))
            os.replace(scratch, target)
        except OSError as err:
            warnings.warn(f"Kiln: couldn't write the GPU autotune cache ({err})")


@dataclass
class Operands:
    """Shared inputs of all trials of one shape, and the float64 product they are checked against."""

    a: torch.Tensor
    b: torch.Tensor
    expected: torch.Tensor
    scale: float

    @classmethod
    def make(cls, batch, m, n, k):
        gen = torch.Generator(device="cpu").manual_seed(0)
        lead = (batch,) if batch > 1 else ()
        dev = device()
        a = torch.randn(*lead, m, k, generator=gen).to(dev)
        b = (torch.randn(*lead, k, n, generator=gen) / k ** 0.5).to(dev)     # products of order one, as in a real layer
        expected = (a.double() @ b.double()).float()
        return cls(a, b, expected, expected.abs().max().item() or 1.0)


@dataclass
class Trial:
    """One candidate configuration: compiled, checked, timed."""

    config: dict
    exe: GPUExecutable | None = None
    why_not: str | None = None
    first_seconds: float = float("inf")
    best_seconds: float = float("inf")
    timer: GraphTimer | None = field(default=None, repr=False)

    @property
    def key(self):
        return frozen(self.config)

    def check(self, build, operands, bound):
        """Build and run once; False (with ``why_not`` set) unless the result is within ``bound``."""
        try:
            self.exe = build(self.config)
            (out,) = self.exe(operands.a, operands.b)
            self.exe.status()
            error = (out - operands.expected).abs().max().item() / operands.scale
        except Exception as err:  # noqa: BLE001  (a configuration this shape or GPU cannot run)
            text = str(err).splitlines()[0][:80] if str(err) else ""
            self.why_not = f"{self.config}: {type(err).__name__}: {text}"
            return False
        if not error <= bound:
            self.why_not = f"{self.config}: relative error {error:.1e}"
            return False
        return True

    def time(self, rounds):
        """Time the matmul on the operands already in its static buffers; keeps the best seen."""
        if self.timer is None:
            self.timer = GraphTimer(self.exe.run_static)
        seconds = min(self.timer.samples(rounds))
        if self.first_seconds == float("inf"):
            self.first_seconds = seconds
        self.best_seconds = min(self.best_seconds, seconds)
        return seconds


class Verdict:
    """Turns the trials of one shape into the entry that is logged and cached."""

    def __init__(self, shape, default, started):
        self.batch, self.m, self.n, self.k = shape
        self.default = dict(default)
        self.started = started

    def _common(self, n_usable):
        return {"default_config": self.default, "candidates": n_usable,
                "seconds": round(time.perf_counter() - self.started, 1)}

    def nothing_usable(self, refused):
        warnings.warn(f"Kiln: no matmul config passed for {self.batch}x{self.m}x{self.n}x{self.k}; keeping the "
                      f"default. " + "; ".join(refused[:3]))
        return {"config": dict(self.default), "tflops": None, "default_tflops": None, **self._common(0)}

    def choose(self, usable, finalists, refused):
        by_key = {t.key: t for t in finalists}
        winner = min(finalists, key=lambda t: t.best_seconds)
        incumbent = by_key.get(frozen(self.default))
        if incumbent is not None and incumbent.best_seconds <= winner.best_seconds * MIN_GAIN:
            winner = incumbent                  # not enough of a gain to move off the default
        flops = 2 * self.batch * self.m * self.n * self.k
        rate = lambda t: round(flops / t.best_seconds / 1e12, 2)
        return {"config": dict(winner.config), "tflops": rate(winner),
                "default_tflops": rate(incumbent) if incumbent is not None else None,
                **self._common(len(usable)), "rejected": refused[:8]}


class GPUAutotuner:
    """Chooses matmul configs by measurement, with an on-disk cache.  ``config_for`` is what
    kiln.api passes to ``generate`` (kiln/api.py:155-160); ``log`` feeds Report.autotune."""

    def __init__(self, allow_tf32=False, use_cache=True):
        self.allow_tf32 = allow_tf32
        self.precision = resolve_precision(allow_tf32)
        self.use_cache = use_cache
        self.log = []
        self.cache = TuningCache(use_cache)

    def config_for(self, graph, kernel):
        mm = next(node for node in kernel.nodes if node.op == "matmul")
        lhs, rhs = mm.inputs
        batch = int(np.prod(lhs.shape[:-2])) if len(lhs.shape) > 2 else 1
        return self.config_for_shape(batch, lhs.shape[-2], rhs.shape[-1], lhs.shape[-1], default_matmul_config(graph, kernel))

    def config_for_shape(self, batch, m, n, k, default):
        key = f"{device_name()}|{self.precision}|{batch}x{m}x{n}x{k}"
        entry, source = self.cache.get(key), "cache"
        if entry is None:
            entry, source = self.tune(batch, m, n, k, default), "tuned"
            if entry["candidates"]:             # a search in which nothing ran is tried again next time
                self.cache.put(key, entry)
        self.log.append({"shape": (batch, m, n, k), "source": source, **entry})
        return dict(entry["config"])

    def _compile(self, batch, m, n, k, config):
        plan = matmul_plan(batch, m, n, k)
        program = program_from_plan(plan, self.precision, {"k0": dict(config)})
        return GPUExecutable(program, 0, {}, plan.input_shapes, plan.output_shapes, cuda_graphs=False)

    def tune(self, batch, m, n, k, default):
        verdict = Verdict((batch, m, n, k), default, time.perf_counter())
        operands = Operands.make(batch, m, n, k)
        default = dict(default)
        wanted = [default] + [c for c in candidates(m, n, k) if c != default]
        build = lambda config: self._compile(batch, m, n, k, config)
        usable, refused = [], []
        for trial in map(Trial, wanted):
            if trial.check(build, operands, ERROR_BOUND[self.precision]):
                trial.time(rounds=5)
                usable.append(trial)
            else:
                refused.append(trial.why_not)
        if not usable:
            return verdict.nothing_usable(refused)
        finalists = sorted(usable, key=lambda t: t.first_seconds)[:FINALISTS]
        finalists += [t for t in usable if t.key == frozen(default) and t not in finalists]
        for _ in range(TIMING_ROUNDS):          # alternate between the finalists: drift hits them alike
            for trial in finalists:
                trial.time(rounds=2)
        entry = verdict.choose(usable, finalists, refused)
        for trial in usable:
            trial.exe.close()
        return entry


def expected_product(a, b):
    """float64 product used as the tuner's reference (exposed for tests)."""
    return np.matmul(np.asarray(a, np.float64), np.asarray(b, np.float64))
