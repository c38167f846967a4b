"""GPU matmul autotuning by measurement (stands in for kiln.gpu.autotune).

Same procedure as the reference's tuner (kiln/gpu/autotune.py:113-193): every candidate is
built as a standalone matmul, rejected unless it matches a float64 product to a tolerance
relative to the output's scale, timed as GPU time only (many launches in one CUDA graph), the
fastest few and the default are re-timed interleaved, and the default is kept unless a candidate
beats it by MIN_GAIN.  Results are cached by GPU name, precision and shape in
$KILN_CACHE_DIR/b200_autotune.json (written to a temporary file and renamed; a corrupt cache is
ignored).

What is searched is this backend's own space, not Triton's: the tcgen05 tile width (BN, with
BM fixed at the 128 rows one CTA's accumulator spans), the number of pipeline stages and the
split-K factor (in exact-FP32 mode the library narrows tiles to 128 columns and fits the stage
count itself); plus the CUDA-core FP32 kernel as a candidate.
"""

from __future__ import annotations

import json
import os
import time
import warnings
from pathlib import Path

import numpy as np
import torch

from kiln_b200.codegen import default_matmul_config, next_pow2, program_from_plan, resolve_precision
from kiln_b200.runtime import GPUExecutable, device, kernel_seconds
from kiln_b200.spec import KernelSpec, NodeSpec, OperandSpec, PlanSpec

MIN_GAIN = 1.03
FINALISTS = 3
SHARED_MEMORY_BYTES = 227 * 1024     # per CTA on B200

TC_CANDIDATES = [  # BN, stages, split_k
    (256, 4, 1), (256, 3, 1), (128, 4, 1), (128, 6, 1), (64, 6, 1), (128, 4, 2), (128, 4, 4), (64, 6, 2), (64, 6, 4),
    (64, 6, 8), (256, 3, 2),
]
EPILOGUE_BYTES = 8 * 7168            # the epilogue warps' transpose / staging buffers


def cache_path() -> Path:
    base = os.environ.get("KILN_CACHE_DIR") or os.path.join(Path.home(), ".cache", "kiln")
    return Path(base) / "b200_autotune.json"


def device_name():
    return torch.cuda.get_device_name(device())


def stage_bytes(cfg):
    """Shared memory one pipeline stage holds: a 128-row A slab and a BN-row B slab of 128 bytes per row."""
    return (cfg["BM"] + cfg["BN"]) * 128


def candidates(m, n, k):
    out = []
    for bn, stages, split in TC_CANDIDATES:
        if bn > max(64, next_pow2(n)):
            continue            # a tile much wider than the problem only adds masked-off work
        if split > 1 and k // split < 128:
            continue
        cfg = {"BM": 128, "BN": bn, "stages": stages, "split_k": split, "impl": "tc"}
        if stage_bytes(cfg) * stages + EPILOGUE_BYTES + 1024 > SHARED_MEMORY_BYTES:
            continue
        out.append(cfg)
    out.append({"BM": 64, "BN": 64, "stages": 1, "split_k": 1, "impl": "simt"})
    return out


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


class GPUAutotuner:
    """Chooses matmul configs by measurement, with an on-disk cache.  ``config_for`` is what
    kiln.api passes to ``generate`` (kiln/api.py:155-160); ``log`` feeds Report.autotune."""

    def __init__(self, allow_tf32=False, use_cache=True):
        self.allow_tf32 = allow_tf32
        self.precision = resolve_precision(allow_tf32)
        self.use_cache = use_cache
        self.log = []
        self._cache = self._load() if use_cache else {}

    def _load(self):
        try:
            data = json.loads(cache_path().read_text())
            return data if isinstance(data, dict) else {}
        except (OSError, ValueError):
            return {}

    def _save(self):
        if not self.use_cache:
            return
        path = cache_path()
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            tmp = path.with_suffix(f".{os.getpid()}.tmp")
            tmp.write_text(json.dumps(self._cache, indent=1, sort_keys=True))
            tmp.replace(path)
        except OSError as err:
            warnings.warn(f"Kiln: couldn't write the GPU autotune cache ({err})")

    def config_for(self, graph, kernel):
        mm = next(n for n in kernel.nodes if n.op == "matmul")
        a, b = mm.inputs
        batch = 1
        for d in a.shape[:-2]:
            batch *= d
        m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
        return self.config_for_shape(batch, m, n, k, default_matmul_config(graph, kernel))

    def config_for_shape(self, batch, m, n, k, default):
        key = f"{device_name()}|{self.precision}|{batch}x{m}x{n}x{k}"
        if key not in self._cache:
            entry = self.tune(batch, m, n, k, default)
            if entry["candidates"]:             # don't cache a failed search
                self._cache[key] = entry
                self._save()
            source = "tuned"
        else:
            entry, source = self._cache[key], "cache"
        self.log.append({"shape": (batch, m, n, k), "source": source, **entry})
        return dict(entry["config"])

    def _compile(self, batch, m, n, k, config):
        plan = matmul_plan(batch, m, n, k)
        program = program_from_plan(plan, self.precision, {"k0": dict(config)})
        return GPUExecutable(program, 0, {}, plan.input_shapes, plan.output_shapes, cuda_graphs=False)

    def tune(self, batch, m, n, k, default):
        start = time.perf_counter()
        dev = device()
        gen = torch.Generator(device="cpu").manual_seed(0)
        lead = (batch,) if batch > 1 else ()
        a = torch.randn(*lead, m, k, generator=gen).to(dev)
        b = (torch.randn(*lead, k, n, generator=gen) / k ** 0.5).to(dev)   # outputs of order 1, like a real layer
        expected = (a.double() @ b.double()).float()
        # error relative to the output's scale (kiln/gpu/autotune.py:147-151)
        tol = {"fp32": 1e-4, "tf32": 2e-2, "bf16": 5e-2}[self.precision]
        scale = expected.abs().max().item() or 1.0
        runs, seconds, rejected = {}, {}, []
        default = dict(default)
        configs = [default] + [c for c in candidates(m, n, k) if c != default]
        for cfg in configs:
            key = tuple(sorted(cfg.items()))
            try:
                exe = self._compile(batch, m, n, k, cfg)
                (out,) = exe(a, b)
                exe.status()
                err = (out - expected).abs().max().item() / scale
                if not err <= tol:
                    rejected.append(f"{cfg}: relative error {err:.1e}")
                    continue
            except Exception as e:  # noqa: BLE001  (a config this shape or GPU cannot run)
                rejected.append(f"{cfg}: {type(e).__name__}: {str(e).splitlines()[0][:80] if str(e) else ''}")
                continue
            runs[key] = exe.run_static
            seconds[key] = kernel_seconds(runs[key])
        default_key = tuple(sorted(default.items()))
        if not seconds:                         # nothing usable: keep the default rather than fail
            warnings.warn(f"Kiln: no matmul config passed for {batch}x{m}x{n}x{k}; keeping the default. "
                          + "; ".join(rejected[:3]))
            return {"config": dict(default), "default_config": default, "tflops": None, "default_tflops": None,
                    "candidates": 0, "seconds": round(time.perf_counter() - start, 1)}
        ranked = sorted(seconds, key=seconds.get)[:FINALISTS]
        if default_key in seconds and default_key not in ranked:
            ranked.append(default_key)
        final = {}
        for _ in range(3):                      # interleaved re-timing
            for key in ranked:
                final[key] = min(final.get(key, float("inf")), kernel_seconds(runs[key], rounds=2))
        winner = min(final, key=final.get)
        if default_key in final and final[default_key] <= final[winner] * MIN_GAIN:
            winner = default_key
        flops = 2 * batch * m * n * k
        return {
            "config": dict(winner),
            "default_config": default,
            "tflops": round(flops / final[winner] / 1e12, 2),
            "default_tflops": round(flops / final[default_key] / 1e12, 2) if default_key in final else None,
            "candidates": len(seconds),
            "seconds": round(time.perf_counter() - start, 1),
            "rejected": rejected[:8],
        }


def expected_product(a, b):
    """float64 product used as the tuner's reference (exposed for tests)."""
    return np.matmul(np.asarray(a, np.float64), np.asarray(b, np.float64))
