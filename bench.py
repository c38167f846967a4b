"""Benchmark of the B200 GPU backend on the reference's headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision bf16|tf32|fp32]

Workload (one "step"): 64 independent sequences of 1024 tokens through the GPT-2-small
transformer block (d_model 768, 12 heads, pre-LN, causal attention, tanh-GELU MLP), weights
N(0, 0.02), inputs N(0, 1), seed 4 -- synthetic tensors of the benchmark's shapes.  Every rank
(one process per GPU, independent replicas, no collective on the data path) processes its own
64 sequences per step, so the job is weak-scaled: tokens/s = N * 64 * 1024 / step time.

The block is compiled through the reference's own ``kiln.compile(model, inputs, device="cuda")``
(frontend and passes from the pip --target copy under baseline/_ref) with this package
registered as ``kiln.gpu``; where that copy is absent the plan those passes produce is loaded
from kiln_b200/plans.  It is compiled for a GROUP of eight sequences, ``[8, 1024, 768]``: the
frontend flattens the leading dims of every Linear, so the projections are 8192-row matmuls (256-row
tiles on SM pairs) and the fused attention kernel takes the sequence as one more grid dimension.
Eight such modules (own arena, static buffers and stream each) are kept in flight, the way a server
overlaps requests, and the whole step of 64 sequences -- eight groups -- is captured as ONE CUDA
graph (kiln_b200.runtime.StreamedBatch).  ``extras.single_sequence_graphs`` is the same step as 64
one-sequence graphs over six modules.

Timed regions, each K steps bracketed by barrier + synchronize, CUDA events, max over ranks:
  value   inputs already resident in HBM (device-to-device copies into the modules' inputs);
  e2e     the same graph with pinned HOST tensors as sources and sinks: every sequence's
          host-to-device copy and every result's device-to-host copy inside the timed region;
          e2e.copy_only_ms is the same step with the kernels left out (the host link alone);
  extras.strong_scaling   64 sequences in total, 64 / N per GPU (BASELINE config 4's sharding).
A step touches 64 x 3 MiB of inputs plus eight arenas of tens of MiB, more than the 126 MB L2, so no
explicit flush is needed between iterations; the weights stay L2-resident, as in serving.

``extras`` (rank 0 of a one-GPU run) measures every other BASELINE configuration at its stated
precision whatever --precision says: the 128-token block in FP32, the 2048-token MLP in TF32,
the six Linear shapes in TF32 and BF16, the fused memory-bound ops in FP32, the 2048-token
block (in the run's precision and in FP32); and, in a process of its own, the reference's Triton
backend on the same shapes.

--impl reference times the CPU implementation of the same block (eager PyTorch float32 on the
host cores, the stand-in for the reference's MLIR CPU backend, see oracle/torch_block.py) on a
bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT / "kiln-compiler_b200", ROOT):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import numpy as np  # noqa: E402
import torch  # noqa: E402

SEQS, TOKENS, D, HEADS, SEED = 64, 1024, 768, 12, 4
GROUP = 8             # sequences per compiled graph: the block is compiled for [8, 1024, 768] (eight independent sequences)
INFLIGHT = 8          # compiled modules kept in flight (own stream, arena and static buffers each): one per group
HEAD_CASE = f"gpt2_block_b{GROUP}_t{TOKENS}"
METRIC, UNIT = "gpt2_block_tokens_per_s", "tokens/s"
REF_INSTALL = ROOT / "baseline" / "_ref"


def peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text()), "measured"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons through NVML every few milliseconds while
    the timed region runs (read-only queries; `nvidia-smi -lms` is too slow for a 40 ms region), with
    nvidia-smi as the fallback when the NVML bindings are missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.rows, self.stamps, self.proc, self.thread = index, [], [], None, None
        self.stop = threading.Event()
        self.nvml = None
        self.t_begin = 0.0

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        self.nvml = pynvml
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:   # noqa: BLE001
            return pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll_nvml(self, handle):
        n = self.nvml
        bits = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        mx = n.nvmlDeviceGetMaxClockInfo(handle, n.NVML_CLOCK_SM)
        while not self.stop.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(handle, n.NVML_CLOCK_SM)
                mask = reasons_fn(handle)
                self.rows.append([str(sm), str(mx)] + ["Active" if mask & bits[k] else "Not Active" for k in self.NAMES])
                self.stamps.append(time.perf_counter())
            except Exception:   # noqa: BLE001
                break
            time.sleep(0.002)

    def __enter__(self):
        try:
            handle = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll_nvml, args=(handle,), daemon=True)
            self.thread.start()
            # the first NVML queries of a process take tens of milliseconds, longer than a short timed
            # region: wait until the poller delivers, then count only what it samples from here on
            deadline = time.perf_counter() + 2.0
            while not self.rows and time.perf_counter() < deadline:
                time.sleep(0.001)
            self.t_begin = time.perf_counter()
            return self
        except Exception:   # noqa: BLE001  (no NVML bindings: fall back to the command-line tool)
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])
            self.stamps.append(time.perf_counter())

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        inside = [r for r, t in zip(self.rows, self.stamps) if t >= self.t_begin]
        for r in inside or self.rows:       # (a region shorter than one poll: what was sampled around it)
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, r[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def dist_setup(n):
    """Process group only for the barrier and the max-over-ranks of the timings."""
    import torch.distributed as dist

    if n <= 1 or "RANK" not in os.environ:
        return None, 0, 1, 0
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    dist.init_process_group(backend, rank=rank, world_size=world)
    return dist, rank, world, local


def barrier(dist):
    if dist is not None:
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def max_over_ranks(dist, ms):
    if dist is None:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bind_to_the_gpu_s_cores(local):
    """Run this rank (and so first-touch its pinned buffers) on the cores next to its GPU: the host
    side of every copy then stays on that NUMA node.  Reads the PCI device's local_cpulist; silently
    keeps the current affinity where sysfs does not say."""
    try:
        prop = torch.cuda.get_device_properties(local)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        text = Path(f"/sys/bus/pci/devices/{bdf}/local_cpulist").read_text().strip()
        cores = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cores.update(range(int(lo), int(hi or lo) + 1))
        cores &= os.sched_getaffinity(0)
        if cores:
            os.sched_setaffinity(0, cores)
        return text
    except Exception:   # noqa: BLE001
        return None


# ---------------------------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------------------------

def cpu_block_tokens_per_s(seconds_budget=12.0, threads=None):
    """Eager-PyTorch float32 block on the host cores, on a bounded sample of the workload."""
    from kiln_b200 import workloads as W
    from oracle.torch_block import block_forward, to_torch

    # every core this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    p = to_torch(W.block_params(SEED, TOKENS))
    xs = [torch.from_numpy(W.block_input(SEED, TOKENS, index=i)) for i in range(2)]
    with torch.no_grad():
        block_forward(p, xs[0], HEADS)
        done, t0 = 0, time.perf_counter()
        while True:
            block_forward(p, xs[done % 2], HEADS)
            done += 1
            if time.perf_counter() - t0 > seconds_budget or done >= SEQS:
                break
        dt = time.perf_counter() - t0
    return done * TOKENS / dt, done, torch.get_num_threads()


def reference_arm(args, rank):
    if rank != 0:
        return
    values = []
    for _ in range(args.warmup + args.steps):
        v, done, cores = cpu_block_tokens_per_s(seconds_budget=max(2.0, 60.0 / (args.warmup + args.steps)))
        values.append(v)
    value = float(np.mean(values[args.warmup:]))
    sample = (f"{done} of {SEQS} sequences x {TOKENS} tokens per step, eager PyTorch float32 (oneDNN) in one process "
              f"on rank 0's host cores")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": SEQS * TOKENS / value * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.precision, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(precision, n):
    return {"workload": f"GPT-2-small block (d_model {D}, {HEADS} heads), {SEQS} sequences x {TOKENS} tokens per GPU "
                        f"per step, independent replicas", "sequences_per_gpu": SEQS, "tokens": TOKENS,
            "sequences_per_graph": GROUP, "precision": precision, "parallelism": f"replicas x{n}", "l2": "inputs larger than L2 (no flush)",
            "seed": SEED}


# ---------------------------------------------------------------------------------------------
# Building modules: through kiln.compile when the reference is installed, else from the stored plan
# ---------------------------------------------------------------------------------------------

_KILN = None


def kiln_frontend():
    """The reference's ``kiln`` module with this package registered as its GPU backend, or None."""
    global _KILN
    if _KILN is None:
        _KILN = False
        if (REF_INSTALL / "kiln" / "api.py").exists():
            try:
                sys.path.insert(0, str(REF_INSTALL))
                import kiln_b200

                _KILN = kiln_b200.install()
            except Exception:   # noqa: BLE001
                _KILN = False
    return _KILN or None


class Built:
    """Executables of one benchmark configuration: the first compiled, further copies bound to
    arenas of their own from the same program and constants."""

    def __init__(self, case, precision, cuda_graphs=False):
        from kiln_b200 import workloads as W
        from kiln_b200.codegen import program_from_plan
        from kiln_b200.runtime import GPUExecutable
        from kiln_b200.spec import PlanSpec

        self.case, self.precision, self.cuda_graphs = case, precision, cuda_graphs
        kiln = kiln_frontend()
        self.inputs = None
        if kiln is not None:
            module, x = W.case_module(case)
            old = os.environ.get("KILN_GPU_PRECISION")
            if precision == "bf16":
                os.environ["KILN_GPU_PRECISION"] = "bf16"
            try:
                compiled = kiln.compile(module, (x,), device="cuda", allow_tf32=precision != "fp32", cuda_graphs=cuda_graphs)
            finally:
                if precision == "bf16":
                    os.environ.pop("KILN_GPU_PRECISION", None) if old is None else os.environ.__setitem__("KILN_GPU_PRECISION", old)
            first = compiled._exe
            self.program, self.constants = first.program, compiled.graph.constants
            self.arena_bytes = compiled.graph.attrs.get("arena_bytes", 0)
            self.plan, self.source, self.inputs = first.program.plan, "kiln.compile (baseline/_ref frontend and passes)", [x]
        else:
            plan_json = W.stored_plan(case)
            self.plan = PlanSpec.from_json(plan_json)
            params, x = W.case_tensors(case)
            self.constants = W.plan_constants(self.plan.const_shapes, params)
            self.program = program_from_plan(self.plan, precision)
            self.arena_bytes = self.plan.arena_bytes
            first = GPUExecutable(self.program, self.arena_bytes, self.constants, self.plan.input_shapes,
                                  self.plan.output_shapes, cuda_graphs=cuda_graphs)
            self.source, self.inputs = "stored plan (kiln_b200/plans)", [torch.from_numpy(x)]
        self.executables = [first]
        self.fill(first)

    def fill(self, exe):
        for static, x in zip(exe.static_inputs, self.inputs):
            static.copy_(x)

    @property
    def exe(self):
        return self.executables[0]

    def another(self):
        from kiln_b200.runtime import GPUExecutable

        exe = GPUExecutable(self.program, self.arena_bytes, self.constants, self.plan.input_shapes,
                            self.plan.output_shapes, cuda_graphs=self.cuda_graphs)
        self.fill(exe)
        self.executables.append(exe)
        return exe

    def close(self):
        for e in self.executables:
            e.close()


def time_region(dist, fn, steps):
    barrier(dist)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    barrier(dist)
    return max_over_ranks(dist, start.elapsed_time(end))


def kernel_flops(kernel):
    """Algorithmic FLOPs (matmul) and bytes (everything) of one plan kernel."""
    flops, byts = 0, 0
    for o in kernel.inputs:
        byts += 4 * int(np.prod(o.shape))
    for _, o in kernel.outputs:
        byts += 4 * int(np.prod(o.shape))
    for n in kernel.nodes:
        if n.op == "matmul":
            a = kernel.inputs[n.inputs[0][1]]
            flops += 2 * int(np.prod(n.shape)) * a.shape[-1]
    return flops, byts


# DRAM bytes (read + write) per launch, copied from `ncu --set full` captures of the same shapes as the
# bench (no scaling): the eight-sequence graph's kernels from
# profiles/gpt2_block_b8_t1024_bf16_launches_and_top_kernels.md ("bf16:b8:" keys; outputs that the next
# kernel reads stay in the 126 MB L2 and are not written back inside the launch).
NCU_DRAM_BYTES = {
    "bf16:b8:k0_row": 25245440,
    "bf16:b8:k1_matmul": 17290496,
    "bf16:b8:k2_ew0": 41667840,
    "bf16:b8:k9_matmul": 39930112,
    "bf16:b8:k10_row": 25245952,
    "bf16:b8:k11_matmul": 21331968,
    "bf16:b8:k13_matmul": 85108992,
}


def roofline_of(built, precision, iters=10):
    """Per-launch CUDA-event times of every kernel of the module (each launch alone on the GPU, `iters`
    launches per CUDA graph); roofline of the one with the largest share."""
    pk, pk_kind = peaks()
    exe, plan = built.exe, built.plan
    times = exe.profile_launches(exe.static_inputs[0], iters=iters)
    total = sum(ms for _, ms in times)
    i = max(range(len(times)), key=lambda j: times[j][1])
    name, ms = times[i]
    ki = exe.program.launches[i].kernel_index
    flops, byts = kernel_flops(plan.kernels[ki])
    if exe.impls[i] == "attention_fused":      # this launch stands for the whole attention chain of the plan
        covered = 1
        while i + covered < len(exe.impls) and exe.impls[i + covered] == "fused_away":
            covered += 1
        flops = sum(kernel_flops(k)[0] for k in plan.kernels[ki:ki + covered])
    if flops:
        achieved, unit, bound = flops / (ms * 1e-3) / 1e12, "TFLOP/s", "tensor"
        peak = pk["bf16_tflops"] if precision == "bf16" else pk["bf16_tflops"] / 2
        peak_note = f"{pk_kind} bf16 burst" + ("" if precision == "bf16" else " / 2 (tf32 and fp32 tensor rate)")
    else:
        achieved, unit, bound, peak, peak_note = byts / (ms * 1e-3) / 1e9, "GB/s", "hbm", pk["hbm_gbs"], f"{pk_kind} copy"
    matmuls = {}
    for j, (n, t) in enumerate(times):
        f = kernel_flops(plan.kernels[exe.program.launches[j].kernel_index])[0]
        if exe.impls[j] == "mm_tcgen05" and t > 0:
            matmuls[n] = round(f / (t * 1e-3) / 1e12 / peak, 3)
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": NCU_DRAM_BYTES.get(f"{precision}:b{GROUP}:{name}"),
            "traffic_unit": "bytes per launch (ncu dram read + write)", "kernel": f"{name} ({exe.impls[i]})", "ms_per_launch": ms,
            "share": ms / total, "peak_source": peak_note, "matmul_frac_of_peak": matmuls,
            "per_kernel_ms": {n: round(t, 5) for n, t in times if t > 0.0}}


def graph_times(fn, repeats=20, replays=200):
    """(best, median) seconds per call of ``fn`` over ``replays`` timed replays of a graph of ``repeats`` calls."""
    from kiln_b200.runtime import GraphTimer

    samples = GraphTimer(fn, repeats).samples(replays)
    return float(np.min(samples)), float(np.median(samples))


def tf32_peak_tflops(n=8192):
    """cuBLAS TF32 GEMM throughput measured the way MEASURED_PEAKS.json measures BF16 (torch.matmul, n^3, burst)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a, b = torch.randn(n, n, device="cuda"), torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(10):
            start.record()
            a @ b
            end.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(end))
        return 2 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def host_latency(exe, x_host, calls=200):
    """p50 / best milliseconds of ``exe(x).cpu()`` with a pinned host input: what a caller waits for."""
    for _ in range(5):
        exe(x_host)
    torch.cuda.synchronize()
    lat = []
    for _ in range(calls):
        t0 = time.perf_counter()
        exe(x_host)[0].cpu()
        lat.append((time.perf_counter() - t0) * 1e3)
    return float(np.median(lat)), float(np.min(lat))


def device_call_ms(fn, calls=200, rounds=5):
    """Milliseconds per call of a compiled module on device tensors, back-to-back calls between two
    CUDA events, best of `rounds` (how the reference's benchmark times a block: bench_gpu.py:54-81)."""
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(rounds):
        start.record()
        for _ in range(calls):
            fn()
        end.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(end) / calls)
    return best


def block_numbers(case, precision):
    """One sequence through the block: GPU time of its kernels, per call on device tensors, host to host."""
    direct = Built(case, precision, cuda_graphs=False)
    kernel_best, kernel_p50 = graph_times(direct.exe.run_static)
    direct.close()
    graphed = Built(case, precision, cuda_graphs=True)
    t = graphed.plan.input_shapes[0][0]
    xd = torch.randn(t, D, device="cuda")
    call_ms = device_call_ms(lambda: graphed.exe(xd))
    p50, best = host_latency(graphed.exe, torch.randn(t, D).pin_memory())
    graphed.close()
    return {"precision": precision, "e2e_p50_ms": round(p50, 4), "e2e_best_ms": round(best, 4), "call_ms": round(call_ms, 4),
            "kernel_ms": round(kernel_best * 1e3, 4), "kernel_p50_ms": round(kernel_p50 * 1e3, 4),
            "tokens_per_s": round(t / call_ms * 1e3), "built_from": graphed.source}


def single_sequence_step(precision, in_flight=6):
    """The same 64 sequences as 64 one-sequence graphs ([1024, 768] modules, the reference's own test
    model shape) over six modules in flight: what the step costs without batching sequences into
    one graph.  Each plan is told how many share the GPU (wide tiles on its share of the SM pairs)."""
    from kiln_b200 import workloads as W
    from kiln_b200.runtime import StreamedBatch

    built = Built(f"gpt2_block_t{TOKENS}", precision)
    for _ in range(in_flight - 1):
        built.another()
    dev_in = torch.stack([torch.from_numpy(W.block_input(SEED, TOKENS, index=i)) for i in range(SEQS)]).cuda()
    dev_out = torch.empty_like(dev_in)
    step = StreamedBatch(built.executables).capture(list(dev_in), list(dev_out))
    for _ in range(3):
        step.run()
    ms = time_region(None, step.run, 10) / 10
    step.status()
    out = {"modules_in_flight": in_flight, "ms_per_step": round(ms, 4), "tokens_per_s": round(SEQS * TOKENS / (ms * 1e-3)),
           "launches_per_step": SEQS * built.exe.device_launches}
    built.close()
    return out


def extras(precision):
    """Every other BASELINE configuration at its stated precision: fused-op GB/s (config 3), Linear
    TFLOP/s in TF32 and BF16 (config 2), the 2048-token MLP in TF32 (config 1), the 128-token block in
    FP32 (config 0), the 128- and 2048-token blocks in the run's precision (config 4, one GPU)."""
    from kiln_b200 import workloads as W

    out = {}
    pk, _ = peaks()
    for case, byts in (("bias_gelu_2048x3072", 50343936), ("layernorm_2048x768", 12589056),
                       ("softmax_12x512x512", 25165824)):
        built = Built(case, "fp32")
        best, p50 = graph_times(built.exe.run_static)
        # cold: rotate through enough copies of the operands that nothing is left in the 126 MB L2
        n_sets = max(2, -(-2 * 126 * 2**20 // byts) + 1)
        for _ in range(n_sets - 1):
            built.another()

        def rotate(sets=built.executables):
            for e in sets:
                e.run_static()

        cold_best, cold_p50 = graph_times(rotate, repeats=2, replays=50)
        out[case] = {"warm_gbs": round(byts / best / 1e9, 1), "warm_p50_gbs": round(byts / p50 / 1e9, 1),
                     "cold_gbs": round(byts * n_sets / cold_best / 1e9, 1), "cold_p50_gbs": round(byts * n_sets / cold_p50 / 1e9, 1),
                     "frac_of_measured_hbm": round(byts * n_sets / cold_best / 1e9 / pk["hbm_gbs"], 3),
                     "buffer_sets": n_sets, "impl": built.exe.impls}
        built.close()
    tf32_peak = tf32_peak_tflops()
    out["tf32_peak_tflops_measured"] = round(tf32_peak, 1)
    for mm_prec, mm_peak in (("tf32", tf32_peak), ("bf16", pk["bf16_tflops"])):
        table = {}
        for m, n, k in W.LINEAR_SHAPES:
            built = Built(f"linear_{m}x{n}x{k}", mm_prec)
            best, p50 = graph_times(built.exe.run_static)
            row = {"tflops": round(2 * m * n * k / best / 1e12, 2), "p50_tflops": round(2 * m * n * k / p50 / 1e12, 2),
                   "us": round(best * 1e6, 2), "impl": built.exe.impls}
            if m > 1:
                row["frac_of_measured_peak"] = round(row["tflops"] / mm_peak, 3)
            else:      # decode GEMV: weights streamed once; cold = weight sets rotated through more than twice the L2
                byts = 4 * k * n + 4 * n + 4 * k
                row["gbs"] = round(byts / best / 1e9, 1)
                n_sets = -(-2 * 126 * 2**20 // byts) + 1
                for _ in range(n_sets - 1):
                    built.another()

                def rotate(sets=built.executables):
                    for e in sets:
                        e.run_static()

                cold_best, _ = graph_times(rotate, repeats=2, replays=50)
                row["cold_gbs"] = round(byts * n_sets / cold_best / 1e9, 1)
                row["cold_frac_of_measured_hbm"] = round(byts * n_sets / cold_best / 1e9 / pk["hbm_gbs"], 3)
            table[f"{m}x{n}x{k}"] = row
            built.close()
        out[f"linear_{mm_prec}"] = table
    built = Built("mlp_2048", "tf32")
    best, p50 = graph_times(built.exe.run_static)
    flops = 2 * 2 * 2048 * 768 * 3072
    out["mlp_2048_tf32"] = {"tflops": round(flops / best / 1e12, 2), "p50_tflops": round(flops / p50 / 1e12, 2), "us": round(best * 1e6, 2),
                            "frac_of_measured_peak": round(flops / best / 1e12 / tf32_peak, 3), "impl": built.exe.impls,
                            "built_from": built.source}
    built.close()
    out["single_sequence_graphs"] = single_sequence_step(precision)
    out["block_t128_fp32"] = block_numbers("gpt2_block_t128", "fp32")
    out["block_t128_tf32"] = block_numbers("gpt2_block_t128", "tf32")      # the precision the reference's Triton arm is timed in
    if precision not in ("fp32", "tf32"):
        out["block_t128"] = block_numbers("gpt2_block_t128", precision)
    out["block_t2048"] = block_numbers("gpt2_block_t2048", precision)
    if precision != "fp32":
        out["block_t2048_fp32"] = block_numbers("gpt2_block_t2048", "fp32")    # FP32 mode's attention runs on the FMA pipes
    return out


# ---------------------------------------------------------------------------------------------
# The reference's own Triton backend on this GPU (an extra comparison point, not `--impl reference`)
# ---------------------------------------------------------------------------------------------

def reference_triton_arm(args):
    """The reference's Triton GPU backend, stock ``kiln.compile`` from baseline/_ref, on the same
    shapes and inputs, timed the way the reference's benchmark does (benchmarks/bench_gpu.py:43-81,
    114-192): kernel time as a CUDA-graph replay for the Linears, the MLP and the fused ops, ms per
    call and host-to-host p50 for the block.  Prints one JSON line per finished section, so that a
    caller with a time limit keeps what was done."""
    from kiln_b200 import workloads as W
    from kiln_b200.install import register_mlir_stub

    tag = {"impl": "reference-triton"}
    if not (REF_INSTALL / "kiln" / "gpu").is_dir():
        print(json.dumps(dict(tag, unavailable="the reference is not installed under baseline/_ref")), flush=True)
        return
    if not torch.cuda.is_available():
        print(json.dumps(dict(tag, unavailable="no CUDA device")), flush=True)
        return
    sys.path.insert(0, str(REF_INSTALL))
    register_mlir_stub()
    import kiln
    from kiln.gpu.runtime import kernel_seconds as reference_kernel_seconds

    def section(name, fn):
        try:
            print(json.dumps(dict(tag, section=name, **fn())), flush=True)
        except Exception as err:   # noqa: BLE001  (an extra: report, never fail the run)
            print(json.dumps(dict(tag, section=name, unavailable=f"{type(err).__name__}: {err}"[:300])), flush=True)

    def block(tokens, seed, allow_tf32, batch=0):
        def run():
            if batch:
                model = W.batched_block_module(seed, tokens)
                x = torch.from_numpy(np.stack([W.block_input(seed, tokens, index=i) for i in range(batch)]))
            else:
                model = W.block_module(seed, tokens)
                x = torch.from_numpy(W.block_input(seed, tokens, index=0))
            t0 = time.perf_counter()
            compiled = kiln.compile(model, (x,), device="cuda", allow_tf32=allow_tf32, autotune=args.autotune)
            compile_s = time.perf_counter() - t0
            xd = x.cuda()
            with torch.no_grad():
                want = model(x).double()
                err = float((compiled(xd).cpu().double() - want).abs().max() / want.abs().max())
                call_ms = device_call_ms(lambda: compiled(xd))
                xp = x.pin_memory()
                for _ in range(5):
                    compiled(xp)
                torch.cuda.synchronize()
                lat = []
                for _ in range(50):
                    t0 = time.perf_counter()
                    compiled(xp).cpu()
                    lat.append((time.perf_counter() - t0) * 1e3)
            return {"precision": "tf32" if allow_tf32 else "fp32", "call_ms": round(call_ms, 4),
                    "e2e_p50_ms": round(float(np.median(lat)), 4), "tokens_per_s": round(max(1, batch) * tokens / call_ms * 1e3),
                    "rel_err_vs_eager": err, "compile_s": round(compile_s, 1), "autotune": bool(args.autotune)}
        return run

    def kernel_case(case, allow_tf32, autotune, flops=None, byts=None):
        def run():
            module, x = W.case_module(case)
            compiled = kiln.compile(module, (x,), device="cuda", allow_tf32=allow_tf32, cuda_graphs=False, autotune=autotune)
            xd = x.cuda()
            with torch.no_grad():
                seconds = reference_kernel_seconds(lambda: compiled(xd))
            row = {"precision": "tf32" if allow_tf32 else "fp32", "us": round(seconds * 1e6, 2), "autotune": bool(autotune)}
            if flops:
                row["tflops"] = round(flops / seconds / 1e12, 2)
            if byts:
                row["warm_gbs"] = round(byts / seconds / 1e9, 1)
            return row
        return run

    section("block_t128_fp32", block(128, 0, False))
    section("block_t128", block(128, 0, True))
    section("block_t2048", block(2048, SEED, True))
    section("block_t2048_fp32", block(2048, SEED, False))
    section("block_t1024", block(1024, SEED, True))
    for m, n, k in W.LINEAR_SHAPES:
        section(f"linear_tf32_{m}x{n}x{k}", kernel_case(f"linear_{m}x{n}x{k}", True, args.autotune, flops=2 * m * n * k))
    section("mlp_2048_tf32", kernel_case("mlp_2048", True, args.autotune, flops=2 * 2 * 2048 * 768 * 3072))
    for case, byts in (("bias_gelu_2048x3072", 50343936), ("layernorm_2048x768", 12589056), ("softmax_12x512x512", 25165824)):
        section(case, kernel_case(case, False, False, byts=byts))
    section(f"block_b{GROUP}_t1024", block(1024, SEED, True, batch=GROUP))


def reference_triton_extra(budget_s=300):
    """Runs the arm above in a process of its own (it registers the same module names this package
    does) and keeps every section that finished within the budget."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference-triton", "--autotune"]
    out = {"impl": "reference-triton", "budget_s": budget_s}
    try:
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        try:
            stdout, _ = proc.communicate(timeout=budget_s)
        except subprocess.TimeoutExpired:
            proc.kill()
            stdout, _ = proc.communicate()
            out["stopped_at_budget"] = True
        for text in stdout.splitlines():
            if not text.startswith("{"):
                continue
            row = json.loads(text)
            if "section" in row:
                out[row["section"]] = {k: v for k, v in row.items() if k not in ("impl", "section")}
            elif "unavailable" in row:
                out["unavailable"] = row["unavailable"]
    except Exception as err:   # noqa: BLE001
        out["unavailable"] = f"{type(err).__name__}: {err}"[:200]
    return out


def dtype_of(precision, impls):
    """The arithmetic the matmuls really ran in: the tensor-core kernels take tf32 / bf16 operands,
    every other kernel (and every accumulation) is float32."""
    if precision == "fp32" or not any(i == "mm_tcgen05" for i in impls):
        return "f32"
    return precision


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def gpu_arm(args, dist, rank, world, local):
    from kiln_b200 import workloads as W
    from kiln_b200.runtime import StreamedBatch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    cpulist = bind_to_the_gpu_s_cores(local)
    precision = args.precision
    groups = SEQS // GROUP
    host = [torch.from_numpy(np.stack([W.block_input(SEED, TOKENS, index=rank * SEQS + g * GROUP + i) for i in range(GROUP)])).pin_memory()
            for g in range(groups)]
    dev_in = [h.cuda(non_blocking=True) for h in host]
    dev_out = [torch.empty_like(t) for t in dev_in]
    host_out = [torch.empty(GROUP, TOKENS, D).pin_memory() for _ in range(groups)]
    torch.cuda.synchronize()

    # INFLIGHT compiled modules (own arena, static buffers and stream each) run round-robin, as a server
    # keeps several requests in flight: copies of one group overlap kernels of another.  A whole step of
    # 64 sequences is one CUDA graph, so a busy host does not starve the GPU of launches.  Every kernel
    # of an eight-sequence graph is large enough for the whole GPU, so the plans are not told to share it.
    built = Built(HEAD_CASE, precision)
    for _ in range(INFLIGHT - 1):
        built.another()
    exes, exe = built.executables, built.exe
    resident = StreamedBatch(exes, concurrency=1).capture(dev_in, dev_out)
    for _ in range(args.warmup):
        resident.run()
    with ClockSampler(local) as clocks:
        resident.run()          # (untimed: the sampler's start-up left the GPU idle for a moment)
        ms = time_region(dist, resident.run, args.steps)
    resident.status()
    # end to end: the same step with pinned host tensors as sources and sinks (201 MB each way per step)
    e2e = StreamedBatch(exes, concurrency=1).capture(host, host_out)
    for _ in range(max(1, args.warmup // 2)):
        e2e.run()
    ms_e2e = time_region(dist, e2e.run, args.steps)
    e2e.status()
    # ... and the same copies with no kernels between them: the host link's share of that step
    copies = StreamedBatch(exes, concurrency=1).capture(host, host_out, kernels=False)
    copies.run()
    ms_copies = time_region(dist, copies.run, args.steps)
    # strong scaling (BASELINE config 4): 64 sequences in total, 64 / world per GPU
    share = max(1, groups // world)
    strong = StreamedBatch(exes, concurrency=1).capture(dev_in[:share], dev_out[:share])
    for _ in range(args.warmup):
        strong.run()
    ms_strong = time_region(dist, strong.run, args.steps)
    strong.status()
    tokens = world * SEQS * TOKENS * args.steps
    value, e2e_value = tokens / (ms * 1e-3), tokens / (ms_e2e * 1e-3)
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_of(precision, exe.impls), "data": "synthetic",
        "config": workload_config(precision, world),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": world * SEQS * TOKENS * D * 4,
                "d2h_bytes_per_step": world * SEQS * TOKENS * D * 4, "ms_per_step": ms_e2e / args.steps,
                "copy_only_ms": ms_copies / args.steps, "modules_in_flight": INFLIGHT, "host_cores_near_gpu": cpulist},
        "gpu_launches": world * args.steps * groups * exe.device_launches, "modules_in_flight": INFLIGHT,
        "sequences_per_graph": GROUP,
        "clocks": clocks.summary(),
        "impls": dict(zip(exe.launch_names, exe.impls)),
        "built_from": built.source,
    }
    line["roofline"] = roofline_of(built, precision)
    line["extras"] = {"strong_scaling": {"sequences_total": share * GROUP * world, "sequences_per_gpu": share * GROUP,
                                         "ms_per_step": ms_strong / args.steps,
                                         "tokens_per_s": share * GROUP * world * TOKENS * args.steps / (ms_strong * 1e-3)}}
    if world == 1:
        v, done, cores = cpu_block_tokens_per_s(seconds_budget=12.0)
        v1, done1, _ = cpu_block_tokens_per_s(seconds_budget=6.0, threads=1)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{done} of {SEQS} sequences x {TOKENS} tokens, eager PyTorch float32 (oneDNN)",
                                "one_thread": {"value": v1, "unit": UNIT, "cores": 1,
                                               "sample": f"{done1} sequences x {TOKENS} tokens"}}
        if not args.no_extras:
            built.close()
            try:
                line["extras"].update(extras(precision))
            except Exception as err:   # noqa: BLE001  (extras never invalidate the headline line)
                line["extras"]["error"] = f"{type(err).__name__}: {err}"[:200]
            line["extras"]["reference_triton"] = reference_triton_extra()
    print(json.dumps(line), flush=True)


def single_case(args):
    """One configuration, launched directly (no CUDA graph) so a profiler sees plain kernel launches."""
    built = Built(args.case, args.precision)
    exe = built.exe
    for _ in range(max(1, args.warmup)):
        exe.run_static()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        exe.run_static()
    end.record()
    torch.cuda.synchronize()
    exe.status()
    print(json.dumps({"case": args.case, "precision": args.precision, "impls": exe.impls, "built_from": built.source,
                      "ms_per_call": start.elapsed_time(end) / args.steps, "launches_per_call": exe.device_launches}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--autotune", action="store_true", help="reference-triton only: let the reference autotune its matmuls")
    ap.add_argument("--precision", default="bf16", choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", default=None,
                    help="run one benchmark configuration (a name under kiln_b200/plans) --steps times and print its "
                         "GPU time per call; the small, single-kernel workload to put under a profiler")
    args = ap.parse_args()
    if args.case:
        single_case(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference-triton":
        if int(os.environ.get("RANK", 0)) == 0:
            reference_triton_arm(args)
        return
    if args.impl == "reference":
        reference_arm(args, int(os.environ.get("RANK", 0)))
        return
    dist, rank, world, local = dist_setup(args.gpus)
    try:
        gpu_arm(args, dist, rank, world, local)
    finally:
        if dist is not None:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
