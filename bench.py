"""Benchmark of the B200 GPU backend on the reference's headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision bf16|tf32|fp32]

Workload (one "step"): 64 independent sequences of 1024 tokens through the GPT-2-small
transformer block (d_model 768, 12 heads, pre-LN, causal attention, tanh-GELU MLP), weights
N(0, 0.02), inputs N(0, 1), seed 4 -- synthetic tensors of the benchmark's shapes.  Every rank
(one process per GPU, independent replicas, no collective on the data path) processes its own
64 sequences per step, so the job is weak-scaled: tokens/s = N * 64 * 1024 / step time.

Two timed regions, both K steps bracketed by barrier + synchronize, CUDA events, max over ranks:
  value  inputs already resident in HBM; each sequence is copied device-to-device into a compiled
         module's static input, its captured CUDA graph is replayed, the result copied out.
  e2e    the public call ``executable(x)`` with pinned host tensors: host-to-device copy of every
         sequence and device-to-host read of every result inside the timed region.
In both regions three compiled modules (own arena, own CUDA graph) are kept in flight on separate
streams, the way a server overlaps requests: copies overlap kernels, and one sequence's kernels fill
SMs another leaves idle.
A step touches 64 x 3 MiB of inputs plus a 105 MiB arena, more than the 126 MB L2, so no explicit
L2 flush is needed between iterations; the weights (14-28 MB) stay L2-resident, as in serving.

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
for _p in (ROOT / "kiln-compiler_b200", ROOT, ROOT / "tests"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import numpy as np  # noqa: E402
import torch  # noqa: E402

SEQS, TOKENS, D, HEADS, SEED = 64, 1024, 768, 12, 4
INFLIGHT = int(os.environ.get("KB200_BENCH_INFLIGHT", "6"))          # compiled modules kept in flight (own stream, arena and CUDA graph each); 6 reaches the host-link bound
METRIC, UNIT = "gpt2_block_tokens_per_s", "tokens/s"


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
        self.index, self.rows, self.proc, self.thread = index, [], None, None
        self.stop = threading.Event()
        self.nvml = None

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
            except Exception:   # noqa: BLE001
                break
            time.sleep(0.002)

    def __enter__(self):
        try:
            handle = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll_nvml, args=(handle,), daemon=True)
            self.thread.start()
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
        for r in self.rows:
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


def reference_arm(args, dist, rank):
    if rank != 0:
        return
    values = []
    for _ in range(args.warmup + args.steps):
        v, done, cores = cpu_block_tokens_per_s(seconds_budget=max(2.0, 60.0 / (args.warmup + args.steps)))
        values.append(v)
    value = float(np.mean(values[args.warmup:]))
    sample = f"{done} of {SEQS} sequences x {TOKENS} tokens per step, eager PyTorch float32 (oneDNN)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": SEQS * TOKENS / value * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(args.precision, args.gpus), cpu_arithmetic="f32, one process on rank 0's host cores"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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


def reference_triton_arm(args):
    """The reference's own Triton GPU backend on this GPU, same block and inputs, timed the way the
    reference's benchmark does (benchmarks/bench_gpu.py:43-49, 54-81): GPU time per call as a CUDA-graph
    replay, and host-to-host p50 latency.  Needs the reference installed under baseline/_ref (a
    git-ignored pip --target directory); prints an `unavailable` line otherwise.  Not the
    `--impl reference` arm: an extra comparison point."""
    from kiln_b200 import workloads as W
    from kiln_b200.install import register_mlir_stub

    def fail(why):
        print(json.dumps(dict(line, unavailable=why)), flush=True)

    root = ROOT / "baseline" / "_ref"
    line = {"impl": "reference-triton", "precision": "tf32" if args.precision != "fp32" else "fp32"}
    if not (root / "kiln" / "gpu").is_dir():
        print(json.dumps(dict(line, unavailable="the reference is not installed under baseline/_ref")), flush=True)
        return
    if not torch.cuda.is_available():
        print(json.dumps(dict(line, unavailable="no CUDA device")), flush=True)
        return
    try:
        sys.path.insert(0, str(root))
        register_mlir_stub()
        import kiln

        allow_tf32 = args.precision != "fp32"
        out = {}
        for tokens, seed in ((128, 0), (1024, SEED), (2048, SEED)):
            model = W.block_module(seed, tokens)
            x = torch.from_numpy(W.block_input(seed, tokens, index=0))
            t0 = time.perf_counter()
            compiled = kiln.compile(model, (x,), device="cuda", allow_tf32=allow_tf32, autotune=args.autotune)
            compile_s = time.perf_counter() - t0
            xd = x.cuda()
            with torch.no_grad():
                want = model(x).double()
                got = compiled(xd).cpu().double()
                err = float((got - want).abs().max() / want.abs().max())
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
            out[f"block_t{tokens}"] = {"call_ms": round(call_ms, 4), "e2e_p50_ms": round(float(np.median(lat)), 4),
                                       "tokens_per_s": round(tokens / call_ms * 1e3), "rel_err_vs_eager": err,
                                       "compile_s": round(compile_s, 1)}
        line.update(out, autotune=bool(args.autotune))
    except Exception as err:   # noqa: BLE001  (an extra: report, never fail the run)
        line["unavailable"] = f"{type(err).__name__}: {err}"[:300]
    print(json.dumps(line), flush=True)


def workload_config(precision, n):
    return {"workload": f"GPT-2-small block (d_model {D}, {HEADS} heads), {SEQS} sequences x {TOKENS} tokens per GPU "
                        f"per step, independent replicas", "sequences_per_gpu": SEQS, "tokens": TOKENS,
            "precision": precision, "parallelism": f"replicas x{n}", "l2": "inputs larger than L2 (no flush)",
            "seed": SEED}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def build_block(precision, tokens, seed, cuda_graphs=True):
    from helpers import load_plan
    from kiln_b200 import workloads as W
    from kiln_b200.codegen import program_from_plan
    from kiln_b200.runtime import GPUExecutable
    from kiln_b200.spec import PlanSpec

    plan = PlanSpec.from_json(load_plan(f"gpt2_block_t{tokens}"))
    consts = W.plan_constants(plan.const_shapes, W.block_params(seed, tokens))
    # per-kernel matmul configurations, e.g. KB200_BENCH_CONFIGS='{"k10": {"BN": 256}}' (experiments; default: the library's choice)
    configs = json.loads(os.environ.get("KB200_BENCH_CONFIGS", "null"))
    program = program_from_plan(plan, precision, configs)
    return GPUExecutable(program, plan.arena_bytes, consts, plan.input_shapes, plan.output_shapes,
                         cuda_graphs=cuda_graphs), plan


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


# DRAM bytes (read + write) per launch of the 1024-token block's kernels in BF16 mode, from the
# `ncu --set full` capture summarised in profiles/gpt2_block_t1024_bf16_launches_and_top_kernels.md.
NCU_DRAM_BYTES = {
    ("bf16", "k0_row"): 3.16e6, ("bf16", "k1_matmul"): 5.21e6, ("bf16", "k2_ew0"): 4.77e6, ("bf16", "k7_matmul"): 6.00e6,
    ("bf16", "k8_row"): 3.16e6, ("bf16", "k9_matmul"): 6.41e6, ("bf16", "k10_matmul"): 14.26e6,
    ("fp32", "k0_row"): 3.16e6, ("fp32", "k1_matmul"): 10.33e6, ("fp32", "k3_matmul"): 10.81e6, ("fp32", "k4_row"): 51.88e6,
    ("fp32", "k5_matmul"): 53.57e6, ("fp32", "k6_ew0"): 3.18e6, ("fp32", "k7_matmul"): 8.75e6, ("fp32", "k8_row"): 3.16e6,
    ("fp32", "k9_matmul"): 12.70e6, ("fp32", "k10_matmul"): 25.28e6,
}


def roofline_of(exe, plan, precision, iters=20):
    """Per-launch CUDA-event times of every kernel; roofline of the one with the largest share."""
    pk, pk_kind = peaks()
    times = exe.profile_launches(exe.static_inputs[0], iters=iters)
    total = sum(ms for _, ms in times)
    i = max(range(len(times)), key=lambda j: times[j][1])
    name, ms = times[i]
    ki = exe.program.launches[i].kernel_index
    flops, byts = kernel_flops(plan.kernels[ki])
    if exe.impls[i] == "attention_fused":      # this launch stands for the whole five-kernel attention chain
        flops = sum(kernel_flops(k)[0] for k in plan.kernels[ki:ki + 5])
    if flops:
        achieved, unit, bound = flops / (ms * 1e-3) / 1e12, "TFLOP/s", "tensor"
        peak = pk["bf16_tflops"] if precision == "bf16" else pk["bf16_tflops"] / 2
        peak_note = f"{pk_kind} bf16 burst" + ("" if precision == "bf16" else " / 2 (tf32 and fp32 tensor rate)")
    else:
        achieved, unit, bound, peak, peak_note = byts / (ms * 1e-3) / 1e9, "GB/s", "hbm", pk["hbm_gbs"], f"{pk_kind} copy"
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": NCU_DRAM_BYTES.get((precision, name)) if TOKENS == 1024 else None,
            "traffic_unit": "bytes per launch (ncu dram read + write)", "kernel": f"{name} ({exe.impls[i]})", "ms_per_launch": ms, "share": ms / total,
            "peak_source": peak_note,
            "per_kernel_ms": {n: round(t, 5) for n, t in times}}


def graph_times(fn, repeats=20, replays=200):
    """(best, median) seconds per call of ``fn``: ``repeats`` calls captured in one CUDA graph, the
    replay timed with CUDA events ``replays`` times (the reference's kernel_seconds, runtime.py:93-132,
    with a p50 beside the best)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(repeats):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    samples = []
    for _ in range(replays):
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(end) / 1e3 / repeats)
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


def extras(precision):
    """The reference's other headline numbers: block latency, Linear TFLOP/s, fused-op GB/s."""
    from gpu_helpers import build_executable
    from helpers import case_data, load_plan

    def filled(case, prec):
        plan = load_plan(case)
        inputs, consts, _ = case_data(case, plan)
        exe = build_executable(case, prec, cuda_graphs=False, plan_json=plan, consts=consts)
        for static, x in zip(exe.static_inputs, inputs):
            static.copy_(torch.from_numpy(np.ascontiguousarray(x)))
        return exe

    out = {}
    pk, _ = peaks()
    for case, byts in (("bias_gelu_2048x3072", 50343936), ("layernorm_2048x768", 12589056),
                       ("softmax_12x512x512", 25165824)):
        exe = filled(case, "fp32")
        best, p50 = graph_times(exe.run_static)
        # cold: rotate through enough copies of the operands that nothing is left in the 126 MB L2
        n_sets = max(2, -(-2 * 126 * 2**20 // byts) + 1)
        sets = [exe] + [filled(case, "fp32") for _ in range(n_sets - 1)]

        def rotate():
            for e in sets:
                e.run_static()

        cold_best, cold_p50 = graph_times(rotate, repeats=2, replays=50)
        out[case] = {"warm_gbs": round(byts / best / 1e9, 1), "warm_p50_gbs": round(byts / p50 / 1e9, 1),
                     "cold_gbs": round(byts * n_sets / cold_best / 1e9, 1), "cold_p50_gbs": round(byts * n_sets / cold_p50 / 1e9, 1),
                     "frac_of_measured_hbm": round(byts * n_sets / cold_best / 1e9 / pk["hbm_gbs"], 3),
                     "buffer_sets": n_sets, "impl": exe.impls}
        for e in sets:
            e.close()
    from kiln_b200 import workloads as W
    mm_prec = precision if precision != "fp32" else "fp32"
    mm_peak = pk["bf16_tflops"] if mm_prec == "bf16" else (tf32_peak_tflops() if mm_prec == "tf32" else None)
    if mm_prec == "tf32":
        out["tf32_peak_tflops_measured"] = round(mm_peak, 1)
    for m, n, k in W.LINEAR_SHAPES:
        exe = filled(f"linear_{m}x{n}x{k}", mm_prec)
        best, p50 = graph_times(exe.run_static)
        row = {"tflops": round(2 * m * n * k / best / 1e12, 2), "p50_tflops": round(2 * m * n * k / p50 / 1e12, 2),
               "us": round(best * 1e6, 2), "precision": mm_prec, "impl": exe.impls}
        if mm_peak and m > 1:
            row["frac_of_measured_peak"] = round(row["tflops"] / mm_peak, 3)
        if m == 1:      # decode GEMV: weights streamed once; cold = weight sets rotated through more than twice the L2
            byts = 4 * k * n + 4 * n + 4 * k
            row["gbs"] = round(byts / best / 1e9, 1)
            n_sets = -(-2 * 126 * 2**20 // byts) + 1
            sets = [exe] + [filled(f"linear_{m}x{n}x{k}", mm_prec) for _ in range(n_sets - 1)]

            def rotate():
                for e in sets:
                    e.run_static()

            cold_best, _ = graph_times(rotate, repeats=2, replays=50)
            row["cold_gbs"] = round(byts * n_sets / cold_best / 1e9, 1)
            row["cold_frac_of_measured_hbm"] = round(byts * n_sets / cold_best / 1e9 / pk["hbm_gbs"], 3)
            for e in sets[1:]:
                e.close()
        out[f"linear_{m}x{n}x{k}"] = row
        exe.close()
    for t, seed in ((128, 0), (2048, 4)):
        direct, _ = build_block(precision, t, seed, cuda_graphs=False)
        kernel_best, kernel_p50 = graph_times(direct.run_static)
        direct.close()
        exe, _ = build_block(precision, t, seed)
        xd = torch.randn(t, D, device="cuda")
        call_ms = device_call_ms(lambda: exe(xd))
        x = torch.randn(t, D).pin_memory()
        for _ in range(5):
            exe(x)
        torch.cuda.synchronize()
        lat = []
        for _ in range(200):
            t0 = time.perf_counter()
            y = exe(x)[0]
            y.cpu()
            lat.append((time.perf_counter() - t0) * 1e3)
        out[f"block_t{t}"] = {"e2e_p50_ms": round(float(np.median(lat)), 4), "e2e_best_ms": round(float(np.min(lat)), 4),
                              "call_ms": round(call_ms, 4), "kernel_ms": round(kernel_best * 1e3, 4),
                              "kernel_p50_ms": round(kernel_p50 * 1e3, 4)}
        exe.close()
    return out


def reference_triton_extra(precision):
    """The reference's Triton backend on this GPU, in a process of its own (it registers the same
    module names this package does); its one JSON line, or why it could not run."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference-triton", "--autotune",
           "--precision", "fp32" if precision == "fp32" else "tf32"]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=420)
        for text in reversed(proc.stdout.strip().splitlines()):
            if text.startswith("{"):
                return json.loads(text)
        return {"impl": "reference-triton", "unavailable": (proc.stderr or "no output")[-200:]}
    except Exception as err:   # noqa: BLE001
        return {"impl": "reference-triton", "unavailable": f"{type(err).__name__}: {err}"[:200]}


def dtype_of(precision, impls):
    """The arithmetic the matmuls really ran in: the tensor-core kernels take tf32 / bf16 operands,
    every other kernel (and every accumulation) is float32."""
    if precision == "fp32" or not any(i == "mm_tcgen05" for i in impls):
        return "f32"
    return precision


def gpu_arm(args, dist, rank, world, local):
    from kiln_b200 import workloads as W

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    precision = args.precision
    host = [torch.from_numpy(W.block_input(SEED, TOKENS, index=rank * SEQS + i)).pin_memory() for i in range(SEQS)]
    dev_in = torch.stack([h.cuda(non_blocking=True) for h in host])
    dev_out = torch.empty_like(dev_in)
    host_out = [torch.empty(TOKENS, D).pin_memory() for _ in range(SEQS)]
    torch.cuda.synchronize()

    # INFLIGHT compiled modules (own arena, static buffers and stream each) run round-robin, as a server
    # keeps several requests in flight: kernels of one sequence fill the SMs another leaves idle, and
    # copies overlap kernels.  A whole step of 64 sequences is one CUDA graph (kiln_b200.runtime.
    # StreamedBatch), so a busy host does not starve the GPU of launches.
    from kiln_b200.runtime import StreamedBatch

    exe, plan = build_block(precision, TOKENS, SEED, cuda_graphs=False)
    exes = [exe] + [build_block(precision, TOKENS, SEED, cuda_graphs=False)[0] for _ in range(INFLIGHT - 1)]
    resident = StreamedBatch(exes).capture(list(dev_in), list(dev_out))
    step_resident = resident.run

    for _ in range(args.warmup):
        step_resident()
    with ClockSampler(local) as clocks:
        ms = time_region(dist, step_resident, args.steps)
    resident.status()
    # end to end: the same step with pinned host tensors as sources and sinks (201 MB each way per step)
    e2e = StreamedBatch(exes).capture(host, host_out)
    step_e2e = e2e.run
    for _ in range(max(1, args.warmup // 2)):
        step_e2e()
    ms_e2e = time_region(dist, step_e2e, args.steps)
    e2e.status()
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
                "modules_in_flight": INFLIGHT},
        "gpu_launches": world * args.steps * SEQS * exe.device_launches, "modules_in_flight": INFLIGHT,
        "clocks": clocks.summary(),
        "impls": dict(zip(exe.launch_names, exe.impls)),
    }
    line["roofline"] = roofline_of(exe, plan, precision)
    if world == 1:
        v, done, cores = cpu_block_tokens_per_s(seconds_budget=12.0)
        v1, done1, _ = cpu_block_tokens_per_s(seconds_budget=6.0, threads=1)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{done} of {SEQS} sequences x {TOKENS} tokens, eager PyTorch float32 (oneDNN)",
                                "one_thread": {"value": v1, "unit": UNIT, "cores": 1,
                                               "sample": f"{done1} sequences x {TOKENS} tokens"}}
        if not args.no_extras:
            try:
                line["extras"] = extras(precision)
                line["extras"]["reference_triton"] = reference_triton_extra(precision)
            except Exception as err:   # noqa: BLE001  (extras never invalidate the headline line)
                line["extras"] = {"error": f"{type(err).__name__}: {err}"[:200]}
    print(json.dumps(line), flush=True)


def single_case(args):
    """One stored plan, launched directly (no CUDA graph) so a profiler sees plain kernel launches."""
    from gpu_helpers import build_executable
    from helpers import case_data, load_plan

    plan = load_plan(args.case)
    inputs, consts, _ = case_data(args.case, plan)
    exe = build_executable(args.case, args.precision, cuda_graphs=False, plan_json=plan, consts=consts)
    for static, x in zip(exe.static_inputs, inputs):
        static.copy_(torch.from_numpy(np.ascontiguousarray(x)))
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
    print(json.dumps({"case": args.case, "precision": args.precision, "impls": exe.impls,
                      "ms_per_call": start.elapsed_time(end) / args.steps, "launches_per_call": exe.device_launches}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--autotune", action="store_true", help="reference-triton only: let the reference autotune its matmuls")
    ap.add_argument("--precision", default=os.environ.get("KB200_BENCH_PRECISION", "bf16"),
                    choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", default=None,
                    help="run one stored plan (a name under tests/golden/plans) --steps times and print its GPU "
                         "time per call; the small, single-kernel workload to put under a profiler")
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
        rank = int(os.environ.get("RANK", 0))
        reference_arm(args, None, rank)
        return
    dist, rank, world, local = dist_setup(args.gpus)
    try:
        gpu_arm(args, dist, rank, world, local)
    finally:
        if dist is not None:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
