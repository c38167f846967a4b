"""GPU runtime (stands in for kiln.gpu.runtime): owns device memory, binds it to the
kernel library's launch plan, captures the launch sequence as one CUDA graph and replays it.

Same contract as the reference's GPUExecutable (kiln/gpu/runtime.py:135-217):

  * one arena holding every intermediate at the planner's offsets, allocated once;
  * frozen constants uploaded once, only those some launch reads (runtime.py:146-154);
  * a MemoryError with the sizes involved before anything is allocated (runtime.py:82-90);
  * ``__call__(*tensors)`` checks shapes (ValueError), coerces inputs to contiguous float32
    on the device, and returns fresh float32 tensors that do not alias internal buffers;
  * not re-entrant: calls share the arena.

The kernels are the hand-written sm_100a ones in libkb200.so, reached through the C ABI of
include/kb200.h with raw device pointers; PyTorch only provides memory, streams and graphs.
There is no CPU path: without a CUDA device or without the library, construction raises.
"""

from __future__ import annotations

import ctypes as C
import hashlib
import os
import time
from pathlib import Path

import numpy as np
import torch

from kiln_b200 import _cabi, lowering


def interpreting() -> bool:
    """The reference can run its kernels under Triton's CPU interpreter; this backend cannot."""
    return False


def device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("Kiln's B200 GPU backend needs a CUDA GPU (sm_100a); there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def cache_dir() -> Path:
    base = os.environ.get("KILN_CACHE_DIR") or os.path.join(Path.home(), ".cache", "kiln")
    return Path(base) / "b200"


class PlanDump:
    """The readable plan dump that ``Report.lowering['source']`` points at, stored under the cache
    directory by content hash (what kiln/gpu/runtime.py:58-79 does for generated Triton source;
    here nothing is imported from the file, it is for people and for the reference's tests)."""

    def __init__(self, text: str):
        self.text = text
        self.path = cache_dir() / ("plan_" + hashlib.sha256(text.encode()).hexdigest()[:16] + ".txt")

    def stored(self) -> bool:
        try:
            return self.path.read_text() == self.text
        except OSError:
            return False

    def store(self) -> Path:
        """Write-then-rename, so a concurrent reader never sees half a file; a damaged copy is replaced."""
        if self.stored():
            return self.path
        self.path.parent.mkdir(parents=True, exist_ok=True)
        scratch = self.path.with_name(f"{self.path.name}.{os.getpid()}.part")
        with open(scratch, "w") as out:
            out.write(self.text)
            out.flush()
            os.fsync(out.fileno())
        os.replace(scratch, self.path)
        return self.path


def write_source(source: str) -> Path:
    return PlanDump(source).store()


def _mib(n_bytes) -> str:
    return f"{n_bytes / 2**20:.1f} MiB"


def check_memory(dev, needed_bytes, what):
    """MemoryError naming the sizes involved when ``needed_bytes`` exceed the device's free memory
    (same message as kiln/gpu/runtime.py:82-90, which the reference's tests match on)."""
    if torch.device(dev).type != "cuda":
        return
    free_bytes, total_bytes = torch.cuda.mem_get_info(dev)
    if needed_bytes <= free_bytes:
        return
    raise MemoryError(f"Kiln needs {_mib(needed_bytes)} of GPU memory for {what}, but only {_mib(free_bytes)} of "
                      f"{_mib(total_bytes)} is free (other processes may be using the GPU). Try a smaller batch or "
                      f"sequence length, or free GPU memory.")


class GraphTimer:
    """GPU time of a callable without the host's launch overhead: ``repeats`` back-to-back calls are
    captured in one CUDA graph (after a warm-up on a side stream, which also loads every kernel) and
    whole replays are timed with CUDA events.  Role of kiln/gpu/runtime.py:93-132."""

    def __init__(self, fn, repeats=20, warmup_calls=3):
        device()
        self.repeats = repeats
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup_calls):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            for _ in range(repeats):
                fn()
        self.graph.replay()                      # first replay: instantiation, not measured
        torch.cuda.synchronize()
        self._begin = torch.cuda.Event(enable_timing=True)
        self._end = torch.cuda.Event(enable_timing=True)

    def sample(self) -> float:
        """Seconds per call over one replay."""
        self._begin.record()
        self.graph.replay()
        self._end.record()
        torch.cuda.synchronize()
        return self._begin.elapsed_time(self._end) * 1e-3 / self.repeats

    def samples(self, n):
        return [self.sample() for _ in range(n)]


def kernel_seconds(fn, repeats=20, rounds=5):
    """Best-of-``rounds`` GPU seconds per call of ``fn`` (see GraphTimer)."""
    return min(GraphTimer(fn, repeats).samples(rounds))


def _ptr_array(tensors):
    n = len(tensors)
    ptrs = (C.c_void_p * max(n, 1))(*[t.data_ptr() for t in tensors])
    sizes = (C.c_uint64 * max(n, 1))(*[t.numel() * t.element_size() for t in tensors])
    return ptrs, sizes, n


class GPUExecutable:
    """Runs one compiled graph on the GPU. Not reentrant: calls share one arena."""

    def __init__(self, program, arena_bytes, constants, input_shapes, output_shapes, cuda_graphs=True):
        self.device = device()
        self.program = program
        self.source_path = PlanDump(program.source).store()
        self.input_shapes = [tuple(s) for s in input_shapes]
        self.output_shapes = [tuple(s) for s in output_shapes]
        self._lib = _cabi.load()
        self._plan = C.c_void_p()

        used = sorted({key[1] for launch in program.launches for key in launch.bases if key[0] == "const"})
        const_bytes = sum(int(np.prod(constants[name].shape)) * 4 for name in used)
        io_bytes = sum(4 * int(np.prod(s)) for s in self.input_shapes + self.output_shapes)
        out_bytes = sum(4 * int(np.prod(s)) for s in self.output_shapes)
        # what the library allocates itself when buffers are bound, in BF16 mode: a bf16 mirror of the
        # arena, packed bf16 copies of the constant matmul operands, and (worst case) bf16 copies of
        # unmirrored activations no larger than the inputs and the arena together
        library_bytes = 0
        if program.precision == "bf16":
            library_bytes = arena_bytes // 2 + 256 + const_bytes // 2 + (io_bytes + arena_bytes) // 2
        elif program.precision == "fp32":
            # the fused attention's scratch: the tails of Q, K and V (a copy of part of the arena) or the
            # split tiles' partial results (smaller than the merged heads)
            library_bytes = arena_bytes
        check_memory(self.device, arena_bytes + const_bytes + io_bytes + out_bytes + library_bytes,
                     f"the arena ({arena_bytes / 2**20:.1f} MiB), weights ({const_bytes / 2**20:.1f} MiB) "
                     f"and outputs")
        self.arena = torch.empty(max(arena_bytes, 4), dtype=torch.uint8, device=self.device)
        self.const_names = used
        self.constants = {name: torch.from_numpy(np.ascontiguousarray(constants[name], np.float32)).to(self.device)
                          for name in used}
        self.arena_bytes = arena_bytes
        self.weight_bytes = const_bytes
        # Static input / output buffers: the plan is bound to fixed addresses once, which is what
        # lets the whole launch sequence be one CUDA graph (kiln/gpu/runtime.py:191-204).
        self.static_inputs = [torch.zeros(max(int(np.prod(s)), 1), device=self.device).view(-1)[:int(np.prod(s))].view(s)
                              if int(np.prod(s)) else torch.zeros(s, device=self.device) for s in self.input_shapes]
        self.static_outputs = [torch.empty(s, device=self.device) for s in self.output_shapes]

        descs = lowering.lower(program.plan, program.launches, program.precision, self.const_names)
        self._descs = descs
        _cabi.check(self._lib.kb200_plan_create(descs, len(program.launches), self.device.index,
                                                C.byref(self._plan)), self._lib)
        # One launch per planned kernel (KILN_GPU_FUSE_ATTENTION=0), or let the library run the
        # attention chain as one fused kernel in the reduced-precision modes (default).
        fuse = os.environ.get("KILN_GPU_FUSE_ATTENTION", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_FUSE_ATTENTION, int(fuse)), self._lib)
        # Programmatic dependent launch between the plan's kernels (KILN_GPU_DEPENDENT_LAUNCH=0: plain stream order).
        pdl = os.environ.get("KILN_GPU_DEPENDENT_LAUNCH", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_DEPENDENT_LAUNCH, int(pdl)), self._lib)
        # One launch per planned kernel also for the copies that only transpose a matmul operand
        # (KILN_GPU_FOLD_COPIES=0); by default the matmul reads the copy's source and the copy is skipped.
        fold = os.environ.get("KILN_GPU_FOLD_COPIES", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_FOLD_OPERAND_COPIES, int(fold)), self._lib)
        # An elementwise kernel that only continues the matmul in front of it runs in that matmul's epilogue
        # (KILN_GPU_ABSORB_ELEMENTWISE=0: one launch per planned kernel); in BF16 mode an intermediate that
        # only bf16 readers consume is not stored as float32 (KILN_GPU_MIRROR_ONLY=0: every planned buffer
        # holds its float32 values, for a caller that looks at intermediates).
        absorb = os.environ.get("KILN_GPU_ABSORB_ELEMENTWISE", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_ABSORB_ELEMENTWISE, int(absorb)), self._lib)
        mirror_only = os.environ.get("KILN_GPU_MIRROR_ONLY", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_MIRROR_ONLY, int(mirror_only)), self._lib)
        # FP32 mode's fused attention: KILN_GPU_FP32_ATTENTION=fma / tensor forces the CUDA-core or the
        # tensor-core kernel (default: by size); KILN_GPU_ATTENTION_SPLIT=0 keeps every query tile on one CTA.
        fp32_attention = {"fma": 1, "tensor": 2}.get(os.environ.get("KILN_GPU_FP32_ATTENTION", "").lower(), 0)
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_FP32_ATTENTION, fp32_attention), self._lib)
        split = os.environ.get("KILN_GPU_ATTENTION_SPLIT", "1") not in ("0", "false", "False", "")
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_ATTENTION_SPLIT, int(split)), self._lib)
        self._bind()
        # launch_names: one per device launch of the plan (k3_matmul, k2_ew0 ...); kernel_names: the Kiln
        # kernels they come from, which is what CompiledModule.profile keys on (kiln/api.py:204-211)
        self.launch_names = [l.name for l in program.launches]
        self.kernel_names = list(dict.fromkeys(l.kernel for l in program.launches))
        self.impls = [self._lib.kb200_kernel_impl(self._plan, i).decode() for i in range(len(program.launches))]
        # fused scalar steps per element of every launch as bound (a matmul that took over the kernel behind it shows more)
        self.chain_lengths = [self._lib.kb200_kernel_chain_length(self._plan, i) for i in range(len(program.launches))]
        self.device_launches = self._lib.kb200_plan_launch_count(self._plan)
        self.graph = None
        self.use_cuda_graphs = bool(cuda_graphs)

    # -- binding and launching ------------------------------------------------------------

    def _bind(self):
        consts = [self.constants[n] for n in self.const_names]
        cp, cs, cn = _ptr_array(consts)
        ip, is_, in_ = _ptr_array(self.static_inputs)
        op, os_, on = _ptr_array(self.static_outputs)
        with torch.cuda.device(self.device):
            _cabi.check(self._lib.kb200_plan_bind(self._plan, self.arena.data_ptr(), self.arena.numel(),
                                                  cp, cs, cn, ip, is_, in_, op, os_, on), self._lib)

    def set_concurrency(self, plans_in_flight):
        """Tell the library how many plans share the GPU at once (a hint for its tile heuristics:
        each matmul then counts on its share of the SMs and prefers fewer, wider tiles); re-binds."""
        _cabi.check(self._lib.kb200_plan_set_option(self._plan, _cabi.OPT_CONCURRENCY, int(plans_in_flight)), self._lib)
        self._bind()
        self.graph = None

    def _launch(self):
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self._lib.kb200_plan_launch(self._plan, C.c_void_p(stream)), self._lib)

    def launch_kernel(self, i):
        """Enqueue launch ``i`` alone on the current stream (profiling, autotuning)."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self._lib.kb200_kernel_launch(self._plan, i, C.c_void_p(stream)), self._lib)

    def status(self):
        """Raises if a bounded device-side wait ran out since the last check."""
        _cabi.check(self._lib.kb200_plan_status(self._plan), self._lib)

    def _prepare(self, inputs):
        if len(inputs) != len(self.input_shapes):
            raise TypeError(f"expected {len(self.input_shapes)} inputs, got {len(inputs)}")
        out = []
        for t, shape in zip(inputs, self.input_shapes):
            if tuple(t.shape) != shape:
                raise ValueError(f"Kiln was compiled for input shape {shape}, got {tuple(t.shape)}")
            out.append(t.detach())
        return out

    def _capture(self):
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):          # warm up: loads every kernel before capture
            self._launch()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._launch()
        self.graph = graph

    def run_static(self):
        """Run on whatever the static input buffers hold; results land in ``static_outputs``."""
        if self.use_cuda_graphs:
            if self.graph is None:
                self._capture()
            self.graph.replay()
        else:
            self._launch()

    def __call__(self, *inputs):
        inputs = self._prepare(inputs)
        with torch.cuda.device(self.device):
            for static, t in zip(self.static_inputs, inputs):
                static.copy_(t, non_blocking=True)       # converts dtype / device / layout as needed
            self.run_static()
            return [o.clone() for o in self.static_outputs]

    def profile_launches(self, *inputs, iters=20):
        """[(launch name, milliseconds)] for every launch of the plan, in order.

        Each launch is timed on its own as GPU time: ``iters`` back-to-back launches of it captured
        in one CUDA graph and the replay timed with CUDA events (a launch takes microseconds, less
        than the host needs to enqueue it).  Launches are idempotent -- no kernel writes a buffer it
        reads -- so repeating one does not disturb the others' inputs.  A launch that a fused kernel
        covers (implementation ``fused_away``) enqueues nothing and is reported as 0.
        """
        inputs = self._prepare(inputs)
        with torch.cuda.device(self.device):
            for static, t in zip(self.static_inputs, inputs):
                static.copy_(t)
            self._launch()
            torch.cuda.synchronize(self.device)
            out = []
            for i, name in enumerate(self.launch_names):
                if self.impls[i] == "fused_away":
                    out.append((name, 0.0))
                    continue
                seconds = kernel_seconds(lambda i=i: self.launch_kernel(i), repeats=iters, rounds=3)
                out.append((name, seconds * 1e3))
        return out

    def profile(self, *inputs, iters=20):
        """[(Kiln kernel name, milliseconds)], the form ``CompiledModule.profile`` expects
        (kiln/api.py:204-211): the launches of one kernel (one per output of an elementwise kernel)
        are summed; the fused attention is booked on the kernel that launches it."""
        by_kernel = dict.fromkeys(self.kernel_names, 0.0)
        for launch, (_, ms) in zip(self.program.launches, self.profile_launches(*inputs, iters=iters)):
            by_kernel[launch.kernel] += ms
        return list(by_kernel.items())

    def close(self):
        if getattr(self, "_plan", None) is not None and self._plan:
            self._lib.kb200_plan_destroy(self._plan)
            self._plan = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001  (interpreter shutdown)
            pass


class StreamedBatch:
    """Many independent requests through copies of one compiled module, as ONE CUDA graph.

    A server that keeps several requests in flight gives each its own module (arena, weights'
    tensor maps, static buffers) and stream, so that kernels of one request fill the SMs another
    leaves idle and copies overlap kernels.  Enqueueing that from Python costs three calls per
    request; under a busy host the GPU then waits for the launches.  Here the whole step -- for
    request ``i``: copy ``sources[i]`` into module ``i % in_flight``'s input, run its kernels, copy
    its output to ``sinks[i]`` -- is captured once, across ``in_flight`` streams, and replayed with
    a single launch.  ``sources`` / ``sinks`` may be device tensors or pinned host tensors (the
    copies are then host<->device copies inside the graph); their addresses are part of the graph,
    so a caller refills the same tensors for the next step.

    The reference has no counterpart: its executable replays one graph per call
    (kiln/gpu/runtime.py:181-217).
    """

    def __init__(self, executables, concurrency=None):
        """``concurrency``: what the plans are told about how many of them share the GPU (default: their
        number; 1 when every kernel of a module is large enough for the whole GPU by itself)."""
        if not executables:
            raise ValueError("StreamedBatch needs at least one executable")
        for e in executables:
            if e.use_cuda_graphs:
                raise ValueError("StreamedBatch captures the launches itself: build the executables with cuda_graphs=False")
        self.executables = list(executables)
        for e in self.executables:
            e.set_concurrency(len(self.executables) if concurrency is None else concurrency)
        self.device = executables[0].device
        self.streams = [torch.cuda.Stream(device=self.device) for _ in executables]
        self.graph = None
        self.requests = 0

    def _enqueue(self, sources, sinks, kernels=True):
        cur = torch.cuda.current_stream(self.device)
        for st in self.streams:
            st.wait_stream(cur)
        n = len(self.executables)
        for i, (src, dst) in enumerate(zip(sources, sinks)):
            exe = self.executables[i % n]
            with torch.cuda.stream(self.streams[i % n]):
                exe.static_inputs[0].copy_(src, non_blocking=True)
                if kernels:
                    exe.run_static()
                dst.copy_(exe.static_outputs[0], non_blocking=True)
        for st in self.streams:
            cur.wait_stream(st)

    def capture(self, sources, sinks, kernels=True):
        """Capture one step over these tensors (single-input, single-output modules).  With
        ``kernels=False`` only the copies in and out are captured: the same traffic over the host
        link with no compute, which tells how much of an end-to-end step is the link's."""
        if len(sources) != len(sinks):
            raise ValueError("one sink per source")
        for t in list(sources) + list(sinks):
            if not t.is_cuda and not t.is_pinned():
                raise ValueError("host tensors of a StreamedBatch must be pinned")
        with torch.cuda.device(self.device):
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._enqueue(sources, sinks, kernels)          # warm-up outside capture (lazy initialisation)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._enqueue(sources, sinks, kernels)
        self.graph = graph
        self.requests = len(sources)
        return self

    def capture_launch(self, index, requests):
        """Capture ``requests`` launches of plan launch ``index`` alone, spread over the modules and
        their streams exactly like the launches of a whole step (profiling: what one kernel of the
        step costs when the modules in flight share the GPU, rather than alone on it)."""
        def enqueue():
            cur = torch.cuda.current_stream(self.device)
            for st in self.streams:
                st.wait_stream(cur)
            n = len(self.executables)
            for i in range(requests):
                with torch.cuda.stream(self.streams[i % n]):
                    self.executables[i % n].launch_kernel(index)
            for st in self.streams:
                cur.wait_stream(st)

        with torch.cuda.device(self.device):
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                enqueue()
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                enqueue()
        self.graph = graph
        self.requests = requests
        return self

    def run(self):
        """Replay the captured step on the current stream (one launch)."""
        if self.graph is None:
            raise RuntimeError("StreamedBatch.run before capture")
        self.graph.replay()

    def status(self):
        for e in self.executables:
            e.status()

    def close(self):
        self.graph = None
        for e in self.executables:
            e.close()
