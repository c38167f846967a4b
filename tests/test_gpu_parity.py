"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle and the golden
vectors the reference produced.  Tolerances: the reference's own assert_close(rtol=1e-4,
atol=1e-5) against eager PyTorch (tests/test_gpu.py:37 of the reference) and, against a float64
evaluation, max|err| / max|expected| <= 1e-5 (FP32), 2e-3 (TF32), 2e-2 (BF16)."""

import numpy as np
import pytest
import torch

from helpers import big_cases, small_cases, subsample
from oracle.plan_oracle import run_plan, scale_relative_error

pytestmark = pytest.mark.gpu

REL_TOL = {"fp32": 1e-5, "tf32": 2e-3, "bf16": 2e-2}


@pytest.fixture(autouse=True)
def private_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("KILN_CACHE_DIR", str(tmp_path))
    yield


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager-launch"])
@pytest.mark.parametrize("case", small_cases())
def test_small_cases_match_reference_vectors(case, graphs):
    from gpu_helpers import run_case

    exe, outs, (plan, inputs, consts, expected) = run_case(case, "fp32", cuda_graphs=graphs)
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for got, eager, ref64 in zip(outs, expected["out"], exact):
        np.testing.assert_allclose(got, eager, rtol=1e-4, atol=1e-5)
        assert scale_relative_error(got, ref64) <= REL_TOL["fp32"], (case, exe.impls)


@pytest.mark.parametrize("case", big_cases())
def test_benchmark_configs_fp32(case):
    from gpu_helpers import run_case

    exe, outs, (plan, inputs, consts, expected) = run_case(case, "fp32")
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for got, ref64, sub, step in zip(outs, exact, expected["sub"], expected["step"]):
        assert scale_relative_error(got, ref64) <= REL_TOL["fp32"], (case, exe.impls)
        # and directly against the stored float64 result of the reference's eager model
        assert scale_relative_error(subsample(got, step), sub) <= REL_TOL["fp32"], (case, exe.impls)


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("case", [c for c in big_cases() if c.startswith(("gpt2_block", "mlp_", "linear_"))]
                         + ["tf32_linear", "transformer_block", "bmm_transposed_operand", "odd_k", "wide_bmm",
                            "erf_gelu_mlp", "decode_m1"])
def test_reduced_precision_matmuls(case, precision):
    from gpu_helpers import run_case

    exe, outs, (plan, inputs, consts, expected) = run_case(case, precision)
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for got, ref64 in zip(outs, exact):
        assert scale_relative_error(got, ref64) <= REL_TOL[precision], (case, precision, exe.impls)


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
def test_every_kernel_of_the_block_matches_the_oracle_step_by_step(precision, monkeypatch):
    """Launch the block's 11 kernels one at a time and compare each kernel's output buffer
    (one launch per planned kernel: no fused attention, no folded operand copies here)."""
    from gpu_helpers import build_executable
    from helpers import case_data, load_plan

    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")
    monkeypatch.setenv("KILN_GPU_FOLD_COPIES", "0")
    monkeypatch.setenv("KILN_GPU_ABSORB_ELEMENTWISE", "0")
    monkeypatch.setenv("KILN_GPU_MIRROR_ONLY", "0")      # every planned buffer holds its float32 values

    case = "gpt2_block_t128"
    plan = load_plan(case)
    inputs, consts, _ = case_data(case, plan)
    exe = build_executable(case, precision, cuda_graphs=False, plan_json=plan, consts=consts)
    exe.static_inputs[0].copy_(torch.from_numpy(inputs[0]))
    _, per_kernel = run_plan(plan, inputs, consts, dtype=np.float64, trace=True)
    arena = exe.arena.view(torch.float32)
    errors = {}
    for i, (kernel, want) in enumerate(zip(plan["kernels"], per_kernel)):
        exe.launch_kernel(i)
        torch.cuda.synchronize()
        exe.status()
        for (_, where), ref in zip(kernel["outputs"], want):
            buf = arena if where["base"][0] == "arena" else exe.static_outputs[where["base"][1]].view(-1)
            got = torch.as_strided(buf, where["shape"], where["strides"], where["offset"]).cpu().numpy()
            errors[f"{kernel['name']}:{exe.impls[i]}"] = scale_relative_error(got, ref)
    # intermediate buffers (attention scores) carry the rounding of the kernels before them and are
    # normalised by their own scale; the end-to-end bound is REL_TOL, per kernel allow twice that
    limit = REL_TOL[precision] * (1 if precision == "fp32" else 2)
    bad = {k: v for k, v in errors.items() if not v <= limit}
    assert not bad, (bad, errors)


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
@pytest.mark.parametrize("tokens", [128, 512, 1024])
def test_fused_attention_equals_the_five_planned_kernels(tokens, precision, monkeypatch):
    """The fused attention kernel (tensor cores in TF32 / BF16 mode, float32 FMAs in FP32 mode) against
    the unfused plan on the same inputs, and both against float64."""
    from gpu_helpers import run_case

    case = f"gpt2_block_t{tokens}"
    fused_exe, fused, (plan, inputs, consts, _) = run_case(case, precision)
    assert "attention_fused" in fused_exe.impls and fused_exe.impls.count("fused_away") == 4
    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")
    plain_exe, plain, _ = run_case(case, precision)
    assert "attention_fused" not in plain_exe.impls
    assert fused_exe.device_launches < plain_exe.device_launches
    (exact,) = run_plan(plan, inputs, consts, dtype=np.float64)
    assert scale_relative_error(fused[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(plain[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(fused[0], plain[0]) <= REL_TOL[precision]


@pytest.mark.parametrize("kernel", ["fma", "tensor"])
@pytest.mark.parametrize("tokens", [128, 1024])
def test_both_fp32_attention_kernels_match_float64(tokens, kernel, monkeypatch):
    """FP32 mode picks the CUDA-core kernel for short sequences and the tensor-core kernel (three TF32
    MMAs per product) for long ones; each is forced here at both lengths."""
    from gpu_helpers import run_case

    monkeypatch.setenv("KILN_GPU_FP32_ATTENTION", kernel)
    case = f"gpt2_block_t{tokens}"
    exe, got, (plan, inputs, consts, _) = run_case(case, "fp32")
    assert "attention_fused" in exe.impls
    # the tensor-core kernel has a launch in front that writes the operands' tails
    monkeypatch.setenv("KILN_GPU_FP32_ATTENTION", "fma" if kernel == "tensor" else "tensor")
    other, _, _ = run_case(case, "fp32")
    assert abs(exe.device_launches - other.device_launches) == 1
    (exact,) = run_plan(plan, inputs, consts, dtype=np.float64)
    assert scale_relative_error(got[0], exact) <= REL_TOL["fp32"]


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
def test_query_tiles_shared_by_two_ctas_merge_to_the_same_rows(precision, monkeypatch):
    """One 1024-token sequence leaves SMs idle, so the long query tiles are worked on by two CTAs each
    and merged by the one that finishes second; replays must keep working (the arrival counters are
    reset by the merging CTA) and the rows must match the unsplit kernel's and float64."""
    from gpu_helpers import run_case

    case = "gpt2_block_t1024"
    split_exe, split, (plan, inputs, consts, _) = run_case(case, precision)
    x = torch.from_numpy(inputs[0])
    again = [split_exe(x)[0].cpu().numpy() for _ in range(3)]
    for other in again:
        assert np.array_equal(other, split[0])      # the merge is symmetric in the halves: the same bits whichever CTA arrives second
    monkeypatch.setenv("KILN_GPU_ATTENTION_SPLIT", "0")
    _, whole, _ = run_case(case, precision)
    (exact,) = run_plan(plan, inputs, consts, dtype=np.float64)
    assert scale_relative_error(split[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(whole[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(split[0], whole[0]) <= REL_TOL[precision]


def test_fp32_mode_fuses_attention_too(monkeypatch):
    """FP32 mode (the reference's allow_tf32=False) takes the CUDA-core fused kernel: the scores are never written."""
    from gpu_helpers import build_executable

    exe = build_executable("gpt2_block_t128", "fp32")
    assert "attention_fused" in exe.impls and exe.impls.count("fused_away") >= 4
    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")
    plain = build_executable("gpt2_block_t128", "fp32")
    assert "attention_fused" not in plain.impls and plain.device_launches > exe.device_launches


def test_replay_with_new_inputs():
    """One captured graph, three different inputs (tests/test_gpu.py:161-169 of the reference)."""
    from gpu_helpers import build_executable
    from helpers import case_data, load_plan

    plan = load_plan("block_d64")
    _, consts, _ = case_data("block_d64", plan)
    exe = build_executable("block_d64", plan_json=plan, consts=consts)
    rng = np.random.default_rng(5)
    for _ in range(3):
        x = rng.standard_normal((16, 64)).astype(np.float32)
        (got,) = exe(torch.from_numpy(x))
        (want,) = run_plan(plan, [x], consts, dtype=np.float64)
        assert scale_relative_error(got.cpu().numpy(), want) <= 1e-5
    assert exe.graph is not None


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("case", ["gpt2_block_t1024", "gpt2_block_t128", "mlp_2048"])
def test_second_mma_issuer_and_dependent_launch(case, precision, monkeypatch):
    """64-column tiles with two MMA issuers (opt-in, even ring), with and without programmatic dependent
    launch between kernels, against the float64 oracle."""
    from gpu_helpers import build_executable, run_case

    monkeypatch.setenv("KILN_GPU_DEPENDENT_LAUNCH", "0" if case == "mlp_2048" else "1")      # both launch orders
    names = [n for n in build_executable(case, precision).launch_names if "matmul" in n]
    exe, outs, (plan, inputs, consts, _) = run_case(
        case, precision, configs={n.split("_")[0]: {"BN": 64, "debug": 512, "impl": "tc"} for n in names})
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for got, ref64 in zip(outs, exact):
        assert scale_relative_error(got, ref64) <= REL_TOL[precision], (case, precision, exe.impls)


@pytest.mark.parametrize("config", [{}, {"split_k": 2}, {"split_k": 4, "BN": 64}, {"BN": 128}, {"debug": 1024}],
                         ids=["auto", "split2", "split4_bn64", "bn128", "cuda_cores"])
@pytest.mark.parametrize("case", ["gpt2_block_t128", "mlp_2048", "odd_k", "wide_bmm", "transformer_block",
                                  "bmm_transposed_operand", "linear_128x768x3072"])
def test_exact_fp32_matmuls_on_the_tensor_cores(case, config):
    """allow_tf32=False (tl.dot with input_precision="ieee", kiln/gpu/codegen.py:515): three TF32 products
    of operands split into head and tail, K steps spread over several accumulators, alone or with K
    shared over a cluster; and the CUDA-core kernel that config bit 1024 selects.  All within 1e-5 of
    float64."""
    from gpu_helpers import build_executable, run_case

    names = [n for n in build_executable(case, "fp32").launch_names if "matmul" in n]
    exe, outs, (plan, inputs, consts, _) = run_case(case, "fp32", configs={n.split("_")[0]: dict(config) for n in names})
    if config.get("debug") == 1024:
        assert "mm_tcgen05" not in exe.impls, exe.impls
    elif case in ("gpt2_block_t128", "mlp_2048", "linear_128x768x3072"):
        assert "mm_tcgen05" in exe.impls and "mm_simt_fp32" not in exe.impls, exe.impls
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for got, ref64 in zip(outs, exact):
        assert scale_relative_error(got, ref64) <= REL_TOL["fp32"], (case, config, exe.impls)


def test_infinite_matmul_operands_on_the_cuda_cores():
    """An infinite element of a matmul OPERAND has no finite head and tail, so the split-operand FP32 mode
    cannot carry it (it yields NaN); config bit 1024 selects the CUDA-core kernel, which multiplies as
    float32 does: the row that holds +inf comes out +inf, every other row as usual."""
    from kiln_b200.autotune import GPUAutotuner

    tuner = GPUAutotuner(allow_tf32=False, use_cache=False)
    gen = torch.Generator(device="cpu").manual_seed(3)
    a = torch.randn(128, 256, generator=gen)
    b = torch.rand(256, 192, generator=gen) + 0.5          # positive: inf * b stays +inf
    a[5, 17] = float("inf")
    exe = tuner._compile(1, 128, 192, 256, {"debug": 1024})
    (out,) = exe(a.cuda(), b.cuda())
    exe.status()
    out = out.cpu()
    assert "mm_tcgen05" not in exe.impls
    assert torch.isinf(out[5]).all() and (out[5] > 0).all()
    keep = [r for r in range(128) if r != 5]
    want = (a[keep].double() @ b.double()).float()
    assert torch.isfinite(out[keep]).all()
    assert (out[keep] - want).abs().max().item() <= 1e-5 * want.abs().max().item()
    split = tuner._compile(1, 128, 192, 256, {})
    (other,) = split(a.cuda(), b.cuda())
    split.status()
    assert "mm_tcgen05" in split.impls and torch.isfinite(other.cpu()[keep]).all()
    assert (other.cpu()[keep] - want).abs().max().item() <= 1e-5 * want.abs().max().item()


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16"])
@pytest.mark.parametrize("case", ["unfrozen_linear", "gpt2_block_t128", "transformer_block", "bmm_transposed_operand", "block_d64"])
def test_folded_operand_copies_change_nothing(case, precision, monkeypatch):
    """A matmul that reads its B operand at the source of the plan's transposing copy, against the same
    plan with the copy launched, and against float64."""
    from gpu_helpers import run_case

    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")
    folded_exe, folded, (plan, inputs, consts, _) = run_case(case, precision)
    monkeypatch.setenv("KILN_GPU_FOLD_COPIES", "0")
    plain_exe, plain, _ = run_case(case, precision)
    assert "fused_away" not in plain_exe.impls and folded_exe.device_launches <= plain_exe.device_launches
    if case in ("unfrozen_linear", "gpt2_block_t128", "transformer_block", "block_d64"):
        assert "fused_away" in folded_exe.impls, folded_exe.impls
    exact = run_plan(plan, inputs, consts, dtype=np.float64)
    for a, b, ref64 in zip(folded, plain, exact):
        assert scale_relative_error(a, ref64) <= REL_TOL[precision]
        assert scale_relative_error(a, b) <= REL_TOL[precision]


def test_streamed_batch_equals_one_call_per_request():
    """Seven requests through three modules in flight, the step captured as one CUDA graph, device and
    pinned-host tensors as sources and sinks: the same bits as one __call__ per request."""
    from gpu_helpers import build_executable
    from kiln_b200 import workloads as W
    from kiln_b200.runtime import StreamedBatch

    case = "gpt2_block_t128"
    xs = [torch.from_numpy(W.block_input(0, 128, index=i)) for i in range(7)]
    single = build_executable(case, "tf32")
    want = [single(x)[0].cpu() for x in xs]
    batch = StreamedBatch([build_executable(case, "tf32", cuda_graphs=False) for _ in range(3)])
    with pytest.raises(ValueError):
        batch.capture(xs, [torch.empty_like(x) for x in xs])          # pageable host memory
    dev_in, dev_out = [x.cuda() for x in xs], [torch.empty(128, 768, device="cuda") for _ in xs]
    batch.capture(dev_in, dev_out).run()
    torch.cuda.synchronize()
    batch.status()
    for got, ref in zip(dev_out, want):
        assert torch.equal(got.cpu(), ref)
    host_in, host_out = [x.pin_memory() for x in xs], [torch.empty(128, 768).pin_memory() for _ in xs]
    batch.capture(host_in, host_out)
    for _ in range(2):
        batch.run()
    torch.cuda.synchronize()
    for got, ref in zip(host_out, want):
        assert torch.equal(got, ref)
    with pytest.raises(ValueError):
        StreamedBatch([single])                                       # modules that replay their own graph


def test_wrong_shape_and_memory_errors(monkeypatch):
    from gpu_helpers import build_executable
    from kiln_b200.runtime import check_memory

    exe = build_executable("layernorm")
    with pytest.raises(ValueError, match="compiled for input shape"):
        exe(torch.zeros(3, 3))
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (10 * 2**20, 32 * 2**30))
    with pytest.raises(MemoryError, match="only 10.0 MiB"):
        check_memory(torch.device("cuda"), 64 * 2**20, "the arena")
    with pytest.raises(MemoryError):
        build_executable("gpt2_block_t128")


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("case", ["gpt2_block_t128", "odd_k", "wide_bmm", "tf32_linear", "transformer_block", "erf_gelu_mlp"])
def test_bulk_tensor_stores_equal_plain_stores(case, precision, monkeypatch):
    """The tensor-core matmul's epilogue writes through bulk tensor stores where the output allows it
    and through ordinary stores otherwise: the same arithmetic, so the same bits."""
    from gpu_helpers import build_executable, run_case

    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")   # keep every planned matmul on the GPU's kernel list
    names = [n for n in build_executable(case, precision).launch_names if "matmul" in n]
    _, bulk, _ = run_case(case, precision)
    for stores in ("plain", "bulk_columns"):     # "auto" keeps a lane per row where the chain allows it
        _, other, _ = run_case(case, precision, configs={n.split("_")[0]: {"stores": stores} for n in names})
        for a, b in zip(bulk, other):
            assert np.array_equal(a, b), (case, precision, stores)


def test_hot_path_kernels_are_the_specialised_ones(monkeypatch):
    from gpu_helpers import build_executable

    monkeypatch.setenv("KILN_GPU_FUSE_ATTENTION", "0")   # the five planned attention kernels, each on its own
    exe = build_executable("gpt2_block_t128")
    by_name = dict(zip(exe.launch_names, exe.impls))
    assert by_name["k0_row"] == "row_layernorm" and by_name["k8_row"] == "row_layernorm"
    assert by_name["k4_row"] == "row_softmax"
    # the K^T copy feeds only the score matmul, which reads K where it lies instead
    assert by_name["k2_ew0"] == "fused_away" and by_name["k6_ew0"] == "ew_chain_vec4"
    assert exe.device_launches == 10
    monkeypatch.setenv("KILN_GPU_FOLD_COPIES", "0")
    unfolded = build_executable("gpt2_block_t128")
    assert dict(zip(unfolded.launch_names, unfolded.impls))["k2_ew0"] == "ew_transpose" and unfolded.device_launches == 11
    monkeypatch.delenv("KILN_GPU_FOLD_COPIES")
    assert build_executable("bias_gelu_2048x3072").impls == ["ew_chain_vec4"]
    assert build_executable("linear_1x3072x768").impls == ["mm_gemv"]


def test_autotune_candidates_fit_shared_memory():
    from kiln_b200.autotune import SHARED_MEMORY_BYTES, SINGLE_CTA_EPILOGUE_BYTES, candidates, stage_bytes

    for m, n, k in [(128, 3072, 768), (1, 768, 768), (7, 13, 5), (2048, 3072, 768)]:
        cands = candidates(m, n, k)
        assert cands and cands[-1]["impl"] == "simt"
        assert any(c["BM"] == 256 for c in cands) == (m > 128 and n >= 128)      # SM-pair tiles only above 128 rows
        for c in cands[:-1]:
            if c["BM"] == 256:        # the pair kernel fits its ring to what is left beside its staging slots
                assert c["BN"] in (128, 256) and 2 * stage_bytes(c) + 8 * 2 * 6144 + 1024 <= SHARED_MEMORY_BYTES
            else:
                assert stage_bytes(c) * c["stages"] + SINGLE_CTA_EPILOGUE_BYTES + 1024 <= SHARED_MEMORY_BYTES
            assert c["BN"] <= max(64, 2 * n)


def test_autotuner_is_correct_then_cached(monkeypatch):
    """Tuned once, then served from the on-disk cache (tests/test_gpu.py:143-158 of the reference)."""
    from kiln_b200.autotune import GPUAutotuner
    from kiln_b200.codegen import default_matmul_config

    default = default_matmul_config(None, None)
    first = GPUAutotuner(allow_tf32=True)
    cfg = first.config_for_shape(1, 256, 768, 512, default)
    (entry,) = first.log
    assert entry["source"] == "tuned" and entry["candidates"] >= 2 and entry["tflops"] > 0
    assert entry["shape"] == (1, 256, 768, 512)
    monkeypatch.setattr(GPUAutotuner, "tune", lambda *a, **k: pytest.fail("cached shape re-tuned"))
    second = GPUAutotuner(allow_tf32=True)
    assert second.config_for_shape(1, 256, 768, 512, default) == cfg
    assert second.log[0]["source"] == "cache"
    exact = GPUAutotuner(allow_tf32=False, use_cache=False)
    monkeypatch.undo()
    exact.config_for_shape(1, 64, 96, 80, default)
    assert exact.log[0]["config"].get("impl") in ("auto", "simt", "tc")
    # exact FP32 searches the tensor-core configurations too, and they win where there is work to share
    exact.config_for_shape(1, 128, 768, 768, default)
    assert exact.log[1]["candidates"] >= 3 and exact.log[1]["config"].get("impl") != "simt", exact.log[1]


def test_nine_reductions_at_one_level_are_refused_not_dropped():
    """The generic row kernel keeps eight running reductions per pass; a ninth must be a clear
    NotImplementedError at bind time, never a silently missing term."""
    from kiln_b200.codegen import program_from_plan
    from kiln_b200.runtime import GPUExecutable
    from kiln_b200.spec import KernelSpec, NodeSpec, OperandSpec, PlanSpec

    rows, cols = 4, 24

    def plan_with(n_reductions):
        nodes = [NodeSpec("mul", [("operand", 0), ("scalar", float(i + 1))], (rows, cols)) for i in range(n_reductions)]
        nodes += [NodeSpec("reduce_sum", [("node", i)], (rows, 1), {"dims": [1], "keepdim": True}) for i in range(n_reductions)]
        acc = n_reductions
        for i in range(1, n_reductions):
            nodes.append(NodeSpec("add", [("node", acc), ("node", n_reductions + i)], (rows, 1)))
            acc = len(nodes) - 1
        kernel = KernelSpec("k0", "reduction", nodes, [OperandSpec(("input", 0), 0, (rows, cols), (cols, 1))],
                            [(acc, OperandSpec(("output", 0), 0, (rows, 1), (1, 1)))])
        return PlanSpec("many_reductions", [(rows, cols)], [(rows, 1)], 0, {}, [kernel])

    x = torch.randn(rows, cols)
    ok = plan_with(8)
    exe = GPUExecutable(program_from_plan(ok, "fp32"), 0, {}, ok.input_shapes, ok.output_shapes, cuda_graphs=False)
    (got,) = exe(x)
    want = sum((i + 1) * x.double().sum(1, keepdim=True) for i in range(8))
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-5, atol=1e-5)
    too_many = plan_with(9)
    with pytest.raises(NotImplementedError, match="reductions at one level"):
        GPUExecutable(program_from_plan(too_many, "fp32"), 0, {}, too_many.input_shapes, too_many.output_shapes, cuda_graphs=False)


def test_a_wait_that_runs_out_is_reported_and_the_plan_stays_usable():
    """Failure detection on the device without faulting it: a wait that nothing can satisfy gives up
    after its limit, the status word names it, and the same plan then runs correctly."""
    import ctypes as C

    from gpu_helpers import run_case
    from kiln_b200 import _cabi

    lib = _cabi.load()
    exe, outs, (plan, inputs, consts, expected) = run_case("mlp", "fp32", cuda_graphs=False)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.kb200_plan_selftest_wait(exe._plan, stream) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded device-side wait ran out.*kernel 65535, site 127"):
        exe.status()
    exe.status()                      # reading the word cleared it
    again = exe(*[torch.from_numpy(np.ascontiguousarray(x)) for x in inputs])
    torch.cuda.synchronize()
    exe.status()
    np.testing.assert_allclose(again[0].cpu().numpy(), outs[0], rtol=0, atol=0)
    np.testing.assert_allclose(again[0].cpu().numpy(), expected["out"][0], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_the_benchmark_s_eight_sequence_graph_matches_the_stored_eager_result(precision):
    """[8, 1024, 768] through the stored plan of the benchmark step: 8192-row matmuls on SM pairs, the
    attention chain of a batched graph fused; against the float64 eager result stored with the plan."""
    from gpu_helpers import run_case

    case = "gpt2_block_b8_t1024"
    exe, outs, (plan, inputs, consts, expected) = run_case(case, precision)
    # six kernels of the attention chain, the GELU and the last residual add launch nothing of their own
    assert "attention_fused" in exe.impls and exe.impls.count("fused_away") == 8
    got = subsample(outs[0], expected["step"][0])
    assert scale_relative_error(got, expected["sub"][0]) <= REL_TOL[precision], (precision, exe.impls)


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_batched_block_with_and_without_cross_kernel_fusion(precision, monkeypatch):
    """The batched block: activation and residual add in the matmuls' epilogues and (BF16) intermediates
    stored as bf16 only, against one launch per planned kernel with every float32 buffer written."""
    from gpu_helpers import run_case

    fused_exe, fused, (plan, inputs, consts, _) = run_case("batched_block", precision)
    names = dict(zip(fused_exe.launch_names, fused_exe.impls))
    absorbed = [n for n, impl in names.items() if "_ew" in n and impl == "fused_away"]
    assert len(absorbed) == 2, names
    monkeypatch.setenv("KILN_GPU_ABSORB_ELEMENTWISE", "0")
    monkeypatch.setenv("KILN_GPU_MIRROR_ONLY", "0")
    plain_exe, plain, _ = run_case("batched_block", precision)
    assert plain_exe.device_launches >= fused_exe.device_launches + 2   # and a bf16 conversion pass behind an elementwise producer
    (exact,) = run_plan(plan, inputs, consts, dtype=np.float64)
    assert scale_relative_error(fused[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(plain[0], exact) <= REL_TOL[precision]
    assert scale_relative_error(fused[0], plain[0]) <= REL_TOL[precision]
