"""``run_fused_rpa``: the CUDA-backend counterpart of the reference's RPA runner
(src/tpu_cake/rpa_runner.py:125-459) and of its device entry point
(src/tpu_cake/rpa_device_main.py:47-159).

Same sequence and evidence as the reference: the predeclared protocol (seed 97, 5 warm-up and 50
measured calls, :82-98), a single-use output directory, ``invocation.json``, ``profiler_config.json``,
the source state, a ledger that moves CREATED -> VERIFIED -> LOWERED -> COMPILED -> CORRECT ->
TIMED / TRACED / COUNTERED (or REJECTED), ``experiment.json``, the physical IR text, the lowered
source, the host-side preflight of the decode metadata, the correctness gate -- output within
``allclose(0.02, 0.02)`` of the expected result AND the updated cache bit-exact (:113-122,298-317) --
fresh device copies of every input for every call, because the cache is updated in place
(:328-343), per-call wall times with a synchronisation after each, the arrays, and ``result.json``.
The compile artifacts of the reference (StableHLO, compiler HLO) are replaced by the kernel
manifest of libcake_b200.so.

The expected result is computed here, in numpy, from the operation's definition
(src/tpu_cake/workloads/inkling_rpa.py:471-589): it is the run's correctness gate, as in the
reference, and never a substitute for the device result.
"""

from __future__ import annotations

import json
import math
import re
import socket
import statistics
import time
from dataclasses import asdict, dataclass, replace
from pathlib import Path

import numpy as np
import torch

from . import _native, ir, rpa_cuda_lowering, run_artifacts, workloads
from .identity import array_sha256, semantic_sha256
from .run_artifacts import ArtifactReference, RunMode
from .run_ledger import RunLedger, RunState

OUTPUT_ATOL = 0.02
OUTPUT_RTOL = 0.02
RPA_KERNELS = ("cake_rpa_plan_sm100", "cake_rpa_cache_update_sm100", "cake_rpa_decode_sm100", "cake_rpa_combine_sm100")


@dataclass(frozen=True)
class FusedRpaRunResult:
    run_id: str
    mode: str
    backend: str
    device_kind: str
    device_count: int
    execution_scope: str
    schedule_sha256: str
    cuda_source_sha256: str
    kernel_manifest_sha256: str
    preflight_passed: bool
    input_sha256: tuple[str, ...]
    output_sha256: tuple[str, ...]
    oracle_sha256: tuple[str, ...]
    passed: bool
    maximum_absolute_errors: tuple[float, float]
    maximum_relative_errors: tuple[float, float]
    compile_duration_ns: int
    warmup_iterations: int
    measured_iterations: int
    samples_ns: tuple[int, ...]
    median_ns: int | None
    p90_ns: int | None
    coefficient_of_variation: float | None
    runtime: dict
    artifacts: tuple[ArtifactReference, ...]


def validate_fused_rpa_run_protocol(*, seed: int, warmup_iterations: int, measured_iterations: int) -> None:
    protocol = workloads.FUSED_RPA_BENCHMARK_PROTOCOL
    if (seed, warmup_iterations, measured_iterations) != (protocol["seed"], protocol["warmup_iterations"], protocol["measured_iterations"]):
        raise ValueError(
            "fused RPA run must use its predeclared benchmark protocol: "
            f"seed={protocol['seed']}, warmup={protocol['warmup_iterations']}, measured={protocol['measured_iterations']}"
        )


def expected_fused_rpa(inputs: tuple, *, softmax_scale: float) -> tuple[np.ndarray, np.ndarray]:
    """What the operation is defined to produce, on the host: first every sequence's new K / V row is
    written at position ``len - 1`` (page ``page_indices[cu_kv[s] // ps + (len-1) // ps]``, interleaved
    head index ``2 h`` for K and ``2 h + 1`` for V, zero beyond ``head_dim``); then each query head
    attends over its sequence's first ``len`` cache rows with the relative bias
    ``states[s, h] . projection[:, distance]`` for distances inside the projection's extent.
    float32 arithmetic; returns (output, updated cache) as bfloat16 arrays."""
    import ml_dtypes

    q, new_k, new_v, cache, lengths, page_indices, _cu_q, cu_kv, _distribution, states, projection = (
        None if value is None else np.asarray(value) for value in inputs)
    cache = np.array(cache, dtype=np.float32)
    q32, k32, v32 = (np.asarray(a, dtype=np.float32) for a in (q, new_k, new_v))
    pages, page_size, _, pack, _ = cache.shape
    sequences, q_heads, dim = q32.shape
    kv_heads = k32.shape[1]
    rows = cache.reshape(pages, page_size, -1, cache.shape[-1])  # a view: [page, slot, 2 h + which, padded dim]
    first_page = np.asarray(cu_kv, dtype=np.int64) // page_size
    for s in range(sequences):
        position = int(lengths[s]) - 1
        page = int(page_indices[first_page[s] + position // page_size])
        for h in range(kv_heads):
            for which, source in ((0, k32), (1, v32)):
                rows[page, position % page_size, 2 * h + which, :] = 0.0
                rows[page, position % page_size, 2 * h + which, :dim] = source[s, h]
    out = np.zeros_like(q32)
    group = q_heads // kv_heads
    for s in range(sequences):
        length = int(lengths[s])
        wanted = page_indices[first_page[s] : first_page[s] + math.ceil(length / page_size)].astype(np.int64)
        tokens = rows[wanted].reshape(-1, rows.shape[2], rows.shape[3])[:length, :, :dim]
        distance = (length - 1) - np.arange(length)
        for h in range(q_heads):
            keys, values = tokens[:, 2 * (h // group)], tokens[:, 2 * (h // group) + 1]
            logits = (keys @ q32[s, h]) * np.float32(softmax_scale)
            if states is not None:
                extent = projection.shape[1]
                bias = np.asarray(states, dtype=np.float32)[s, h] @ np.asarray(projection, dtype=np.float32)[:, np.clip(distance, 0, extent - 1)]
                logits = logits + np.where(distance < extent, bias, np.float32(0.0)).astype(np.float32)
            weights = np.exp(logits - logits.max(), dtype=np.float32)
            out[s, h] = (weights / weights.sum()) @ values
    return out.astype(ml_dtypes.bfloat16), cache.astype(ml_dtypes.bfloat16)


def _errors(actual: np.ndarray, expected: np.ndarray) -> tuple[float, float]:
    a, e = actual.astype(np.float32), expected.astype(np.float32)
    absolute = np.abs(a - e)
    return float(absolute.max()), float((absolute / np.maximum(np.abs(e), np.finfo(np.float32).tiny)).max())


def fused_rpa_outputs_pass(actual, expected, *, output_atol: float, output_rtol: float) -> bool:
    """Output within allclose(atol, rtol) and the updated cache bit for bit (rpa_runner.py:113-122)."""
    return bool(np.allclose(actual[0].astype(np.float32), expected[0].astype(np.float32), atol=output_atol, rtol=output_rtol)
                and np.array_equal(actual[1].view(np.uint16), expected[1].view(np.uint16)))


def _to_device(value, device):
    if value is None:
        return None
    array = np.ascontiguousarray(value)
    if array.dtype.itemsize == 2 and array.dtype.kind not in "iu":
        return torch.from_numpy(array.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(array.copy()).to(device)


def _bf16_host(tensor: torch.Tensor) -> np.ndarray:
    import ml_dtypes

    return tensor.detach().cpu().view(torch.uint16).numpy().view(ml_dtypes.bfloat16)


def _percentile(samples: list[int], fraction: float) -> int:
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, int(round(fraction * (len(ordered) - 1))))]


def fused_rpa_schedule_of(physical_schedule: Path | None):
    """The kernel the toy experiment runs: this backend's own schedule of it, or the one a saved
    ``physical.xdsl`` holds (this backend's or the reference's ``inkling_fused_rpa_schedule``,
    src/tpu_cake/workloads/inkling_rpa.py:145-195). A saved kernel must have the experiment's eleven
    input shapes, since the inputs are drawn for those (``FUSED_RPA_SCHEDULE_SHAPE_MISMATCH``)."""
    own = workloads.inkling_fused_rpa_schedule()
    if physical_schedule is None:
        return own
    from . import xdsl_text

    saved = xdsl_text.parse_reference_physical_kernel(Path(physical_schedule).read_text())
    saved.verify()
    expected = [tuple(value.type.shape) for value in own.ops[0].body.args]
    found = [tuple(value.type.shape) for value in saved.ops[0].body.args]
    if found != expected:
        raise ValueError(f"FUSED_RPA_SCHEDULE_SHAPE_MISMATCH expected={expected} found={found}")
    return saved


def run_fused_rpa(output_dir: Path, *, mode: RunMode | str = RunMode.TIMING, seed: int = 97, warmup_iterations: int = 5,
                  measured_iterations: int = 50, kv_chunk_tokens: int = 0, corrupt_device_cache_for_testing: bool = False,
                  physical_schedule: Path | None = None) -> FusedRpaRunResult:
    """Runs the toy fused-RPA experiment on the current GPU and writes its bundle.
    ``corrupt_device_cache_for_testing`` flips one cache element after the device call and before the
    check, to show that a single forged cache byte is refused. ``physical_schedule`` names a saved
    kernel to run instead of this backend's own schedule of the experiment."""
    if not torch.cuda.is_available():
        raise RuntimeError("run_fused_rpa needs a CUDA device: the CUDA backend has no CPU fallback")
    mode = RunMode(mode)
    validate_fused_rpa_run_protocol(seed=seed, warmup_iterations=warmup_iterations, measured_iterations=measured_iterations)
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=False)
    device = torch.device("cuda", torch.cuda.current_device())
    schedule = fused_rpa_schedule_of(physical_schedule)
    plan = rpa_cuda_lowering.lower_inkling_rpa_to_cuda(schedule, kv_chunk_tokens=kv_chunk_tokens)
    run_id = semantic_sha256("inkling-fused-rpa-run", mode.value, str(seed), str(warmup_iterations), str(measured_iterations),
                             plan.schedule_sha256, plan.source_sha256())
    invocation = {"mode": mode.value, "seed": seed, "warmup_iterations": warmup_iterations, "measured_iterations": measured_iterations,
                  "kv_chunk_tokens": kv_chunk_tokens, "execution_scope": plan.execution_scope, "schedule_sha256": plan.schedule_sha256,
                  "cuda_source_sha256": plan.source_sha256()}
    artifacts: list[ArtifactReference] = []
    contract = run_artifacts.profiler_contract(mode)
    run_artifacts.validate_profiler_contract(contract)
    run_artifacts.write_json(output_dir, output_dir / "invocation.json", invocation, "invocation", artifacts)
    run_artifacts.write_json(output_dir, output_dir / "profiler_config.json", {**contract, "attached": run_artifacts.profiler_attached()},
                             "profiler_config", artifacts)
    run_artifacts.source_state(output_dir, artifacts)
    ledger_path = output_dir / "ledger.sqlite"

    def record(state: RunState, payload: dict) -> None:
        with RunLedger(ledger_path) as ledger:
            if state is RunState.CREATED:
                ledger.create(run_id, payload)
            else:
                ledger.transition(run_id, state, payload)

    record(RunState.CREATED, invocation)
    schedule.verify()
    physical_text = ir.canonical_text(schedule)
    record(RunState.VERIFIED, {"physical_ir_sha256": ir.schedule_sha256(schedule)})
    experiment = run_artifacts.experiment_record(
        workload={"name": "inkling-fused-ragged-paged-attention", "stage": "steady_decode",
                  "inputs": [{"name": name, "shape": None if shape is None else list(shape)} for name, shape in
                             zip(rpa_cuda_lowering.FUSED_INPUT_NAMES, plan.input_shapes, strict=True)],
                  "outputs": [{"name": "output", "shape": list(plan.output_shape)}, {"name": "updated_cache", "shape": list(plan.fused_cache_shape)}]},
        schedule_sha256=plan.schedule_sha256, warmup_iterations=warmup_iterations, measured_iterations=measured_iterations,
        profile_expectation={"name": "inkling-fused-rpa-steady-decode", "required_timed_hlo_markers": ["cake_rpa_decode_sm100"],
                             "forbidden_timed_hlo_fragments": ["flash_fwd", "paged_attention_v", "BatchDecode"],
                             "require_tensor_core_activity": False},
        tolerance={"reference": "expected_fused_rpa (numpy float32)", "absolute_tolerance": OUTPUT_ATOL, "relative_tolerance": OUTPUT_RTOL,
                   "cache": "bit-exact"},
    )
    run_artifacts.write_json(output_dir, output_dir / "experiment.json", experiment, "experiment", artifacts)
    run_artifacts.write_text(output_dir, output_dir / "physical.xdsl", physical_text, "physical_schedule", artifacts)
    run_artifacts.write_text(output_dir, output_dir / "lowered_cuda.py", plan.render_executable_source(), "lowered_source", artifacts)
    record(RunState.LOWERED, {"schedule_sha256": plan.schedule_sha256, "cuda_source_sha256": plan.source_sha256(),
                              "execution_scope": plan.execution_scope})

    host_inputs = workloads.inkling_fused_rpa_inputs(seed)
    plan.preflight(*host_inputs)
    run_artifacts.write_json(output_dir, output_dir / "preflight.json", {
        "passed": True, "validator": "CudaFusedRpaPlan.preflight", "input_shapes": [list(np.asarray(v).shape) for v in host_inputs],
        "input_dtypes": [str(np.asarray(v).dtype) for v in host_inputs]}, "preflight_result", artifacts)
    expected = expected_fused_rpa(host_inputs, softmax_scale=plan.softmax_scale)

    compile_started = time.perf_counter_ns()
    executable = plan.build(device)
    compile_duration_ns = time.perf_counter_ns() - compile_started
    library = _native.library_path()
    manifest = {"library": library.name, "library_size_bytes": library.stat().st_size, "library_sha256": run_artifacts.sha256_file(library),
                "abi_version": int(_native.load().cake_abi_version()), "kernels": list(RPA_KERNELS)}
    manifest_reference = run_artifacts.write_json(output_dir, output_dir / "kernel_manifest.json", manifest, "kernel_manifest", artifacts)
    record(RunState.COMPILED, {"kernel_manifest_sha256": manifest_reference.sha256, "compile_duration_ns": compile_duration_ns})

    def fresh_device_inputs() -> tuple:
        return tuple(_to_device(value, device) for value in host_inputs)

    try:
        output, cache = plan.invoke(executable, *fresh_device_inputs())
        torch.cuda.synchronize(device)
        executable.status()
        if corrupt_device_cache_for_testing:
            flat = cache.view(torch.int16).view(-1)
            flat[12345] ^= 1
        actual = (_bf16_host(output), _bf16_host(cache))
        maximum_errors = tuple(_errors(a, e) for a, e in zip(actual, expected, strict=True))
        passed = fused_rpa_outputs_pass(actual, expected, output_atol=OUTPUT_ATOL, output_rtol=OUTPUT_RTOL)
        if not passed:
            record(RunState.REJECTED, {"reason": "numerical mismatch", "maximum_errors": [list(e) for e in maximum_errors],
                                       "cache_exact": bool(np.array_equal(actual[1].view(np.uint16), expected[1].view(np.uint16)))})
            raise ValueError(f"FUSED_RPA_CORRECTNESS_FAILED errors={maximum_errors}")
        record(RunState.CORRECT, {"output_shapes": [list(a.shape) for a in actual], "maximum_errors": [list(e) for e in maximum_errors]})

        # The cache is updated in place: every call gets device copies of its own.
        warmup_inputs = [fresh_device_inputs() for _ in range(warmup_iterations)]
        measured_inputs = [fresh_device_inputs() for _ in range(measured_iterations)]
        torch.cuda.synchronize(device)
        for inputs in warmup_inputs:
            plan.invoke(executable, *inputs)
            torch.cuda.synchronize(device)
        samples: list[int] = []
        for inputs in measured_inputs:
            started = time.perf_counter_ns()
            plan.invoke(executable, *inputs)
            torch.cuda.synchronize(device)
            if mode is RunMode.TIMING:
                samples.append(time.perf_counter_ns() - started)
        executable.status()
    finally:
        executable.close()

    names = rpa_cuda_lowering.FUSED_INPUT_NAMES
    input_refs, output_refs, oracle_refs = [], [], []
    for index, (name, value) in enumerate(zip(names, host_inputs, strict=True)):
        path = output_dir / "inputs" / f"{index:02d}-{name}.npy"
        path.parent.mkdir(exist_ok=True)
        array = np.asarray(value)
        np.save(path, array.view(np.uint16) if array.dtype.itemsize == 2 and array.dtype.kind not in "iu" else array)
        input_refs.append(run_artifacts.reference_of(output_dir, path, "correctness_input"))
    for folder, values, role, refs in (("outputs", actual, "correctness_output", output_refs), ("oracle", expected, "oracle_output", oracle_refs)):
        for index, (name, value) in enumerate(zip(("output", "updated_cache"), values, strict=True)):
            path = output_dir / folder / f"{index:02d}-{name}.npy"
            path.parent.mkdir(exist_ok=True)
            np.save(path, np.asarray(value).view(np.uint16))
            refs.append(run_artifacts.reference_of(output_dir, path, role))
    artifacts.extend((*input_refs, *output_refs, *oracle_refs))
    median_ns = int(statistics.median(samples)) if samples else None
    p90_ns = _percentile(samples, 0.9) if samples else None
    coefficient = statistics.pstdev(samples) / statistics.mean(samples) if len(samples) > 1 and statistics.mean(samples) else None
    terminal = {RunMode.TIMING: RunState.TIMED, RunMode.TRACE: RunState.TRACED, RunMode.COUNTERS: RunState.COUNTERED}[mode]
    payload = {"measured_iterations": measured_iterations, "warmup_iterations": warmup_iterations}
    if mode is RunMode.TIMING:
        payload.update(median_ns=median_ns, p90_ns=p90_ns, sample_count=len(samples))
    else:
        payload.update(profiler_attached=run_artifacts.profiler_attached(), capture="launches.csv, attached when the bundle is finalised")
    record(terminal, payload)
    artifacts.append(run_artifacts.reference_of(output_dir, ledger_path, "execution_ledger"))
    result = FusedRpaRunResult(
        run_id=run_id, mode=mode.value, backend="cuda", device_kind=torch.cuda.get_device_name(device), device_count=1,
        execution_scope=plan.execution_scope, schedule_sha256=plan.schedule_sha256, cuda_source_sha256=plan.source_sha256(),
        kernel_manifest_sha256=manifest_reference.sha256, preflight_passed=True,
        input_sha256=tuple(r.sha256 for r in input_refs), output_sha256=tuple(r.sha256 for r in output_refs),
        oracle_sha256=tuple(r.sha256 for r in oracle_refs), passed=passed,
        maximum_absolute_errors=(maximum_errors[0][0], maximum_errors[1][0]), maximum_relative_errors=(maximum_errors[0][1], maximum_errors[1][1]),
        compile_duration_ns=compile_duration_ns, warmup_iterations=warmup_iterations, measured_iterations=measured_iterations,
        samples_ns=tuple(samples), median_ns=median_ns, p90_ns=p90_ns, coefficient_of_variation=coefficient,
        runtime={"python": __import__("sys").version.split()[0], "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
                 "gpu_name": torch.cuda.get_device_name(device), "abi_version": int(_native.load().cake_abi_version()), "hostname": socket.gethostname()},
        artifacts=tuple(artifacts),
    )
    (output_dir / "result.json").write_text(json.dumps(asdict(result), indent=2) + "\n")
    return result


def validate_fused_rpa_bundle(root: Path) -> dict:
    """Re-checks a finished RPA bundle from its files: every listed artifact has the recorded size
    and hash, the saved output passes the tolerance against the saved expectation and the saved
    caches are identical, and the expectation itself is recomputed from the saved inputs."""
    import ml_dtypes

    root = Path(root)
    result = json.loads((root / "result.json").read_text())
    for artifact in result["artifacts"]:
        path = root / artifact["path"]
        if not path.is_file():
            raise ValueError(f"ARTIFACT_MISSING path={artifact['path']}")
        if path.stat().st_size != artifact["size_bytes"] or run_artifacts.sha256_file(path) != artifact["sha256"]:
            raise ValueError(f"ARTIFACT_CHANGED path={artifact['path']}")

    def load(folder: str, index: int, name: str, bf16: bool) -> np.ndarray:
        array = np.load(root / folder / f"{index:02d}-{name}.npy")
        return array.view(ml_dtypes.bfloat16) if bf16 else array

    names = rpa_cuda_lowering.FUSED_INPUT_NAMES
    bf16_inputs = {0, 1, 2, 3, 9, 10}
    inputs = tuple(load("inputs", i, name, i in bf16_inputs) for i, name in enumerate(names))
    actual = tuple(load("outputs", i, name, True) for i, name in enumerate(("output", "updated_cache")))
    saved_expectation = tuple(load("oracle", i, name, True) for i, name in enumerate(("output", "updated_cache")))
    invocation = json.loads((root / "invocation.json").read_text())
    # The kernel that ran is the one saved in the bundle (its bytes were checked above): parse it,
    # verify it and lower it again.
    plan = rpa_cuda_lowering.lower_inkling_rpa_to_cuda(fused_rpa_schedule_of(root / "physical.xdsl"), kv_chunk_tokens=invocation["kv_chunk_tokens"])
    # The canonical text carries the fixed symbol ``kernel``; the name the run used is in its source.
    named = re.match(r"# [^\n]*\nname = '([^'\n]*)'\n", (root / "lowered_cuda.py").read_text())
    if named is None:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    plan = replace(plan, name=named.group(1))
    if plan.schedule_sha256 != result["schedule_sha256"] or plan.source_sha256() != result["cuda_source_sha256"]:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    recomputed = expected_fused_rpa(inputs, softmax_scale=plan.softmax_scale)
    if not all(np.array_equal(a.view(np.uint16), b.view(np.uint16)) for a, b in zip(recomputed, saved_expectation, strict=True)):
        raise ValueError("EXPECTATION_DOES_NOT_REPLAY")
    if not fused_rpa_outputs_pass(actual, saved_expectation, output_atol=OUTPUT_ATOL, output_rtol=OUTPUT_RTOL):
        raise ValueError("FUSED_RPA_CORRECTNESS_FAILED saved outputs do not pass against the saved expectation")
    return result


def rpa_device_main(argv: list[str] | None = None) -> int:
    """``rpa_device_main OUT --mode timing``: the device entry point of the reference
    (src/tpu_cake/rpa_device_main.py:47-159) for this backend."""
    import argparse

    parser = argparse.ArgumentParser(prog="rpa_device_main")
    parser.add_argument("output_dir", type=Path)
    parser.add_argument("--mode", choices=[m.value for m in RunMode], default=RunMode.TIMING.value)
    parser.add_argument("--kv-chunk-tokens", type=int, default=0)
    parser.add_argument("--from-physical", type=Path, default=None)
    args = parser.parse_args(argv)
    protocol = workloads.FUSED_RPA_BENCHMARK_PROTOCOL
    result = run_fused_rpa(args.output_dir, mode=args.mode, seed=protocol["seed"], warmup_iterations=protocol["warmup_iterations"],
                           measured_iterations=protocol["measured_iterations"], kv_chunk_tokens=args.kv_chunk_tokens,
                           physical_schedule=args.from_physical)
    print(f"FUSED_RPA_RUN run_id={result.run_id} mode={result.mode} passed={result.passed} median_ns={result.median_ns}")
    return 0
