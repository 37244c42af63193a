"""``run_distributed_matmul``: the CUDA-backend counterpart of the reference's runner
(src/tpu_cake/runner.py:264-634).

Same sequence and evidence: a single-use output directory, ``invocation.json``, a run id that is a
semantic hash of the invocation, a ledger that moves CREATED -> VERIFIED -> LOWERED -> COMPILED ->
CORRECT -> TIMED (or REJECTED), the two IR texts, the lowered source, the cost model, seeded inputs
(:439-456), warm-up, the correctness check ``allclose(actual, bf16(lhs) @ bf16(rhs), 1e-3, 1e-3)``
in float32 (:488-525), timed calls each followed by a synchronisation (:526-531), the arrays, and
``result.json``. The compile artifacts (StableHLO / compiler HLO in the reference) are replaced by
a kernel manifest: library path, size and SHA-256, ABI version, kernel names.

Execution models: ``mesh_size == 1`` runs on the current GPU; ``mesh_size > 1`` runs one process
per GPU when launched under ``torch.distributed.run`` with a matching world size. Without such a
launch a mesh larger than one is refused, unless the caller asks for ``emulate_on_one_gpu``: every
mesh position's kernels then run on the current GPU (all pushes enqueued before any reduction),
which checks correctness but whose timing is marked ``emulated-on-one-gpu`` and is not a multi-GPU
number.

Modes (``RunMode``, src/tpu_cake/runner.py:54-57): ``timing`` times every measured call on the host;
``trace`` and ``counters`` run the same calls untimed for a profiler that wraps the process
(``profiler_config.json`` names the ``ncu`` invocation; src/tpu_cake/runner.py:144-217) and end in
TRACED / COUNTERED (:570-571).
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import socket
import statistics
import sys
import time
from dataclasses import asdict, dataclass
from pathlib import Path

import numpy as np
import torch

from . import _native, cost_model, cuda_lowering, dialects, ir, run_artifacts, schedule_lowering, workloads
from .identity import array_sha256, semantic_sha256
from .mesh import ProcessMesh
from .run_artifacts import RunMode
from .run_ledger import RunLedger, RunState

_IMPLEMENTATION = {
    cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER: dialects.CollectiveImplementation.NCCL,
    cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE: dialects.CollectiveImplementation.P2P_OWNER_PUSH,
    cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT: dialects.CollectiveImplementation.P2P_OWNER_PUSH_BF16,
}


@dataclass(frozen=True)
class ArtifactReference:
    path: str
    size_bytes: int
    sha256: str
    role: str


@dataclass(frozen=True)
class MatmulRunResult:
    run_id: str
    mode: str
    backend: str
    device_kind: str
    device_count: int
    execution: str
    collective_strategy: str
    hostname: str
    schedule_sha256: str
    cuda_source_sha256: str
    kernel_manifest_sha256: str
    lhs_sha256: str
    rhs_sha256: str
    output_sha256: str
    passed: bool
    maximum_absolute_error: float
    maximum_relative_error: float
    compile_duration_ns: int
    warmup_iterations: int
    measured_iterations: int
    samples_ns: tuple[int, ...]
    median_ns: int | None
    p90_ns: int | None
    coefficient_of_variation: float | None
    runtime: dict
    artifacts: tuple[ArtifactReference, ...]


def _sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        for block in iter(lambda: handle.read(1 << 20), b""):
            digest.update(block)
    return digest.hexdigest()


def _write(path: Path, text: str, role: str, artifacts: list[ArtifactReference]) -> ArtifactReference:
    path.write_text(text)
    reference = ArtifactReference(path.name, path.stat().st_size, _sha256_file(path), role)
    artifacts.append(reference)
    return reference


def _percentile(samples: list[int], fraction: float) -> int:
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, int(round(fraction * (len(ordered) - 1))))]


def _runtime_identity() -> dict:
    return {
        "python": sys.version.split()[0], "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
        "gpu_name": torch.cuda.get_device_name(torch.cuda.current_device()), "abi_version": int(_native.load().cake_abi_version()),
    }


def _to_device(array: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array).view(np.uint16).copy()).view(torch.bfloat16).to(device)


class _EmulatedMesh:
    """Every mesh position's kernels on the current GPU, pushes of all positions before any
    reduction so that no launch waits on a later one."""

    def __init__(self, plan: cuda_lowering.CudaMatmulRsPlan, device: torch.device):
        self.plan, self.device, self.lib = plan, device, _native.load()
        world = plan.mesh_size
        peer = plan.collective_implementation is not cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER
        self.peer = peer
        self.handles, self.slots, self.flags = [], [], []
        for rank in range(world):
            desc = _native.MatmulRsDesc(
                m=plan.partial_local_shape[0], n=plan.partial_local_shape[1], k_local=plan.lhs_local_shape[1], world=world, rank=rank,
                scatter_dim=plan.scatter_dimension, out_dtype=cuda_lowering._CAKE_DTYPE[plan.output_dtype],
                transport_dtype=cuda_lowering._CAKE_DTYPE[plan.transport_dtype],
                strategy=_native.CAKE_RS_P2P_OWNER_PUSH if peer else _native.CAKE_RS_LOCAL_PARTIAL, tile_m=plan.tile_m, tile_n=plan.tile_n,
                rhs_layout=0, wait_budget_ms=0,
            )
            handle = ctypes.c_void_p()
            _native.check(self.lib.cake_matmul_rs_create(ctypes.byref(desc), ctypes.byref(handle)))
            self.handles.append(handle)
        if peer:
            for handle in self.handles:
                slot, flag = ctypes.c_void_p(), ctypes.c_void_p()
                _native.check(self.lib.cake_symm_alloc(self.lib.cake_matmul_rs_slot_bytes(handle), ctypes.byref(slot)))
                _native.check(self.lib.cake_symm_alloc(self.lib.cake_matmul_rs_flag_bytes(handle), ctypes.byref(flag)))
                self.slots.append(slot.value)
                self.flags.append(flag.value)
            array = ctypes.c_void_p * world
            for handle in self.handles:
                _native.check(self.lib.cake_matmul_rs_bind_peers(handle, array(*self.slots), array(*self.flags)))

    def __call__(self, lhs_shards, rhs_shards) -> list[torch.Tensor]:
        plan, world = self.plan, self.plan.mesh_size
        stream = torch.cuda.current_stream(self.device).cuda_stream
        dtype = torch.float32 if plan.output_dtype == "f32" else torch.bfloat16
        outs = [torch.empty(plan.output_local_shape, dtype=dtype, device=self.device) for _ in range(world)]
        if self.peer:
            for handle, lhs, rhs in zip(self.handles, lhs_shards, rhs_shards):
                _native.check(self.lib.cake_matmul_rs_enqueue_push(handle, lhs.data_ptr(), rhs.data_ptr(), stream))
            for handle, out in zip(self.handles, outs):
                _native.check(self.lib.cake_matmul_rs_enqueue_reduce(handle, out.data_ptr(), stream))
            return outs
        total = torch.zeros((world,) + plan.output_local_shape, dtype=torch.float32, device=self.device)
        for handle, lhs, rhs in zip(self.handles, lhs_shards, rhs_shards):
            partial = torch.empty((world,) + plan.output_local_shape, dtype=torch.float32, device=self.device)
            _native.check(self.lib.cake_matmul_rs_enqueue(handle, lhs.data_ptr(), rhs.data_ptr(), partial.data_ptr(), stream))
            total += partial  # stands in for the library reduce-scatter, rank order
        for rank in range(world):
            outs[rank].copy_(total[rank])
        return outs

    def status(self) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        for handle in self.handles:
            word = _native.CakeStatus()
            _native.check(self.lib.cake_matmul_rs_status(handle, stream, ctypes.byref(word)))

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for handle in self.handles:
            self.lib.cake_matmul_rs_destroy(handle)
        for pointer in self.slots + self.flags:
            self.lib.cake_symm_free(pointer)
        self.handles, self.slots, self.flags = [], [], []


def lower_invocation(invocation: dict):
    """The logical schedule, the physical kernel and the CUDA plan an invocation record names. The
    runner and the receipt both go through here, so a bundle replays exactly what ran -- also when
    the run was started from a saved physical schedule, whose target description and whether its
    collective names an implementation are then part of the record."""
    logical = workloads.distributed_matmul_schedule(
        mesh_size=invocation["mesh_size"], m=invocation["m"], k=invocation["k"], n=invocation["n"],
        scatter_dimension=invocation["scatter_dimension"],
    )
    tile = schedule_lowering.MatmulTile(*invocation["tile"]) if invocation.get("tile") else None
    strategy = cuda_lowering.MatmulCollectiveStrategy(invocation["collective_strategy"])
    target = schedule_lowering.LoweringTarget(**invocation["target"]) if invocation.get("target") else schedule_lowering.B200_TARGET
    declare = invocation.get("declare_implementation", True) and invocation["mesh_size"] > 1
    physical = schedule_lowering.lower_distributed_matmul(
        logical, target=target, tile=tile, collective_implementation=_IMPLEMENTATION[strategy] if declare else None
    )
    return logical, physical, cuda_lowering.lower_physical_matmul_to_cuda(physical, output_dtype=invocation["output_dtype"])


def invocation_of_saved_schedule(path: Path) -> dict:
    """What ``run_distributed_matmul`` needs to run the kernel a saved ``physical.xdsl`` holds: the
    file is parsed, verified and lowered once to read mesh, shapes, tile, scatter dimension, target
    and collective from it. The run regenerates the kernel from these and refuses to start if the
    text it gets is not the saved one (``SAVED_PHYSICAL_IR_NOT_REPRODUCED``)."""
    from . import xdsl_text

    module = xdsl_text.parse_reference_physical_kernel(Path(path).read_text())
    module.verify()
    plan = cuda_lowering.lower_physical_matmul_to_cuda(module)
    kernel = module.ops[0]
    matmul = next(op for op in kernel.body.ops if op.name == "tpu_schedule.mxu_matmul")
    collective = next(op for op in kernel.body.ops if op.name == "tpu_schedule.collective")
    bandwidth = dict(plan.collective_link_bandwidths)[plan.mesh_axis]
    strategy = plan.collective_implementation or cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER
    target = {"name": kernel.properties["target"], "vmem_capacity_bytes": kernel.properties["vmem_capacity_bytes"],
              "smem_capacity_bytes": kernel.properties["smem_capacity_bytes"], "ici_bandwidth_bytes_per_second": bandwidth}
    return {
        "mesh_size": plan.mesh_size, "m": plan.lhs_local_shape[0], "k": plan.lhs_local_shape[1] * plan.mesh_size, "n": plan.rhs_local_shape[1],
        "tile": schedule_lowering.MatmulTile(matmul.properties["tile_m"], matmul.properties["tile_n"]),
        "scatter_dimension": "MN"[plan.scatter_dimension], "collective_strategy": strategy.value, "target": target,
        "declare_implementation": "implementation" in collective.properties, "expected_schedule_sha256": plan.schedule_sha256,
    }


def run_distributed_matmul(
    output_dir: Path,
    *,
    mesh_size: int,
    m: int,
    k: int,
    n: int,
    warmup_iterations: int,
    measured_iterations: int,
    tile: schedule_lowering.MatmulTile | None = None,
    collective_strategy: str = "nccl_reduce_scatter",
    scatter_dimension: str = "N",
    output_dtype: str = "f32",
    mode: RunMode | str = RunMode.TIMING,
    emulate_on_one_gpu: bool = False,
    target: dict | None = None,
    declare_implementation: bool = True,
    expected_schedule_sha256: str | None = None,
) -> MatmulRunResult:
    if not torch.cuda.is_available():
        raise RuntimeError("run_distributed_matmul needs a CUDA device: the CUDA backend has no CPU fallback")
    if measured_iterations <= 0 or warmup_iterations < 0:
        raise ValueError("measured_iterations must be positive and warmup_iterations non-negative")
    mode = RunMode(mode)
    strategy = cuda_lowering.MatmulCollectiveStrategy(collective_strategy)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    distributed = mesh_size > 1 and world == mesh_size
    if mesh_size > 1 and not distributed and not emulate_on_one_gpu:
        raise ValueError(
            f"MESH_NOT_AVAILABLE mesh_size={mesh_size} world_size={world}: launch one process per GPU "
            "(python -m torch.distributed.run --nproc-per-node MESH ...), or ask for emulate_on_one_gpu "
            "(correctness only: its timing is not a multi-GPU number)"
        )
    mesh = ProcessMesh.from_environment() if distributed else ProcessMesh.single()
    leader = mesh.rank == 0
    output_dir = Path(output_dir)
    artifacts: list[ArtifactReference] = []
    if leader:
        output_dir.mkdir(parents=True, exist_ok=False)
    invocation = {
        "mesh_size": mesh_size, "m": m, "k": k, "n": n, "warmup_iterations": warmup_iterations,
        "measured_iterations": measured_iterations, "tile": None if tile is None else [tile.m, tile.n],
        "collective_strategy": strategy.value, "scatter_dimension": scatter_dimension, "output_dtype": output_dtype, "mode": mode.value,
        "execution": "one-process-per-gpu" if distributed or mesh_size == 1 else "emulated-on-one-gpu",
    }
    if target is not None:  # a run started from a saved physical schedule
        invocation["target"] = dict(target)
        invocation["declare_implementation"] = bool(declare_implementation)
    run_id = semantic_sha256("distributed-matmul-run", json.dumps(invocation, sort_keys=True))
    ledger_path = output_dir / "ledger.sqlite"

    def record(state: RunState, payload: dict) -> None:
        if not leader:
            return
        with RunLedger(ledger_path) as ledger:
            if state is RunState.CREATED:
                ledger.create(run_id, payload)
            else:
                ledger.transition(run_id, state, payload)

    contract = run_artifacts.profiler_contract(mode)
    run_artifacts.validate_profiler_contract(contract)
    if leader:
        _write(output_dir / "invocation.json", json.dumps(invocation, indent=2, sort_keys=True) + "\n", "invocation", artifacts)
        _write(output_dir / "profiler_config.json", json.dumps({**contract, "attached": run_artifacts.profiler_attached()}, indent=2, sort_keys=True) + "\n",
               "profiler_config", artifacts)
        shared: list[run_artifacts.ArtifactReference] = []
        run_artifacts.source_state(output_dir, shared)
        artifacts.extend(ArtifactReference(a.path, a.size_bytes, a.sha256, a.role) for a in shared)
    record(RunState.CREATED, invocation)

    logical, physical, plan = lower_invocation(invocation)
    logical.verify()
    record(RunState.VERIFIED, {"distributed_sha256": ir.schedule_sha256(logical)})
    if expected_schedule_sha256 is not None and plan.schedule_sha256 != expected_schedule_sha256:
        raise ValueError(f"SAVED_PHYSICAL_IR_NOT_REPRODUCED expected={expected_schedule_sha256} regenerated={plan.schedule_sha256}")
    record(RunState.LOWERED, {"schedule_sha256": plan.schedule_sha256, "cuda_source_sha256": plan.source_sha256()})
    library = _native.library_path()
    manifest = {
        "library": library.name, "library_size_bytes": library.stat().st_size, "library_sha256": _sha256_file(library),
        "abi_version": int(_native.load().cake_abi_version()),
        "kernels": [f"cake_matmul_rs_sm100<{plan.tile_n}>"] + (["cake_reduce_slots_sm100"] if mesh_size > 1 and strategy is not cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER else []),
    }
    if leader:
        _write(output_dir / "distributed.xdsl", ir.canonical_text(logical), "schedule", artifacts)
        _write(output_dir / "physical.xdsl", ir.canonical_text(physical), "physical_schedule", artifacts)
        _write(output_dir / "lowered_cuda.py", plan.render_executable_source(), "lowered_source", artifacts)
        wanted_kernels = [name.split("<")[0] for name in manifest["kernels"][:1]]
        experiment = run_artifacts.experiment_record(
            workload={"name": "distributed-matmul-reduce-scatter", "identity": workloads.distributed_matmul_workload_identity(mesh_size, m, k, n),
                      "mesh_size": mesh_size, "m": m, "k": k, "n": n, "scatter_dimension": scatter_dimension, "input_dtype": "bf16",
                      "accumulate": "f32", "output_dtype": output_dtype, "collective_strategy": strategy.value},
            schedule_sha256=plan.schedule_sha256, warmup_iterations=warmup_iterations, measured_iterations=measured_iterations,
            profile_expectation={"name": f"matmul-{strategy.value}", "required_timed_hlo_markers": wanted_kernels,
                                 "forbidden_timed_hlo_fragments": [] if strategy is cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER else ["ncclDevKernel_ReduceScatter"],
                                 "require_tensor_core_activity": mode is RunMode.COUNTERS},
            tolerance={"reference": "bf16(lhs).astype(f32) @ bf16(rhs).astype(f32)", "absolute_tolerance": 1e-3, "relative_tolerance": 1e-3,
                       "bf16_rule": "relative L2 <= 1e-2 when the output or the transport is bf16"},
        )
        _write(output_dir / "experiment.json", json.dumps(experiment, indent=2, sort_keys=True) + "\n", "experiment", artifacts)
        hardware = cost_model.B200_MEASURED
        _write(output_dir / "cost_model_input.json", json.dumps({
            "plan": {"mesh_size": plan.mesh_size, "lhs_local_shape": plan.lhs_local_shape, "rhs_local_shape": plan.rhs_local_shape,
                     "partial_local_shape": plan.partial_local_shape, "output_local_shape": plan.output_local_shape,
                     "scatter_dimension": plan.scatter_dimension, "tile": [plan.tile_m, plan.tile_k, plan.tile_n],
                     "output_dtype": plan.output_dtype, "transport_dtype": plan.transport_dtype,
                     "collective_implementation": None if plan.collective_implementation is None else plan.collective_implementation.value},
            "hardware": asdict(hardware),
        }, indent=2, sort_keys=True, default=str) + "\n", "cost_model_input", artifacts)
        report = cost_model.estimate_distributed_matmul(plan)
        _write(output_dir / "cost_model.json", json.dumps({**asdict(report.counts), "compute_ns": str(report.compute_ns), "memory_ns": str(report.memory_ns),
                                                          "communication_ns": str(report.communication_ns), "lower_bound_ns": str(report.lower_bound_ns),
                                                          "limiting_resource": report.limiting_resource}, indent=2) + "\n", "cost_model", artifacts)
    manifest_reference = None
    if leader:
        manifest_reference = _write(output_dir / "kernel_manifest.json", json.dumps(manifest, indent=2, sort_keys=True) + "\n", "kernel_manifest", artifacts)

    compile_start = time.perf_counter_ns()
    if distributed or mesh_size == 1:
        executable, _ = plan.build(mesh=mesh)
        emulated = None
    else:
        executable, emulated = None, _EmulatedMesh(plan, mesh.device)
    compile_duration_ns = time.perf_counter_ns() - compile_start
    record(RunState.COMPILED, {"kernel_manifest_sha256": manifest_reference.sha256 if manifest_reference else "", "compile_duration_ns": compile_duration_ns})

    lhs, rhs = workloads.distributed_matmul_inputs(mesh_size, m, k, n)
    lhs32, rhs32 = lhs.astype(np.float32), rhs.astype(np.float32)
    expected = lhs32 @ rhs32
    axis = 0 if scatter_dimension == "M" else 1
    if emulated is not None:
        shards = [workloads.shard_matmul_inputs(lhs, rhs, mesh_size, r) for r in range(mesh_size)]
        lhs_d = [_to_device(a, mesh.device) for a, _ in shards]
        rhs_d = [_to_device(b, mesh.device) for _, b in shards]
        call = lambda: emulated(lhs_d, rhs_d)  # noqa: E731
    else:
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, mesh_size, mesh.rank)
        lhs_d, rhs_d = _to_device(lhs_r, mesh.device), _to_device(rhs_r, mesh.device)
        call = lambda: executable(lhs_d, rhs_d)  # noqa: E731
    for _ in range(warmup_iterations):
        call()
        torch.cuda.synchronize(mesh.device)
    result = call()
    torch.cuda.synchronize(mesh.device)
    (emulated or executable).status()  # raises if a bounded device-side wait ran out
    if emulated is not None:
        actual = np.concatenate([t.float().cpu().numpy() for t in result], axis=axis)
        reference_slice = expected
    else:
        actual = result.float().cpu().numpy()
        step = expected.shape[axis] // mesh_size
        reference_slice = np.take(expected, range(mesh.rank * step, (mesh.rank + 1) * step), axis=axis) if mesh_size > 1 else expected
    absolute = np.abs(actual - reference_slice)
    maximum_absolute_error = float(absolute.max())
    maximum_relative_error = float((absolute / np.maximum(np.abs(reference_slice), np.finfo(np.float32).tiny)).max())
    # The reference's rule is for f32 outputs; a bf16 output is compared after rounding the oracle too.
    if output_dtype == "bf16" or plan.transport_dtype == "bf16":
        passed = bool(np.sqrt(np.sum(absolute.astype(np.float64) ** 2) / np.sum(reference_slice.astype(np.float64) ** 2)) <= 1e-2)
    else:
        passed = bool(np.allclose(actual, reference_slice, atol=1e-3, rtol=1e-3))
    if distributed:
        flag = torch.tensor([0 if passed else 1], device=mesh.device)
        torch.distributed.all_reduce(flag, group=mesh.group)
        passed = int(flag.item()) == 0
    if not passed:
        record(RunState.REJECTED, {"reason": "numerical mismatch", "maximum_absolute_error": maximum_absolute_error,
                                   "maximum_relative_error": maximum_relative_error})
        raise ValueError(
            f"MATMUL_CORRECTNESS_FAILED maximum_absolute_error={maximum_absolute_error} maximum_relative_error={maximum_relative_error}"
        )
    record(RunState.CORRECT, {"lhs_sha256": array_sha256(lhs32), "rhs_sha256": array_sha256(rhs32), "output_sha256": array_sha256(actual),
                              "oracle_sha256": array_sha256(reference_slice)})
    samples: list[int] = []
    for _ in range(measured_iterations):
        mesh.barrier()
        started = time.perf_counter_ns()
        call()
        torch.cuda.synchronize(mesh.device)
        if mode is RunMode.TIMING:  # under a profiler the host clock measures the profiler
            samples.append(time.perf_counter_ns() - started)
    (emulated or executable).status()
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
    if leader:
        for name, array, role in (("lhs.npy", lhs32, "correctness_input"), ("rhs.npy", rhs32, "correctness_input"),
                                  ("output.npy", actual, "correctness_output"), ("oracle.npy", reference_slice, "oracle_output")):
            np.save(output_dir / name, array)
            path = output_dir / name
            artifacts.append(ArtifactReference(name, path.stat().st_size, _sha256_file(path), role))
        artifacts.append(ArtifactReference(ledger_path.name, ledger_path.stat().st_size, _sha256_file(ledger_path), "execution_ledger"))
    outcome = MatmulRunResult(
        run_id=run_id, mode=mode.value, backend="cuda", device_kind=torch.cuda.get_device_name(mesh.device), device_count=mesh_size,
        execution="one-process-per-gpu" if distributed or mesh_size == 1 else "emulated-on-one-gpu", collective_strategy=strategy.value,
        hostname=socket.gethostname(), schedule_sha256=plan.schedule_sha256, cuda_source_sha256=plan.source_sha256(),
        kernel_manifest_sha256=manifest_reference.sha256 if manifest_reference else "", lhs_sha256=array_sha256(lhs32),
        rhs_sha256=array_sha256(rhs32), output_sha256=array_sha256(actual), passed=passed, maximum_absolute_error=maximum_absolute_error,
        maximum_relative_error=maximum_relative_error, compile_duration_ns=compile_duration_ns, warmup_iterations=warmup_iterations,
        measured_iterations=measured_iterations, samples_ns=tuple(samples), median_ns=median_ns, p90_ns=p90_ns,
        coefficient_of_variation=coefficient, runtime=_runtime_identity(), artifacts=tuple(artifacts),
    )
    if leader:
        (output_dir / "result.json").write_text(json.dumps(asdict(outcome), indent=2) + "\n")
    (emulated or executable).close()
    return outcome
