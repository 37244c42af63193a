"""Correctness and timing protocol of the data x tensor sharded fused decode (the 2 x 4 surface).

Counterpart of ``run_inkling_sharded_rpa_surface`` (src/tpu_cake/rpa_surface_runner.py:1045) reduced
to what the hot path needs: the protocol of the shipped surface contract
(contracts/inkling-sharded-rpa-surface.json -- five correctness seeds, two executions each, exact
repeat, exact cache, output within 1e-3 max-abs and 6e-3 relative L2; then 5 warm-up calls and 16
timing rounds of 5 chained calls on the timing seed), the observation records
(``_correctness_observation``, :433-487) and the chained timing rounds (``_timing_rounds``, :490-517).
The evidence logistics around it (source manifests, relocation archives, HLO identities) are not
rebuilt.

The eight mesh positions exchange nothing (the reference's partition specs: sequences, pages and
metadata split over ``data``, heads over ``tensor``), so one process per GPU runs its own position
and the host gathers the shards for the record; with fewer GPUs than positions the positions can be
run one after the other on one GPU, which the record then says (``execution: emulated``).
"""

from __future__ import annotations

import json
import math
import statistics
from dataclasses import asdict, dataclass
from pathlib import Path

import numpy as np
import torch

from . import ir, rpa_cuda_lowering, run_artifacts, workloads
from .identity import array_sha256, semantic_sha256
from .rpa_runner import expected_fused_rpa
from .run_artifacts import ArtifactReference
from .run_ledger import RunLedger, RunState

SURFACE_PROTOCOL = {
    "correctness_seeds": (9423267841700844256, 15922986200921398903, 8194600149824386114, 12302695436007217200, 7696556979164032646),
    "timing_seed": 9423267841700844256,
    "repeat_executions": 2,
    "warmup_iterations": 5,
    "timing_rounds": 16,
    "samples_per_round": 5,
    "output_maximum_absolute_error": 1e-3,
    "output_relative_l2_error": 6e-3,
    "require_exact_cache": True,
}


@dataclass(frozen=True)
class SurfaceCorrectnessObservation:
    seed: int
    input_sha256: tuple[str, ...]
    output_sha256: str
    repeat_output_sha256: str
    oracle_output_sha256: str
    cache_sha256: str
    repeat_cache_sha256: str
    oracle_cache_sha256: str
    repeated_output_exact: bool
    repeated_cache_exact: bool
    cache_exact: bool
    maximum_absolute_error: float
    relative_l2_error: float
    passed: bool


def surface_error_metrics(actual: np.ndarray, expected: np.ndarray) -> tuple[float, float]:
    """(max-abs, relative L2) in float64 with the reference's refusals (src/tpu_cake/rpa_surface_runner.py:394-411)."""
    if actual.shape != expected.shape or actual.dtype != expected.dtype:
        raise ValueError(f"INKLING_SHARDED_RPA_OUTPUT_ABI_MISMATCH actual={actual.shape}/{actual.dtype} expected={expected.shape}/{expected.dtype}")
    a, e = actual.astype(np.float64), expected.astype(np.float64)
    if not np.all(np.isfinite(a)) or not np.all(np.isfinite(e)):
        raise ValueError("INKLING_SHARDED_RPA_OUTPUT_NONFINITE")
    difference = a - e
    maximum = float(np.abs(difference).max(initial=0.0))
    relative_l2 = math.sqrt(math.fsum((difference.ravel() ** 2).tolist()) / max(math.fsum((e.ravel() ** 2).tolist()), 1e-60))
    return maximum, round(relative_l2, 15)


def expected_surface(plan: rpa_cuda_lowering.ShardedCudaFusedRpaPlan, global_inputs: tuple) -> tuple[np.ndarray, np.ndarray]:
    """The host definition of the surface's result: every mesh position's shard through
    ``expected_fused_rpa``, assembled with the output partition specs
    (src/tpu_cake/workloads/inkling_rpa.py:640-691)."""
    outputs, caches = {}, {}
    for rank in range(plan.mesh_shape[0] * plan.mesh_shape[1]):
        position = plan.mesh_position(rank)
        shard = tuple(np.ascontiguousarray(v) for v in plan.shard_inputs(global_inputs, position))
        outputs[position], caches[position] = expected_fused_rpa(shard, softmax_scale=plan.local_plan.softmax_scale)
    return plan.assemble(outputs, 0), plan.assemble(caches, 1)


def _bf16_host(tensor: torch.Tensor) -> np.ndarray:
    import ml_dtypes

    return tensor.detach().contiguous().view(torch.int16).cpu().numpy().view(np.dtype(ml_dtypes.bfloat16))


class _SurfaceExecutor:
    """Runs the surface once: every position this process owns on its GPU, then the shards of all
    positions assembled on the host (gathered over ``torch.distributed`` when there is one process
    per position)."""

    def __init__(self, plan: rpa_cuda_lowering.ShardedCudaFusedRpaPlan, device: torch.device, *, emulate_on_one_gpu: bool):
        self.plan, self.device = plan, device
        self.positions = plan.mesh_shape[0] * plan.mesh_shape[1]
        distributed = torch.distributed.is_available() and torch.distributed.is_initialized()
        self.world = torch.distributed.get_world_size() if distributed else 1
        self.rank = torch.distributed.get_rank() if distributed else 0
        if self.world == self.positions:
            self.execution, self.owned = "one-process-per-gpu", (self.rank,)
        elif self.world == 1 and emulate_on_one_gpu:
            self.execution, self.owned = "emulated", tuple(range(self.positions))
        else:
            raise ValueError(f"MESH_NOT_AVAILABLE the surface has {self.positions} positions, this run has {self.world} process(es); "
                             "launch one process per GPU or pass emulate_on_one_gpu")
        self.executable = plan.build_executable(device)

    def close(self) -> None:
        self.executable.close()

    def run(self, global_inputs: tuple) -> tuple[np.ndarray, np.ndarray] | None:
        """(global output, global updated cache) on rank 0, None elsewhere."""
        outputs, caches = {}, {}
        for rank in self.owned:
            local = self.plan.place_inputs(global_inputs, rank, self.device)
            output, cache = self.plan.run_local(self.executable, *local)
            torch.cuda.synchronize(self.device)
            self.executable.status()
            outputs[self.plan.mesh_position(rank)] = _bf16_host(output)
            caches[self.plan.mesh_position(rank)] = _bf16_host(cache)
        if self.world > 1:
            gathered: list = [None] * self.world if self.rank == 0 else None
            torch.distributed.gather_object((outputs, caches), gathered, dst=0)
            if self.rank != 0:
                return None
            outputs, caches = {}, {}
            for part_outputs, part_caches in gathered:
                outputs.update(part_outputs)
                caches.update(part_caches)
        return self.plan.assemble(outputs, 0), self.plan.assemble(caches, 1)


def run_inkling_sharded_rpa_surface(output_dir: Path, *, emulate_on_one_gpu: bool = False, protocol: dict | None = None) -> dict:
    """Runs the surface protocol and writes its record under ``output_dir`` (rank 0 writes).
    ``protocol`` may shorten the timing part for tests; the correctness part is the contract's."""
    if not torch.cuda.is_available():
        raise RuntimeError("the sharded RPA surface needs CUDA devices: the CUDA backend has no CPU fallback")
    settings = {**SURFACE_PROTOCOL, **(protocol or {})}
    device = torch.device("cuda", torch.cuda.current_device())
    schedule = workloads.inkling_sharded_rpa_schedule()
    plan = rpa_cuda_lowering.lower_inkling_sharded_rpa_to_cuda(schedule)
    executor = _SurfaceExecutor(plan, device, emulate_on_one_gpu=emulate_on_one_gpu)
    leader = executor.rank == 0
    output_dir = Path(output_dir)
    artifacts: list[ArtifactReference] = []
    run_id = semantic_sha256("inkling-sharded-rpa-surface-run", plan.schedule_sha256, json.dumps(settings, sort_keys=True, default=list), executor.execution)
    ledger_path = output_dir / "ledger.sqlite"

    def record(state: RunState, payload: dict) -> None:
        if not leader:
            return
        with RunLedger(ledger_path) as ledger:
            if state is RunState.CREATED:
                ledger.create(run_id, payload)
            else:
                ledger.transition(run_id, state, payload)

    try:
        if leader:
            output_dir.mkdir(parents=True, exist_ok=False)
            run_artifacts.write_json(output_dir, output_dir / "contract.json", {**settings, "correctness_seeds": list(settings["correctness_seeds"]),
                                                                                "mesh_axes": list(plan.mesh_axes), "mesh_shape": list(plan.mesh_shape),
                                                                                "global_input_shapes": [None if s is None else list(s) for s in plan.global_input_shapes],
                                                                                "execution": executor.execution}, "contract", artifacts)
            run_artifacts.source_state(output_dir, artifacts)
            run_artifacts.write_text(output_dir, output_dir / "physical.xdsl", ir.canonical_text(schedule), "physical_schedule", artifacts)
        record(RunState.CREATED, {"run_id": run_id, "execution": executor.execution})
        schedule.verify()
        record(RunState.VERIFIED, {"physical_ir_sha256": ir.schedule_sha256(schedule)})
        record(RunState.LOWERED, {"schedule_sha256": plan.schedule_sha256, "mesh_shape": list(plan.mesh_shape)})
        record(RunState.COMPILED, {"device_kind": torch.cuda.get_device_name(device), "process_count": executor.world})

        observations = []
        for seed in settings["correctness_seeds"]:
            host_inputs = workloads.inkling_sharded_fused_rpa_inputs(seed)
            executions = [executor.run(host_inputs) for _ in range(settings["repeat_executions"])]
            if not leader:
                continue
            oracle_output, oracle_cache = expected_surface(plan, host_inputs)
            (first_output, first_cache), (second_output, second_cache) = executions[0], executions[-1]
            maximum, relative_l2 = surface_error_metrics(first_output, oracle_output)
            repeated_output_exact = bool(np.array_equal(first_output.view(np.uint16), second_output.view(np.uint16)))
            repeated_cache_exact = bool(np.array_equal(first_cache.view(np.uint16), second_cache.view(np.uint16)))
            cache_exact = bool(np.array_equal(first_cache.view(np.uint16), oracle_cache.view(np.uint16)))
            passed = (repeated_output_exact and repeated_cache_exact and (cache_exact or not settings["require_exact_cache"])
                      and maximum <= settings["output_maximum_absolute_error"] and relative_l2 <= settings["output_relative_l2_error"])
            observation = SurfaceCorrectnessObservation(
                seed=seed, input_sha256=tuple(array_sha256(np.asarray(v)) for v in host_inputs), output_sha256=array_sha256(first_output),
                repeat_output_sha256=array_sha256(second_output), oracle_output_sha256=array_sha256(oracle_output),
                cache_sha256=array_sha256(first_cache), repeat_cache_sha256=array_sha256(second_cache), oracle_cache_sha256=array_sha256(oracle_cache),
                repeated_output_exact=repeated_output_exact, repeated_cache_exact=repeated_cache_exact, cache_exact=cache_exact,
                maximum_absolute_error=maximum, relative_l2_error=relative_l2, passed=passed)
            seed_root = output_dir / "correctness" / f"seed-{seed}"
            seed_root.mkdir(parents=True)
            for name, value in (("output", first_output), ("repeat_output", second_output), ("oracle_output", oracle_output)):
                np.save(seed_root / f"{name}.npy", value.view(np.uint16))
                artifacts.append(run_artifacts.reference_of(output_dir, seed_root / f"{name}.npy", f"correctness_{name}"))
            run_artifacts.write_json(output_dir, seed_root / "observation.json", asdict(observation), "correctness_observation", artifacts)
            observations.append(observation)
            if not passed:
                record(RunState.REJECTED, {"reason": "numerical mismatch", "seed": seed, "maximum_absolute_error": maximum,
                                           "relative_l2_error": relative_l2, "cache_exact": cache_exact})
                break
        # Every process learns the verdict before anyone goes on to the timing part.
        verdict = [all(o.passed for o in observations) if leader else None]
        if executor.world > 1:
            torch.distributed.broadcast_object_list(verdict, src=0)
        if not verdict[0]:
            raise ValueError(f"INKLING_SHARDED_RPA_CORRECTNESS_FAILED observation={observations[-1] if observations else None}")
        if leader:
            run_artifacts.write_json(output_dir, output_dir / "correctness.json", [asdict(o) for o in observations], "correctness", artifacts)
        record(RunState.CORRECT, {"seeds": [str(s) for s in settings["correctness_seeds"]]})

        # Timing: every position times its own chained calls; the surface's sample is the slowest position's.
        timing_inputs = workloads.inkling_sharded_fused_rpa_inputs(settings["timing_seed"])
        per_position = {}
        for rank in executor.owned:
            shard = tuple(np.ascontiguousarray(v) for v in plan.shard_inputs(timing_inputs, plan.mesh_position(rank)))
            per_position[rank] = plan.timing_rounds(executor.executable, shard, warmup_iterations=settings["warmup_iterations"],
                                                    timing_rounds=settings["timing_rounds"], samples_per_round=settings["samples_per_round"])
        if executor.world > 1:
            gathered = [None] * executor.world if leader else None
            torch.distributed.gather_object(per_position, gathered, dst=0)
            if leader:
                per_position = {rank: rounds for part in gathered for rank, rounds in part.items()}
        if not leader:
            return {}
        rounds = []
        for index in range(settings["timing_rounds"]):
            samples = tuple(max(per_position[rank][index]["samples_ns"][k] for rank in per_position) for k in range(settings["samples_per_round"]))
            rounds.append({"round_index": index, "samples_ns": samples, "median_ns": float(statistics.median(samples))})
        run_artifacts.write_json(output_dir, output_dir / "rounds.json", rounds, "timing_rounds", artifacts)
        medians = sorted(r["median_ns"] for r in rounds)
        record(RunState.TIMED, {"median_of_round_medians_ns": statistics.median(medians), "rounds": len(rounds)})
        artifacts.append(run_artifacts.reference_of(output_dir, ledger_path, "execution_ledger"))
        result = {
            "run_id": run_id, "execution": executor.execution, "process_count": executor.world, "device_kind": torch.cuda.get_device_name(device),
            "schedule_sha256": plan.schedule_sha256, "mesh_shape": list(plan.mesh_shape),
            "correctness": [asdict(o) for o in observations], "passed": all(o.passed for o in observations),
            "round_medians_ns": [r["median_ns"] for r in rounds], "median_ns": statistics.median(medians),
            "minimum_round_median_ns": medians[0], "maximum_round_median_ns": medians[-1],
            "artifacts": [asdict(a) for a in artifacts],
        }
        (output_dir / "result.json").write_text(json.dumps(result, indent=2, sort_keys=True) + "\n")
        return result
    finally:
        executor.close()
