"""Receipts for run bundles of the CUDA backend: ``finalize-matmul-run`` and ``verify-matmul-bundle``.

Mirrors what the reference's receipt checks for a distributed-matmul run (src/tpu_cake/receipt.py):
every artifact of the bundle re-hashed against the run result (:296-320), the executed code matching
the declared collective strategy (:173-293; there on StableHLO / compiler HLO text, here on the kernel
manifest the runner wrote and, when a profiler capture is attached, on the kernels that actually
launched), the cost model recomputed from the invocation (:600-645), a roofline input / metrics pair
with the reference's field names and formulae recomputed to 1e-12 (:647-709) and the measured-to-floor
ratios (src/tpu_cake/receipt_metrics.py:111-187). A receipt is refused for a run that did not pass its
correctness check, and validation refuses a bundle in which any byte changed after finalisation.
"""

from __future__ import annotations

import hashlib
import json
import math
from dataclasses import asdict
from decimal import Decimal
from pathlib import Path

from . import cost_model, cuda_lowering, profile_evidence, schedule_lowering, workloads
from .identity import semantic_sha256

RECEIPT_SCHEMA = "cake-b200-run-receipt-v1"


def _sha256(path: Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        for block in iter(lambda: handle.read(1 << 20), b""):
            digest.update(block)
    return digest.hexdigest()


def _artifact(root: Path, relative: str, role: str) -> dict:
    path = root / relative
    return {"path": relative, "size_bytes": path.stat().st_size, "sha256": _sha256(path), "role": role}


def expected_kernels(strategy: str, mesh_size: int, tile_n: int) -> tuple[list[str], tuple[str, ...]]:
    """(kernels the manifest must list, kernel-name fragments that must not launch) for a strategy."""
    main = f"cake_matmul_rs_sm100<{tile_n}>"
    if mesh_size == 1:
        return [main], ("cake_reduce_slots_sm100", "ncclDevKernel")
    if strategy == cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER.value:
        return [main], ("cake_reduce_slots_sm100",)
    return [main, "cake_reduce_slots_sm100"], ("ncclDevKernel_ReduceScatter",)


def required_profile_markers(strategy: str, mesh_size: int, tile_n: int, execution: str) -> tuple[str, ...]:
    """Kernel-name fragments a profile of the run must contain. One process per GPU launches the
    contraction alone (its last warps are the slot reduction); only the one-GPU emulation of a mesh
    launches the reduction as a kernel of its own."""
    wanted, _ = expected_kernels(strategy, mesh_size, tile_n)
    markers = [wanted[0].split("<")[0]]
    if len(wanted) > 1 and execution == "emulated-on-one-gpu":
        markers.append(wanted[1])
    return tuple(markers)


def _validate_strategy(manifest: dict, strategy: str, mesh_size: int, tile_n: int) -> None:
    wanted, _ = expected_kernels(strategy, mesh_size, tile_n)
    if list(manifest.get("kernels", ())) != wanted:
        raise ValueError(f"KERNEL_MANIFEST_DOES_NOT_MATCH_STRATEGY expected={wanted} observed={manifest.get('kernels')}")


def _plan_of(invocation: dict):
    from .runner import lower_invocation

    return lower_invocation(invocation)[2]


def _cost_payload(report: cost_model.CostModelReport) -> dict:
    return {**asdict(report.counts), "compute_ns": str(report.compute_ns), "memory_ns": str(report.memory_ns),
            "communication_ns": str(report.communication_ns), "lower_bound_ns": str(report.lower_bound_ns),
            "limiting_resource": report.limiting_resource}


def roofline_metrics(model_input: dict) -> dict:
    """The reference's roofline arithmetic (src/tpu_cake/receipt.py:673-700) on an input document."""
    hardware, workload = model_input["hardware"], model_input["workload"]
    operations = float(workload["operations"])
    total_bytes = float(workload["bytes_read"] + workload["bytes_written"])
    compute_peak = float(hardware["compute_peak_ops_s"]) * float(hardware["effective_compute_fraction"])
    memory_peak = float(hardware["memory_bandwidth_bytes_s"]) * float(hardware["effective_memory_fraction"])
    measured = float(workload["measured_time_s"])
    metrics = {
        "operations": operations, "total_bytes": total_bytes, "arithmetic_intensity_ops_per_byte": operations / total_bytes,
        "effective_compute_peak_ops_s": compute_peak, "effective_memory_bandwidth_bytes_s": memory_peak,
        "compute_time_s": operations / compute_peak, "memory_time_s": total_bytes / memory_peak,
        "lower_bound_time_s": max(operations / compute_peak, total_bytes / memory_peak), "measured_time_s": measured,
        "measured_throughput_ops_s": operations / measured,
    }
    metrics["attainable_throughput_ops_s"] = min(compute_peak, memory_peak * metrics["arithmetic_intensity_ops_per_byte"])
    metrics["attainable_efficiency"] = metrics["measured_throughput_ops_s"] / metrics["attainable_throughput_ops_s"]
    metrics["peak_efficiency"] = metrics["measured_throughput_ops_s"] / compute_peak
    metrics["headroom_to_attainable"] = metrics["attainable_throughput_ops_s"] / metrics["measured_throughput_ops_s"]
    return metrics


def _load_bundle(root: Path) -> tuple[dict, dict, dict]:
    result = json.loads((root / "result.json").read_text())
    invocation = json.loads((root / "invocation.json").read_text())
    manifest = json.loads((root / "kernel_manifest.json").read_text())
    return result, invocation, manifest


def _check_result_artifacts(root: Path, result: dict) -> None:
    for artifact in result["artifacts"]:
        path = root / artifact["path"]
        if not path.is_file():
            raise ValueError(f"ARTIFACT_MISSING path={artifact['path']}")
        if path.stat().st_size != artifact["size_bytes"] or _sha256(path) != artifact["sha256"]:
            raise ValueError(f"ARTIFACT_CHANGED path={artifact['path']}")


def finalize_matmul_run(root: Path, *, profile_csv: Path | None = None) -> dict:
    """Checks a finished run bundle and writes ``roofline/input.json``, ``roofline/metrics.json`` and
    ``receipt.json`` into it. With ``profile_csv`` (an ``ncu --csv`` launch list of the same run) the
    capture must contain the strategy's kernels and none of the forbidden ones."""
    root = Path(root)
    result, invocation, manifest = _load_bundle(root)
    if not result["passed"] or result["median_ns"] is None:
        raise ValueError("RECEIPT_REQUIRES_A_PASSED_TIMED_RUN")
    _check_result_artifacts(root, result)
    plan = _plan_of(invocation)
    if plan.schedule_sha256 != result["schedule_sha256"] or plan.source_sha256() != result["cuda_source_sha256"]:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    # The saved IR text and lowered source themselves, not only their recorded hashes.
    saved_plan = cuda_lowering.validate_saved_cuda_plan(root / "physical.xdsl", root / "lowered_cuda.py", schedule_sha256=result["schedule_sha256"],
                                                        source_sha256=result["cuda_source_sha256"])
    if saved_plan != plan:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    _validate_strategy(manifest, invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n)
    report = cost_model.estimate_distributed_matmul(plan)
    if json.loads((root / "cost_model.json").read_text()) != _cost_payload(report):
        raise ValueError("COST_MODEL_DOES_NOT_REPLAY")
    hardware = cost_model.B200_MEASURED
    model_input = {
        "hardware": {"name": hardware.name, "compute_peak_ops_s": hardware.compute_flops_per_second,
                     "memory_bandwidth_bytes_s": hardware.hbm_bytes_per_second, "effective_compute_fraction": 1.0,
                     "effective_memory_fraction": 1.0},
        "workload": {"operations": report.counts.operations_per_device, "bytes_read": report.counts.hbm_read_bytes_per_device,
                     "bytes_written": report.counts.hbm_write_bytes_per_device, "measured_time_s": result["median_ns"] / 1_000_000_000},
    }
    (root / "roofline").mkdir(exist_ok=True)
    (root / "roofline" / "input.json").write_text(json.dumps(model_input, indent=2) + "\n")
    metrics = roofline_metrics(model_input)
    (root / "roofline" / "metrics.json").write_text(json.dumps(metrics, indent=2) + "\n")
    artifacts = [dict(a) for a in result["artifacts"]]
    artifacts.append(_artifact(root, "result.json", "timing_result"))
    artifacts.append(_artifact(root, "roofline/input.json", "roofline_input"))
    artifacts.append(_artifact(root, "roofline/metrics.json", "roofline_metrics"))
    profile = {"attached": False}
    if profile_csv is not None:
        _, forbidden = expected_kernels(invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n)
        expectation = profile_evidence.ProfileExpectation(
            name=f"matmul-{invocation['collective_strategy']}", require_tensor_core_activity=False,
            required_timed_hlo_markers=required_profile_markers(invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n, result["execution"]),
            forbidden_timed_hlo_fragments=forbidden,
        )
        assessment = profile_evidence.assess_capture(Path(profile_csv), expectation)
        if not assessment.accepted:
            raise ValueError("PROFILE_CAPTURE_REJECTED " + ",".join(f.code for f in assessment.findings))
        target = root / "profile" / "launches.csv"
        target.parent.mkdir(exist_ok=True)
        target.write_bytes(Path(profile_csv).read_bytes())
        artifacts.append(_artifact(root, "profile/launches.csv", "profile_capture"))
        profile = {"attached": True, "marker_launches": assessment.marker_launches,
                   "marker_time_ns": assessment.marker_time_ns}
    floor_ns = float(report.lower_bound_ns)
    receipt = {
        "schema": RECEIPT_SCHEMA, "run_id": result["run_id"], "collective_strategy": invocation["collective_strategy"],
        "mesh_size": invocation["mesh_size"], "execution": result["execution"], "device_kind": result["device_kind"],
        "schedule_sha256": result["schedule_sha256"], "cuda_source_sha256": result["cuda_source_sha256"],
        "kernel_manifest_sha256": result["kernel_manifest_sha256"], "artifacts": artifacts, "profile": profile,
        "metrics": {
            "median_ns": result["median_ns"], "p90_ns": result["p90_ns"],
            "roofline_two_resource_time_floor_s": metrics["lower_bound_time_s"],
            "measured_to_two_resource_floor": metrics["measured_time_s"] / metrics["lower_bound_time_s"],
            "compute_hbm_link_floor_ns": floor_ns, "measured_to_compute_hbm_link_floor": result["median_ns"] / floor_ns,
            "peak_efficiency": metrics["peak_efficiency"],
        },
    }
    receipt["receipt_id"] = semantic_sha256("run-receipt", json.dumps(receipt, sort_keys=True))
    (root / "receipt.json").write_text(json.dumps(receipt, indent=2) + "\n")
    return receipt


def validate_receipt(root: Path) -> dict:
    """Re-derives everything a receipt states from the bundle's files; raises ValueError on the first
    disagreement."""
    root = Path(root)
    receipt = json.loads((root / "receipt.json").read_text())
    if receipt.get("schema") != RECEIPT_SCHEMA:
        raise ValueError("RECEIPT_SCHEMA_UNKNOWN")
    body = {key: value for key, value in receipt.items() if key != "receipt_id"}
    if receipt.get("receipt_id") != semantic_sha256("run-receipt", json.dumps(body, sort_keys=True)):
        raise ValueError("RECEIPT_ID_MISMATCH")
    for artifact in receipt["artifacts"]:
        path = root / artifact["path"]
        if not path.is_file() or path.stat().st_size != artifact["size_bytes"] or _sha256(path) != artifact["sha256"]:
            raise ValueError(f"ARTIFACT_CHANGED path={artifact['path']}")
    result, invocation, manifest = _load_bundle(root)
    if result["run_id"] != receipt["run_id"] or not result["passed"]:
        raise ValueError("RECEIPT_DOES_NOT_MATCH_RUN")
    plan = _plan_of(invocation)
    if plan.schedule_sha256 != receipt["schedule_sha256"] or plan.source_sha256() != receipt["cuda_source_sha256"]:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    # The saved IR text and lowered source themselves, not only their recorded hashes.
    saved_plan = cuda_lowering.validate_saved_cuda_plan(root / "physical.xdsl", root / "lowered_cuda.py", schedule_sha256=receipt["schedule_sha256"],
                                                        source_sha256=receipt["cuda_source_sha256"])
    if saved_plan != plan:
        raise ValueError("LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY")
    _validate_strategy(manifest, invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n)
    report = cost_model.estimate_distributed_matmul(plan)
    model_input = json.loads((root / "roofline" / "input.json").read_text())
    workload, hardware = model_input["workload"], model_input["hardware"]
    if float(workload["operations"]) != report.counts.operations_per_device or float(workload["bytes_read"] + workload["bytes_written"]) != (
        report.counts.hbm_read_bytes_per_device + report.counts.hbm_write_bytes_per_device
    ):
        raise ValueError("ROOFLINE_WORKLOAD_DOES_NOT_MATCH_COST_MODEL")
    if (float(hardware["compute_peak_ops_s"]) != cost_model.B200_MEASURED.compute_flops_per_second
            or float(hardware["memory_bandwidth_bytes_s"]) != cost_model.B200_MEASURED.hbm_bytes_per_second):
        raise ValueError("ROOFLINE_HARDWARE_DOES_NOT_MATCH_COST_MODEL")
    saved = json.loads((root / "roofline" / "metrics.json").read_text())
    for name, value in roofline_metrics(model_input).items():
        if name not in saved or not math.isclose(float(saved[name]), value, rel_tol=1e-12, abs_tol=1e-15):
            raise ValueError(f"ROOFLINE_METRIC_MISMATCH field={name}")
    if not math.isclose(float(workload["measured_time_s"]), result["median_ns"] / 1_000_000_000, rel_tol=0, abs_tol=1e-15):
        raise ValueError("ROOFLINE_TIMING_SOURCE_MISMATCH")
    if receipt["profile"]["attached"]:
        _, forbidden = expected_kernels(invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n)
        expectation = profile_evidence.ProfileExpectation(
            name="revalidation", require_tensor_core_activity=False,
            required_timed_hlo_markers=required_profile_markers(invocation["collective_strategy"], invocation["mesh_size"], plan.tile_n, result["execution"]),
            forbidden_timed_hlo_fragments=forbidden,
        )
        if not profile_evidence.assess_capture(root / "profile" / "launches.csv", expectation).accepted:
            raise ValueError("PROFILE_CAPTURE_REJECTED")
    return receipt


# ------------------------------------------------------------------------------ three-phase bundle

BUNDLE_SCHEMA = "cake-b200-run-bundle-v1"
_PHASES = ("timing", "trace", "counters")
_SAME_ACROSS_PHASES = ("schedule_sha256", "cuda_source_sha256", "kernel_manifest_sha256", "lhs_sha256", "rhs_sha256", "output_sha256",
                       "collective_strategy", "device_count", "execution", "device_kind")


def finalize_matmul_bundle(root: Path, *, trace_profile: Path, counters_profile: Path) -> dict:
    """A run bundle is three runs of one invocation -- ``timing/``, ``trace/`` and ``counters/`` under
    ``root`` -- that must agree on everything but the mode: the same schedule, lowered code, kernel
    manifest, input and output hashes (src/tpu_cake/run_bundle.py:88-112). The timing run gets its
    receipt; the trace capture (kernel durations only) must show the strategy's kernels and none of
    the forbidden ones; the counters capture must in addition carry tensor-pipe activity and DRAM
    byte counters. Writes ``bundle.json`` and returns it."""
    root = Path(root)
    loaded = {}
    for phase in _PHASES:
        directory = root / phase
        if not (directory / "result.json").is_file():
            raise ValueError(f"BUNDLE_PHASE_MISSING phase={phase}")
        result, invocation, manifest = _load_bundle(directory)
        if result["mode"] != phase or invocation["mode"] != phase:
            raise ValueError(f"BUNDLE_PHASE_MODE_MISMATCH phase={phase} mode={result['mode']}")
        if not result["passed"]:
            raise ValueError(f"BUNDLE_PHASE_NOT_CORRECT phase={phase}")
        _check_result_artifacts(directory, result)
        contract = json.loads((directory / "profiler_config.json").read_text())
        from . import run_artifacts

        run_artifacts.validate_profiler_contract(contract)
        if contract["mode"] != phase:
            raise ValueError(f"PROFILER_CONTRACT_VIOLATION phase={phase} profiler_config is for {contract['mode']}")
        loaded[phase] = (result, invocation, manifest)
    reference_result, reference_invocation, _ = loaded["timing"]
    for phase in ("trace", "counters"):
        result, invocation, _ = loaded[phase]
        for name in _SAME_ACROSS_PHASES:
            if result[name] != reference_result[name]:
                raise ValueError(f"BUNDLE_IDENTITY_MISMATCH phase={phase} field={name}")
        if {k: v for k, v in invocation.items() if k != "mode"} != {k: v for k, v in reference_invocation.items() if k != "mode"}:
            raise ValueError(f"BUNDLE_INVOCATION_MISMATCH phase={phase}")
        if result["samples_ns"]:
            raise ValueError(f"BUNDLE_PHASE_CARRIES_HOST_TIMINGS phase={phase}")
    receipt = finalize_matmul_run(root / "timing")
    plan = _plan_of(reference_invocation)
    strategy, mesh_size = reference_invocation["collective_strategy"], reference_invocation["mesh_size"]
    _, forbidden = expected_kernels(strategy, mesh_size, plan.tile_n)
    markers = required_profile_markers(strategy, mesh_size, plan.tile_n, reference_result["execution"])
    assessments = {}
    for phase, capture, counters in (("trace", trace_profile, False), ("counters", counters_profile, True)):
        expectation = profile_evidence.ProfileExpectation(
            name=f"matmul-{strategy}-{phase}", require_tensor_core_activity=counters, require_hbm_read_counters=counters,
            require_hbm_write_counters=counters, required_timed_hlo_markers=markers, forbidden_timed_hlo_fragments=forbidden,
        )
        assessment = profile_evidence.assess_capture(Path(capture), expectation)
        if not assessment.accepted:
            raise ValueError(f"PROFILE_CAPTURE_REJECTED phase={phase} " + ",".join(f.code for f in assessment.findings))
        if not counters:
            evidence = profile_evidence.read_ncu_csv(Path(capture).read_text())
            if any(name.startswith(("dram__", "sm__")) for name in evidence.metric_names):
                raise ValueError("PROFILER_CONTRACT_VIOLATION phase=trace capture carries hardware counters")
        target = root / phase / "profile" / "launches.csv"
        target.parent.mkdir(exist_ok=True)
        target.write_bytes(Path(capture).read_bytes())
        assessments[phase] = {"capture": _artifact(root, f"{phase}/profile/launches.csv", "profile_capture"),
                              "marker_launches": assessment.marker_launches, "marker_time_ns": assessment.marker_time_ns}
    bundle = {
        "schema": BUNDLE_SCHEMA, "run_ids": {phase: loaded[phase][0]["run_id"] for phase in _PHASES},
        "identities": {name: reference_result[name] for name in _SAME_ACROSS_PHASES}, "timing_receipt_id": receipt["receipt_id"],
        "profiles": assessments,
    }
    bundle["bundle_id"] = semantic_sha256("run-bundle", json.dumps(bundle, sort_keys=True))
    (root / "bundle.json").write_text(json.dumps(bundle, indent=2) + "\n")
    return bundle
