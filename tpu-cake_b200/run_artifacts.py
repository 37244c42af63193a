"""Pieces of a run bundle that the matmul runner and the RPA runner share: run modes and their
profiler contract, the source-state record, the experiment record and small file helpers.

Counterparts in the reference: ``RunMode`` (src/tpu_cake/runner.py:54-57), ``_profiler_contract`` /
``_profiler_options`` (:144-217 -- timing and trace runs may never carry counter options),
``_source_state`` (:384-437), ``experiment.json`` (src/tpu_cake/contracts.py:275-296).

On the GPU the profiler is ``ncu`` wrapped around the runner's process, so a trace or counters run
cannot read its own capture: it records which ``ncu`` invocation must wrap it, runs the measured
calls without host timing, and ends in TRACED / COUNTERED; the launch list ``ncu --csv`` wrote is
attached and assessed when the bundle is finalised.
"""

from __future__ import annotations

import hashlib
import json
import os
import subprocess
from dataclasses import dataclass
from enum import StrEnum
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPOSITORY_ROOT = PACKAGE_DIR.parent

TRACE_METRICS = ("gpu__time_duration.sum",)
COUNTER_METRICS = (
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
)


class RunMode(StrEnum):
    TIMING = "timing"
    TRACE = "trace"
    COUNTERS = "counters"


@dataclass(frozen=True)
class ArtifactReference:
    path: str
    size_bytes: int
    sha256: str
    role: str


def sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        for block in iter(lambda: handle.read(1 << 20), b""):
            digest.update(block)
    return digest.hexdigest()


def reference_of(root: Path, path: Path, role: str) -> ArtifactReference:
    return ArtifactReference(str(path.relative_to(root)), path.stat().st_size, sha256_file(path), role)


def write_text(root: Path, path: Path, text: str, role: str, artifacts: list[ArtifactReference]) -> ArtifactReference:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(text)
    reference = reference_of(root, path, role)
    artifacts.append(reference)
    return reference


def write_json(root: Path, path: Path, payload, role: str, artifacts: list[ArtifactReference]) -> ArtifactReference:
    return write_text(root, path, json.dumps(payload, indent=2, sort_keys=True) + "\n", role, artifacts)


def profiler_contract(mode: RunMode) -> dict:
    """What must wrap the run's process for ``mode``. A timing run has no profiler; a trace run
    collects kernel durations only (one pass, nothing replayed); only a counters run may ask for
    hardware counters (several passes per launch, so its durations are not timings)."""
    mode = RunMode(mode)
    if mode is RunMode.TIMING:
        return {"mode": mode.value, "profiler": None, "arguments": [], "counters": False}
    metrics = TRACE_METRICS if mode is RunMode.TRACE else COUNTER_METRICS
    return {
        "mode": mode.value, "profiler": "ncu", "counters": mode is RunMode.COUNTERS,
        "arguments": ["--metrics", ",".join(metrics), "--clock-control", "none", "--csv", "--log-file", "launches.csv"],
        "capture": "launches.csv: one row per launch and metric, attached when the bundle is finalised",
    }


def validate_profiler_contract(contract: dict) -> None:
    """Timing and trace runs may never carry counter options (src/tpu_cake/runner.py:144-217)."""
    mode = RunMode(contract["mode"])
    arguments = " ".join(contract.get("arguments", ()))
    asks_for_counters = any(metric in arguments for metric in COUNTER_METRICS[1:]) or "--set" in arguments or "--section" in arguments
    if mode is RunMode.TIMING and (contract.get("profiler") is not None or contract.get("arguments")):
        raise ValueError("PROFILER_CONTRACT_VIOLATION mode=timing carries profiler options")
    if mode is not RunMode.COUNTERS and (asks_for_counters or contract.get("counters")):
        raise ValueError(f"PROFILER_CONTRACT_VIOLATION mode={mode.value} carries counter options")
    if mode is not RunMode.TIMING and "--clock-control none" not in arguments:
        raise ValueError(f"PROFILER_CONTRACT_VIOLATION mode={mode.value} would lock the GPU clocks")


def profiler_attached() -> bool:
    """Whether this process runs under NVIDIA's compute profiler (it injects itself through these)."""
    return any(name in os.environ for name in ("NV_COMPUTE_PROFILER_PERFWORKS_DIR", "NV_NSIGHT_INJECTION_PORT_BASE")) or \
        "nsight-compute" in os.environ.get("CUDA_INJECTION64_PATH", "").lower()


def _git(*arguments: str) -> str | None:
    try:
        done = subprocess.run(["git", "-C", str(REPOSITORY_ROOT), *arguments], capture_output=True, text=True, timeout=30, check=False)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return done.stdout if done.returncode == 0 else None


def source_state(root: Path, artifacts: list[ArtifactReference]) -> dict:
    """``source_state.json`` + ``source_diff.patch``: the commit the code was run from, whether the
    tree was clean, and the hash of every source file of the backend, so that a bundle names the
    code that produced it even when git is not available where it ran."""
    head = _git("rev-parse", "HEAD")
    diff = _git("diff", "HEAD") if head is not None else None
    files = {}
    for path in sorted(list(PACKAGE_DIR.glob("*.py")) + list((PACKAGE_DIR / "csrc").glob("*")) + [REPOSITORY_ROOT / "include" / "cake_abi.h"]):
        if path.is_file():
            files[str(path.relative_to(REPOSITORY_ROOT))] = sha256_file(path)
    state = {
        "git_head": head.strip() if head else None, "git_available": head is not None,
        "dirty": bool(diff.strip()) if diff is not None else None, "source_files": files,
        "source_tree_sha256": hashlib.sha256(json.dumps(files, sort_keys=True).encode()).hexdigest(),
    }
    write_text(root, root / "source_diff.patch", diff or "", "source_diff", artifacts)
    write_json(root, root / "source_state.json", state, "source_state", artifacts)
    return state


def experiment_record(*, workload: dict, schedule_sha256: str, warmup_iterations: int, measured_iterations: int,
                      profile_expectation: dict, tolerance: dict) -> dict:
    """``experiment.json``: the workload, the target, the benchmark protocol and what a profile of the
    run must show (src/tpu_cake/contracts.py: KernelExperiment; field names kept, values for B200)."""
    return {
        "workload": workload,
        "target": {"accelerator": "B200", "topology": "nvlink5-nvswitch", "runtime_target": "cake-b200 sm_100a kernels",
                   "shared_memory_budget_bytes_per_sm": 232448, "tensor_memory_columns_per_sm": 512},
        "benchmark": {"warmup_iterations": warmup_iterations, "measured_iterations": measured_iterations,
                      "synchronization": "synchronize the device after every call", "statistic": "median wall duration"},
        "numerical": tolerance,
        "profile": profile_expectation,
        "schedule_sha256": schedule_sha256,
    }
