"""Profile reader for the CUDA backend: Nsight Compute CSV -> capture evidence -> acceptance.

The reference reads XProf captures (XPlane + hlo_stats) and rejects those that do not contain the
intended work (src/tpu_cake/xprof_evidence.py:286-447): too few device planes, no Tensor Core
events, no device events, missing HBM / cycle counters, no timed program, a required marker absent,
a forbidden fragment present. This module applies the same rejections to what ``ncu --csv`` writes
(long format: one row per kernel launch and metric). The expectation keeps the reference's field
names (``minimum_tpu_device_planes``, ``required_timed_hlo_markers``, ...; src/tpu_cake/contracts.py:96-107),
read for GPUs as: device planes -> distinct device ordinals with kernel records; Tensor Core
activity -> a tensor-pipe metric above zero on a marker kernel; markers -> substrings of kernel
names; forbidden fragments -> kernel-name substrings that must not occur (for example
``ncclDevKernel_ReduceScatter`` when the fused epilogue is the declared strategy). A capture that
cannot be read is rejected, never accepted.
"""

from __future__ import annotations

import csv
import io
from dataclasses import dataclass, field
from pathlib import Path

TENSOR_METRICS = ("sm__pipe_tensor_cycles_active", "sm__inst_executed_pipe_tensor", "sm__pipe_tensor_op")
HBM_READ_METRIC = "dram__bytes_read.sum"
HBM_WRITE_METRIC = "dram__bytes_write.sum"
CYCLE_METRICS = ("sm__cycles_elapsed", "gpc__cycles_elapsed", "sm__cycles_active")
_UNIT_TO_NS = {"ns": 1.0, "nsecond": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6, "s": 1e9, "second": 1e9}


@dataclass(frozen=True)
class ProfileExpectation:
    name: str
    minimum_tpu_device_planes: int = 1
    require_tensor_core_activity: bool = True
    require_hbm_read_counters: bool = False
    require_hbm_write_counters: bool = False
    require_cycle_counters: bool = False
    required_timed_hlo_markers: tuple[str, ...] = ()
    forbidden_timed_hlo_fragments: tuple[str, ...] = ()
    expected_marker_launches: int | None = None  # launches of the first marker kernel, if pinned


@dataclass
class KernelRecord:
    launch_id: str
    name: str
    device: str
    metrics: dict[str, float] = field(default_factory=dict)

    @property
    def duration_ns(self) -> float:
        return self.metrics.get("gpu__time_duration.sum", 0.0)


@dataclass(frozen=True)
class CaptureEvidence:
    kernels: tuple[KernelRecord, ...]
    metric_names: frozenset[str]

    @property
    def devices(self) -> frozenset[str]:
        return frozenset(k.device for k in self.kernels)


@dataclass(frozen=True)
class Finding:
    code: str
    message: str
    evidence: tuple[str, ...] = ()


@dataclass(frozen=True)
class CaptureAssessment:
    accepted: bool
    findings: tuple[Finding, ...]
    marker_launches: dict[str, int]
    marker_time_ns: dict[str, float]


def _number(text: str) -> float:
    cleaned = text.replace(",", "").strip()
    try:
        return float(cleaned)
    except ValueError:
        return float("nan")


def read_ncu_csv(text: str) -> CaptureEvidence:
    """Parses ``ncu --csv`` output (long format). Lines before the header (``==PROF==`` ...) are skipped."""
    lines = [line for line in text.splitlines() if line and not line.startswith("==")]
    start = next((i for i, line in enumerate(lines) if line.startswith('"ID"')), None)
    if start is None:
        raise ValueError("PROFILE_CAPTURE_UNREADABLE no ncu CSV header")
    reader = csv.DictReader(io.StringIO("\n".join(lines[start:])))
    needed = {"ID", "Kernel Name", "Device", "Metric Name", "Metric Unit", "Metric Value"}
    if not needed.issubset(reader.fieldnames or ()):
        raise ValueError(f"PROFILE_CAPTURE_UNREADABLE missing columns {sorted(needed - set(reader.fieldnames or ()))}")
    kernels: dict[str, KernelRecord] = {}
    metric_names: set[str] = set()
    for row in reader:
        record = kernels.setdefault(row["ID"], KernelRecord(row["ID"], row["Kernel Name"], row["Device"]))
        value = _number(row["Metric Value"])
        name = row["Metric Name"]
        if name == "gpu__time_duration.sum":
            value *= _UNIT_TO_NS.get(row["Metric Unit"], 1.0)
        record.metrics[name] = value
        metric_names.add(name)
    return CaptureEvidence(tuple(kernels.values()), frozenset(metric_names))


def assess_evidence(capture: CaptureEvidence, expectation: ProfileExpectation) -> CaptureAssessment:
    findings: list[Finding] = []
    if len(capture.devices) < expectation.minimum_tpu_device_planes:
        findings.append(Finding("INSUFFICIENT_GPU_DEVICES", "capture does not contain kernel records from the required number of GPUs",
                                (f"observed={len(capture.devices)}", f"required={expectation.minimum_tpu_device_planes}")))
    if not capture.kernels:
        findings.append(Finding("INSUFFICIENT_DEVICE_EVENTS", "capture contains no kernel launches", ("observed=0", "required=1")))
    markers = expectation.required_timed_hlo_markers
    launches = {m: sum(m in k.name for k in capture.kernels) for m in markers}
    time_ns = {m: sum(k.duration_ns for k in capture.kernels if m in k.name) for m in markers}
    for marker in markers:
        if launches[marker] == 0:
            findings.append(Finding("REQUIRED_TIMED_MARKER_MISSING", f"required kernel marker {marker!r} is absent from the capture"))
    for fragment in expectation.forbidden_timed_hlo_fragments:
        hits = sum(fragment in k.name for k in capture.kernels)
        if hits:
            findings.append(Finding("FORBIDDEN_TIMED_FRAGMENT_PRESENT", f"forbidden kernel {fragment!r} was launched", (f"launches={hits}",)))
    if expectation.expected_marker_launches is not None and markers and launches[markers[0]] != expectation.expected_marker_launches:
        findings.append(Finding("MARKER_LAUNCH_COUNT_MISMATCH", "the marker kernel was not launched the expected number of times",
                                (f"observed={launches[markers[0]]}", f"required={expectation.expected_marker_launches}")))
    if expectation.require_tensor_core_activity:
        scope = [k for k in capture.kernels if any(m in k.name for m in markers)] if markers else list(capture.kernels)
        active = any(value > 0 for k in scope for name, value in k.metrics.items() if name.startswith(TENSOR_METRICS))
        if not active:
            findings.append(Finding("NO_TENSOR_CORE_ACTIVITY", "no tensor-pipe activity was recorded for the marked kernels"))
    counter_rules = (
        (expectation.require_hbm_read_counters, any(n.startswith(HBM_READ_METRIC) for n in capture.metric_names), "HBM_READ"),
        (expectation.require_hbm_write_counters, any(n.startswith(HBM_WRITE_METRIC) for n in capture.metric_names), "HBM_WRITE"),
        (expectation.require_cycle_counters, any(n.startswith(CYCLE_METRICS) for n in capture.metric_names), "CYCLE"),
    )
    for required, present, label in counter_rules:
        if required and not present:
            findings.append(Finding(f"MISSING_{label}_COUNTERS", f"capture has no {label.lower()} hardware counters"))
    return CaptureAssessment(not findings, tuple(findings), launches, time_ns)


def assess_capture(path: Path, expectation: ProfileExpectation) -> CaptureAssessment:
    """Reads an ncu CSV file and assesses it; an unreadable or missing capture is a rejection."""
    try:
        capture = read_ncu_csv(Path(path).read_text())
    except (OSError, ValueError) as error:
        return CaptureAssessment(False, (Finding("PROFILE_CAPTURE_UNREADABLE", str(error)),), {}, {})
    return assess_evidence(capture, expectation)
