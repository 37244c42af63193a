"""Tile search for the distributed matmul on the CUDA backend: the ``search-matmul`` target.

Mirrors the reference's search driver (src/tpu_cake/search.py): the contract
(``MatmulSearchContract``, :49-77: mesh, shape, iterations, at least 5 rounds, unique candidates that
divide M and N), the protocol (:499-644: every round runs every candidate, the order reversed on odd
rounds; all runs must pass the oracle, share inputs and give one output hash per candidate) and the
statistics (:109-128, :578-628: per-round medians, paired improvement over the first candidate, a
bootstrap interval of the median paired improvement seeded from the candidate's name, promotion only
when the interval's low end clears ``minimum_practical_improvement``). Candidates here name a CTA
output tile of the sm_100a kernel (tile_m 128, tile_n 64 / 128 / 256) and the collective strategy is
part of the contract instead of being fixed to the compiler's collective (:411-416).
"""

from __future__ import annotations

import hashlib
import json
import re
import statistics
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable

import numpy as np

from .identity import semantic_sha256


@dataclass(frozen=True)
class MatmulSearchCandidate:
    name: str
    tile_m: int
    tile_n: int

    def __post_init__(self) -> None:
        if not re.fullmatch(r"[a-z0-9-]+", self.name):
            raise ValueError(f"candidate name {self.name!r} must match [a-z0-9-]+")
        if self.tile_m <= 0 or self.tile_n <= 0:
            raise ValueError("candidate tiles must be positive")


@dataclass(frozen=True)
class MatmulSearchContract:
    mesh_size: int
    m: int
    k: int
    n: int
    warmup_iterations: int
    measured_iterations: int
    rounds: int
    candidates: tuple[MatmulSearchCandidate, ...]
    bootstrap_samples: int = 10_000
    minimum_practical_improvement: float = 0.01
    collective_strategy: str = "p2p_fused_epilogue_bf16_transport"
    scatter_dimension: str = "M"
    output_dtype: str = "bf16"
    execution: str = "one-process-per-gpu"  # or "emulated-on-one-gpu": every mesh position on the current GPU (correctness, not multi-GPU timing)

    def __post_init__(self) -> None:
        if self.execution not in ("one-process-per-gpu", "emulated-on-one-gpu"):
            raise ValueError(f"execution must be one-process-per-gpu or emulated-on-one-gpu, got {self.execution}")
        if min(self.mesh_size, self.m, self.k, self.n, self.measured_iterations) <= 0 or self.warmup_iterations < 0:
            raise ValueError("mesh, shape and measured iterations must be positive; warmup non-negative")
        if self.rounds < 5:
            raise ValueError("a search needs at least 5 rounds")
        if self.bootstrap_samples < 1000:
            raise ValueError("bootstrap_samples must be at least 1000")
        if not 0 < self.minimum_practical_improvement < 1:
            raise ValueError("minimum_practical_improvement must lie in (0, 1)")
        if len(self.candidates) < 2:
            raise ValueError("a search needs at least two candidates")
        names = [c.name for c in self.candidates]
        tiles = [(c.tile_m, c.tile_n) for c in self.candidates]
        if len(set(names)) != len(names) or len(set(tiles)) != len(tiles):
            raise ValueError("search candidates need unique names and tile shapes")
        for candidate in self.candidates:
            if self.m % candidate.tile_m or self.n % candidate.tile_n:
                raise ValueError(f"candidate {candidate.name} does not divide M and N")

    @classmethod
    def from_json(cls, text: str) -> "MatmulSearchContract":
        raw = json.loads(text)
        known = set(cls.__dataclass_fields__)
        unknown = set(raw) - known
        if unknown:
            raise ValueError(f"unknown contract fields {sorted(unknown)}")
        raw["candidates"] = tuple(MatmulSearchCandidate(**c) for c in raw["candidates"])
        return cls(**raw)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2) + "\n"

    @property
    def search_id(self) -> str:
        return semantic_sha256("matmul-search-contract", json.dumps(asdict(self), sort_keys=True, separators=(",", ":")))


@dataclass(frozen=True)
class CandidateStatistics:
    name: str
    tile_m: int
    tile_n: int
    run_count: int
    sample_count: int
    median_ns: float
    p90_ns: int
    median_absolute_deviation_ns: float
    coefficient_of_variation: float
    improvement_over_baseline: float | None
    improvement_confidence_interval: tuple[float, float] | None
    promotable: bool


@dataclass(frozen=True)
class MatmulSearchResult:
    search_id: str
    baseline: str
    winner: str | None
    matched_input_sha256: tuple[str, str]
    execution_orders: tuple[tuple[str, ...], ...]
    candidates: tuple[CandidateStatistics, ...]
    run_results: tuple[str, ...] = field(default_factory=tuple)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2) + "\n"


def percentile(samples: list[int], fraction: float) -> int:
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, round((len(ordered) - 1) * fraction))]


def improvement_interval(paired_round_improvements: list[float], *, samples: int, seed: int) -> tuple[float, float]:
    """95 % bootstrap interval of the median of the per-round paired improvements."""
    generator = np.random.default_rng(seed)
    values = np.asarray(paired_round_improvements, dtype=np.float64)
    estimates = np.empty(samples, dtype=np.float64)
    for index in range(samples):
        estimates[index] = np.median(generator.choice(values, len(values), replace=True))
    low, high = np.quantile(estimates, (0.025, 0.975))
    return float(low), float(high)


def summarise(contract: MatmulSearchContract, runs: list[tuple[int, str, object]], execution_orders, run_paths=()) -> MatmulSearchResult:
    """Statistics and winner from (round, candidate name, run result) triples. A run result needs
    ``passed``, ``lhs_sha256``, ``rhs_sha256``, ``output_sha256``, ``schedule_sha256``,
    ``cuda_source_sha256`` and ``samples_ns``."""
    failed = [name for _, name, result in runs if not result.passed]
    if failed:
        raise ValueError(f"SEARCH_CORRECTNESS_FAILED candidates={failed}")
    inputs = {(result.lhs_sha256, result.rhs_sha256) for _, _, result in runs}
    if len(inputs) != 1:
        raise ValueError("SEARCH_INPUTS_ARE_NOT_MATCHED")
    names = [c.name for c in contract.candidates]
    for name in names:
        mine = [result for _, n, result in runs if n == name]
        if len({r.output_sha256 for r in mine}) != 1:
            raise ValueError("SEARCH_OUTPUTS_ARE_NOT_DETERMINISTIC")
        if len({(r.schedule_sha256, r.cuda_source_sha256) for r in mine}) != 1:
            raise ValueError("SEARCH_CANDIDATE_CODE_IDENTITIES_ARE_NOT_STABLE")
    samples = {name: [] for name in names}
    round_medians = {name: {} for name in names}
    for round_index, name, result in runs:
        samples[name].extend(result.samples_ns)
        round_medians[name][round_index] = float(statistics.median(result.samples_ns))
    baseline = names[0]
    baseline_median = float(statistics.median(samples[baseline]))
    rows: list[CandidateStatistics] = []
    for candidate in contract.candidates:
        values = samples[candidate.name]
        median = float(statistics.median(values))
        improvement = interval = None
        promotable = True
        if candidate.name != baseline:
            paired = [
                (round_medians[baseline][r] - round_medians[candidate.name][r]) / round_medians[baseline][r]
                for r in range(contract.rounds)
            ]
            improvement = float(statistics.median(paired))
            seed = int(hashlib.sha256(candidate.name.encode()).hexdigest()[:16], 16)
            interval = improvement_interval(paired, samples=contract.bootstrap_samples, seed=seed)
            promotable = interval[0] > contract.minimum_practical_improvement
        rows.append(CandidateStatistics(
            name=candidate.name, tile_m=candidate.tile_m, tile_n=candidate.tile_n, run_count=contract.rounds, sample_count=len(values),
            median_ns=median, p90_ns=percentile(values, 0.9),
            median_absolute_deviation_ns=float(statistics.median(abs(v - median) for v in values)),
            coefficient_of_variation=statistics.pstdev(values) / statistics.mean(values),
            improvement_over_baseline=improvement, improvement_confidence_interval=interval, promotable=promotable,
        ))
    promoted = [row for row in rows[1:] if row.promotable and row.median_ns < baseline_median]
    winner = min(promoted, key=lambda row: row.median_ns).name if promoted else None
    return MatmulSearchResult(
        search_id=contract.search_id, baseline=baseline, winner=winner, matched_input_sha256=next(iter(inputs)),
        execution_orders=tuple(execution_orders), candidates=tuple(rows), run_results=tuple(run_paths),
    )


def run_matmul_search(output_dir: Path, contract: MatmulSearchContract, *, run: Callable | None = None, write_result: bool = True) -> MatmulSearchResult:
    """Runs every candidate in every round (order reversed on odd rounds) through the runner and
    writes ``contract.json`` and ``result.json``. ``run(path, contract, candidate)`` defaults to the
    CUDA runner. A directory that holds a different contract is refused (the contract must be
    byte-identical on resume, src/tpu_cake/search.py:507-514); a round directory that already holds a
    finished run is validated and reused, one without a result is refused (:461-496)."""
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    contract_path = output_dir / "contract.json"
    if contract_path.exists():
        if contract_path.read_text() != contract.to_json():
            raise ValueError("SEARCH_CONTRACT_CHANGED")
    else:
        contract_path.write_text(contract.to_json())
    if run is None:
        run = _run_candidate
    runs, orders, paths = [], [], []
    for round_index in range(contract.rounds):
        order = contract.candidates if round_index % 2 == 0 else contract.candidates[::-1]
        orders.append(tuple(c.name for c in order))
        for candidate in order:
            path = output_dir / f"round-{round_index:02d}" / candidate.name
            runs.append((round_index, candidate.name, _load_or_run(path, contract, candidate, run)))
            paths.append(str(path.relative_to(output_dir)))
    result = summarise(contract, runs, orders, paths)
    if write_result:
        (output_dir / "result.json").write_text(result.to_json())
    return result


def _expected_invocation(contract: MatmulSearchContract, candidate: MatmulSearchCandidate) -> dict:
    return {
        "mesh_size": contract.mesh_size, "m": contract.m, "k": contract.k, "n": contract.n,
        "warmup_iterations": contract.warmup_iterations, "measured_iterations": contract.measured_iterations,
        "tile": [candidate.tile_m, candidate.tile_n], "collective_strategy": contract.collective_strategy,
        "scatter_dimension": contract.scatter_dimension, "output_dtype": contract.output_dtype, "mode": "timing",
        "execution": contract.execution if contract.mesh_size > 1 else "one-process-per-gpu",
    }


def validate_saved_run_evidence(path: Path, contract: MatmulSearchContract, candidate: MatmulSearchCandidate):
    """A finished run directory as search evidence: its invocation must be the one this contract
    and candidate would make, the run must have passed with the declared number of samples, and
    every artifact it lists must still have the recorded size and hash
    (src/tpu_cake/search.py:166-372). Returns the saved result."""
    import hashlib

    from . import runner

    result_path, invocation_path = path / "result.json", path / "invocation.json"
    if not result_path.is_file() or not invocation_path.is_file():
        raise ValueError(f"SEARCH_RUN_INCOMPLETE path={path}")
    invocation = json.loads(invocation_path.read_text())
    expected = _expected_invocation(contract, candidate)
    if invocation != expected:
        changed = sorted(key for key in set(invocation) | set(expected) if invocation.get(key) != expected.get(key))
        raise ValueError(f"SEARCH_RUN_INVOCATION_MISMATCH path={path} fields={changed}")
    raw = json.loads(result_path.read_text())
    if not raw.get("passed") or raw.get("mode") != "timing" or len(raw.get("samples_ns", ())) != contract.measured_iterations:
        raise ValueError(f"SEARCH_RUN_EVIDENCE_REJECTED path={path}")
    for artifact in raw["artifacts"]:
        target = path / artifact["path"]
        if not target.is_file() or target.stat().st_size != artifact["size_bytes"] or hashlib.sha256(target.read_bytes()).hexdigest() != artifact["sha256"]:
            raise ValueError(f"SEARCH_RUN_ARTIFACT_CHANGED path={target}")
    raw["artifacts"] = tuple(runner.ArtifactReference(**artifact) for artifact in raw["artifacts"])
    raw["samples_ns"] = tuple(raw["samples_ns"])
    return runner.MatmulRunResult(**raw)


def _load_or_run(path: Path, contract: MatmulSearchContract, candidate: MatmulSearchCandidate, run: Callable):
    """Resume rule: a directory that exists holds either a finished, valid run (reused) or the
    remains of one that died (refused: delete it deliberately, never silently)."""
    if path.exists() and run is _run_candidate:
        return validate_saved_run_evidence(path, contract, candidate)
    return run(path, contract, candidate)


def _run_candidate(path: Path, contract: MatmulSearchContract, candidate: MatmulSearchCandidate):
    from . import runner, schedule_lowering

    path.parent.mkdir(parents=True, exist_ok=True)
    return runner.run_distributed_matmul(
        path, mesh_size=contract.mesh_size, m=contract.m, k=contract.k, n=contract.n, warmup_iterations=contract.warmup_iterations,
        measured_iterations=contract.measured_iterations, tile=schedule_lowering.MatmulTile(candidate.tile_m, candidate.tile_n),
        collective_strategy=contract.collective_strategy, scatter_dimension=contract.scatter_dimension, output_dtype=contract.output_dtype,
        emulate_on_one_gpu=contract.execution == "emulated-on-one-gpu",
    )
