"""Search over the decode kernel's split-KV chunk size on the CUDA backend.

Mirrors the reference's RPA block search (src/tpu_cake/rpa_search.py: contract :71-108 with a named
baseline, at least 5 rounds, unique candidates; device timing per run :127-134, there read from
profiler events, here taken with CUDA events on the launching stream; the paired-bootstrap promotion
rule shared with the matmul search). The reference's candidates are TPU block and cluster sizes
(:23-50); the sm_100a decode kernel's tunable is the number of KV tokens per work item
(``kv_chunk_tokens``: smaller chunks balance the persistent CTAs better, larger ones write fewer
partials).
"""

from __future__ import annotations

import json
import re
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable

from . import search
from .identity import semantic_sha256


@dataclass(frozen=True)
class RpaSearchCandidate:
    name: str
    kv_chunk_tokens: int

    def __post_init__(self) -> None:
        if not re.fullmatch(r"[a-z0-9-]+", self.name):
            raise ValueError(f"candidate name {self.name!r} must match [a-z0-9-]+")
        if self.kv_chunk_tokens <= 0 or self.kv_chunk_tokens % 32:
            raise ValueError("kv_chunk_tokens must be a positive multiple of the 32-token stage")


@dataclass(frozen=True)
class RpaSearchContract:
    workload: str                 # a decode configuration of tpu_cake_b200.workloads, by name
    baseline: str
    candidates: tuple[RpaSearchCandidate, ...]
    seed: int = 97
    warmup_iterations: int = 5
    measured_iterations: int = 50
    rounds: int = 5
    bootstrap_samples: int = 10_000
    minimum_practical_improvement: float = 0.01
    pool_pages: int = 0           # 0 = the configuration's own pool

    def __post_init__(self) -> None:
        if self.rounds < 5:
            raise ValueError("a search needs at least 5 rounds")
        if self.bootstrap_samples < 1000 or not 0 < self.minimum_practical_improvement < 1:
            raise ValueError("bootstrap_samples >= 1000 and 0 < minimum_practical_improvement < 1")
        if self.measured_iterations <= 0 or self.warmup_iterations < 0:
            raise ValueError("measured_iterations must be positive and warmup_iterations non-negative")
        if len(self.candidates) < 2:
            raise ValueError("a search needs at least two candidates")
        names = [c.name for c in self.candidates]
        chunks = [c.kv_chunk_tokens for c in self.candidates]
        if len(set(names)) != len(names) or len(set(chunks)) != len(chunks):
            raise ValueError("search candidates need unique names and chunk sizes")
        if self.baseline != names[0]:
            raise ValueError("the baseline must be the first candidate")

    @classmethod
    def from_json(cls, text: str) -> "RpaSearchContract":
        raw = json.loads(text)
        unknown = set(raw) - set(cls.__dataclass_fields__)
        if unknown:
            raise ValueError(f"unknown contract fields {sorted(unknown)}")
        raw["candidates"] = tuple(RpaSearchCandidate(**c) for c in raw["candidates"])
        return cls(**raw)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2) + "\n"

    @property
    def search_id(self) -> str:
        return semantic_sha256("rpa-search-contract", json.dumps(asdict(self), sort_keys=True, separators=(",", ":")))


@dataclass
class RpaRunEvidence:
    """What one candidate run reports: device timing samples and the identities the search matches."""

    candidate: str
    passed: bool
    samples_ns: tuple[int, ...]
    lhs_sha256: str          # metadata (lengths + page table) hash
    rhs_sha256: str          # query hash
    output_sha256: str
    schedule_sha256: str
    cuda_source_sha256: str


def run_rpa_search(output_dir: Path, contract: RpaSearchContract, *, run: Callable | None = None, write_result: bool = True) -> search.MatmulSearchResult:
    """Every candidate in every round, order reversed on odd rounds; statistics and promotion rule of
    the matmul search. Writes ``contract.json`` and ``result.json``."""
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    contract_path = output_dir / "contract.json"
    if contract_path.exists():
        if contract_path.read_text() != contract.to_json():
            raise ValueError("SEARCH_CONTRACT_CHANGED")
    else:
        contract_path.write_text(contract.to_json())
    session = None
    if run is None:
        session = _DecodeSession(contract)
        run = session.run
    try:
        runs, orders = [], []
        for round_index in range(contract.rounds):
            order = contract.candidates if round_index % 2 == 0 else contract.candidates[::-1]
            orders.append(tuple(c.name for c in order))
            for candidate in order:
                evidence = run(contract, candidate)
                runs.append((round_index, candidate.name, evidence))
    finally:
        if session is not None:
            session.close()
    shim = _StatisticsContract(contract)
    result = search.summarise(shim, runs, orders)
    if write_result:
        (output_dir / "result.json").write_text(result.to_json())
    return result


class _StatisticsContract:
    """The fields ``search.summarise`` reads, taken from an RPA contract."""

    def __init__(self, contract: RpaSearchContract):
        self.candidates = tuple(search.MatmulSearchCandidate(c.name, 1, c.kv_chunk_tokens) for c in contract.candidates)
        self.rounds = contract.rounds
        self.bootstrap_samples = contract.bootstrap_samples
        self.minimum_practical_improvement = contract.minimum_practical_improvement
        self.search_id = contract.search_id


class _DecodeSession:
    """Holds the decode workload on the GPU across the rounds so that every run sees the same KV
    pool, queries and page table; one plan per candidate chunk size."""

    def __init__(self, contract: RpaSearchContract):
        import dataclasses

        import numpy as np
        import torch

        from . import rpa_cuda_lowering, workloads
        from .identity import array_sha256

        configs = {c.name: c for c in (workloads.DECODE_64, workloads.DECODE_SHARDED_256)}
        if contract.workload not in configs:
            raise ValueError(f"unknown decode workload {contract.workload!r}; known: {sorted(configs)}")
        config = configs[contract.workload]
        if contract.pool_pages:
            config = dataclasses.replace(config, total_pages=contract.pool_pages)
        self.config = config
        self.torch = torch
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lengths, self.table = workloads.decode_metadata(config)
        generator = torch.Generator(device=self.device).manual_seed(contract.seed)
        shape = (config.total_pages, config.page_size, config.kv_heads, 2, config.head_dim)
        self.cache = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        for start in range(0, config.total_pages, 4096):
            block = self.cache[start : start + 4096]
            block.copy_(torch.randn(block.shape, generator=generator, device=self.device))
        self.query = torch.randn((config.num_seqs, config.q_heads, config.head_dim), generator=generator, device=self.device).to(torch.bfloat16)
        self.table_d = torch.from_numpy(self.table).to(self.device)
        self.lengths_d = torch.from_numpy(self.lengths).to(self.device)
        self.out = torch.empty_like(self.query)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
        self.metadata_sha256 = array_sha256(np.concatenate([self.lengths.astype(np.int64).ravel(), self.table.astype(np.int64).ravel()]))
        self.query_sha256 = array_sha256(self.query.float().cpu().numpy())
        self.plans: dict[int, tuple] = {}
        self.lowering = rpa_cuda_lowering
        self.array_sha256 = array_sha256
        self.reference = None

    def _plan(self, chunk: int):
        if chunk not in self.plans:
            config = self.config
            plan = self.lowering.CudaPagedAttentionPlan(
                name=config.name, schedule_sha256="0" * 64, query_shape=(config.num_seqs, config.q_heads, config.head_dim),
                cache_shape=(config.total_pages, config.page_size, config.kv_heads, config.head_dim), page_table_shape=self.table.shape,
                bias_shape=None, softmax_scale=config.softmax_scale, cache_layout="fused", kv_chunk_tokens=chunk,
            )
            self.plans[chunk] = (plan, plan.build(self.device))
        return self.plans[chunk]

    def run(self, contract: RpaSearchContract, candidate: RpaSearchCandidate) -> RpaRunEvidence:
        torch = self.torch
        plan, executable = self._plan(candidate.kv_chunk_tokens)

        def call():
            plan.invoke(executable, self.query, self.cache, None, self.table_d, self.lengths_d, out=self.out)

        for _ in range(contract.warmup_iterations):
            call()
        torch.cuda.synchronize(self.device)
        samples = []
        for _ in range(contract.measured_iterations):
            self.flush.fill_(1)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            call()
            stop.record()
            stop.synchronize()
            samples.append(int(start.elapsed_time(stop) * 1e6))
        executable.status()
        output = self.out.float().cpu().numpy()
        # Candidates split the KV range differently, so their outputs differ in the last bits; every
        # candidate must agree with the first one run within the attention tolerance.
        if self.reference is None:
            self.reference = output
        difference = abs(output - self.reference).max()
        passed = bool(difference <= 2e-2) and bool((output == output).all())
        return RpaRunEvidence(
            candidate=candidate.name, passed=passed, samples_ns=tuple(samples), lhs_sha256=self.metadata_sha256, rhs_sha256=self.query_sha256,
            output_sha256=self.array_sha256(output), schedule_sha256=plan.schedule_sha256, cuda_source_sha256=plan.source_sha256(),
        )

    def close(self) -> None:
        for _, executable in self.plans.values():
            executable.close()
        self.plans.clear()
