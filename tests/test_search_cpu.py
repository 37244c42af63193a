"""The tile-search driver: contract rules, protocol and statistics, with runs injected so that no
GPU is needed (the search itself only orders runs and does arithmetic on their samples)."""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import pytest

from tpu_cake_b200 import search

ROOT = Path(__file__).resolve().parent.parent


@dataclass
class FakeRun:
    samples_ns: tuple[int, ...]
    passed: bool = True
    lhs_sha256: str = "a" * 64
    rhs_sha256: str = "b" * 64
    output_sha256: str = "c" * 64
    schedule_sha256: str = "d" * 64
    cuda_source_sha256: str = "e" * 64


def contract(**overrides):
    fields = dict(
        mesh_size=8, m=1024, k=4096, n=1024, warmup_iterations=2, measured_iterations=8, rounds=5, bootstrap_samples=1000,
        candidates=(search.MatmulSearchCandidate("base", 128, 256), search.MatmulSearchCandidate("fast", 128, 128),
                    search.MatmulSearchCandidate("same", 128, 64)),
    )
    fields.update(overrides)
    return search.MatmulSearchContract(**fields)


def fake_runner(speed):
    generator = np.random.default_rng(0)

    def run(path, contract_, candidate):
        base = speed[candidate.name]
        samples = tuple(int(base * (1 + 0.002 * generator.standard_normal())) for _ in range(contract_.measured_iterations))
        return FakeRun(samples, output_sha256=candidate.name.ljust(64, "0"), schedule_sha256=candidate.name.ljust(64, "1"))

    return run


def test_contract_rules():
    with pytest.raises(ValueError, match="at least 5 rounds"):
        contract(rounds=4)
    with pytest.raises(ValueError, match="does not divide"):
        contract(candidates=(search.MatmulSearchCandidate("a", 128, 256), search.MatmulSearchCandidate("b", 96, 128)))
    with pytest.raises(ValueError, match="unique names and tile shapes"):
        contract(candidates=(search.MatmulSearchCandidate("a", 128, 256), search.MatmulSearchCandidate("b", 128, 256)))
    with pytest.raises(ValueError, match="must match"):
        search.MatmulSearchCandidate("Tile_1", 128, 128)
    assert contract().search_id == contract().search_id != contract(k=8192).search_id


def test_shipped_contract_parses_and_round_trips():
    text = (ROOT / "tpu-cake_b200" / "contracts" / "matmul-tile-search-b200.json").read_text()
    parsed = search.MatmulSearchContract.from_json(text)
    assert parsed.mesh_size == 8 and [c.tile_n for c in parsed.candidates] == [256, 128, 64]
    assert search.MatmulSearchContract.from_json(parsed.to_json()) == parsed
    with pytest.raises(ValueError, match="unknown contract fields"):
        search.MatmulSearchContract.from_json(json.dumps({**json.loads(text), "backend": "tpu"}))


def test_search_alternates_order_and_promotes_only_clear_wins(tmp_path):
    c = contract()
    result = search.run_matmul_search(tmp_path / "s", c, run=fake_runner({"base": 1_000_000, "fast": 900_000, "same": 999_000}))
    assert result.execution_orders[0] == ("base", "fast", "same") and result.execution_orders[1] == ("same", "fast", "base")
    rows = {row.name: row for row in result.candidates}
    assert result.baseline == "base" and result.winner == "fast"
    assert rows["fast"].promotable and 0.09 < rows["fast"].improvement_over_baseline < 0.11
    low, high = rows["fast"].improvement_confidence_interval
    assert 0.01 < low <= rows["fast"].improvement_over_baseline <= high
    assert not rows["same"].promotable  # a 0.1 % gain does not clear the 1 % bar
    assert rows["base"].improvement_over_baseline is None and rows["base"].sample_count == 5 * 8
    saved = json.loads((tmp_path / "s" / "result.json").read_text())
    assert saved["winner"] == "fast" and len(saved["run_results"]) == 15
    # Same directory, another contract: refused.
    with pytest.raises(ValueError, match="SEARCH_CONTRACT_CHANGED"):
        search.run_matmul_search(tmp_path / "s", contract(k=8192), run=fake_runner({"base": 1, "fast": 1, "same": 1}))


def test_search_rejects_failed_unmatched_or_unstable_runs(tmp_path):
    c = contract()

    def failing(path, contract_, candidate):
        return FakeRun((100,) * 8, passed=candidate.name != "fast")

    with pytest.raises(ValueError, match=r"SEARCH_CORRECTNESS_FAILED candidates=\['fast'"):
        search.run_matmul_search(tmp_path / "a", c, run=failing)
    counter = iter(range(1000))

    def drifting_inputs(path, contract_, candidate):
        return FakeRun((100,) * 8, lhs_sha256=f"{next(counter):064d}")

    with pytest.raises(ValueError, match="SEARCH_INPUTS_ARE_NOT_MATCHED"):
        search.run_matmul_search(tmp_path / "b", c, run=drifting_inputs)

    def unstable_output(path, contract_, candidate):
        return FakeRun((100,) * 8, output_sha256=f"{next(counter):064d}")

    with pytest.raises(ValueError, match="SEARCH_OUTPUTS_ARE_NOT_DETERMINISTIC"):
        search.run_matmul_search(tmp_path / "c", c, run=unstable_output)


def test_bootstrap_interval_is_seeded_and_brackets_the_median():
    paired = [0.05, 0.06, 0.04, 0.055, 0.052]
    first = search.improvement_interval(paired, samples=2000, seed=7)
    assert first == search.improvement_interval(paired, samples=2000, seed=7)
    assert 0.04 <= first[0] <= 0.052 <= first[1] <= 0.06


# ------------------------------------------------------------------------------------ RPA chunk search


def rpa_contract(**overrides):
    from tpu_cake_b200 import rpa_search

    fields = dict(workload="rpa-decode-64seq", baseline="chunk-512", bootstrap_samples=1000, measured_iterations=8,
                  candidates=(rpa_search.RpaSearchCandidate("chunk-512", 512), rpa_search.RpaSearchCandidate("chunk-256", 256)))
    fields.update(overrides)
    return rpa_search.RpaSearchContract(**fields)


def test_rpa_search_contract_rules_and_shipped_contract():
    from tpu_cake_b200 import rpa_search

    with pytest.raises(ValueError, match="multiple of the 32-token stage"):
        rpa_search.RpaSearchCandidate("c", 48)
    with pytest.raises(ValueError, match="baseline must be the first candidate"):
        rpa_contract(baseline="chunk-256")
    with pytest.raises(ValueError, match="at least 5 rounds"):
        rpa_contract(rounds=3)
    text = (ROOT / "tpu-cake_b200" / "contracts" / "rpa-chunk-search-b200.json").read_text()
    parsed = rpa_search.RpaSearchContract.from_json(text)
    assert parsed.baseline == "chunk-512" and [c.kv_chunk_tokens for c in parsed.candidates] == [512, 256, 1024]
    assert rpa_search.RpaSearchContract.from_json(parsed.to_json()) == parsed


def test_rpa_search_protocol_with_injected_runs(tmp_path):
    from tpu_cake_b200 import rpa_search

    generator = np.random.default_rng(1)
    speed = {"chunk-512": 210_000, "chunk-256": 200_000}

    def run(contract_, candidate):
        samples = tuple(int(speed[candidate.name] * (1 + 0.003 * generator.standard_normal())) for _ in range(contract_.measured_iterations))
        return rpa_search.RpaRunEvidence(candidate.name, True, samples, "a" * 64, "b" * 64, candidate.name.ljust(64, "0"), "d" * 64,
                                         candidate.name.ljust(64, "e"))

    result = rpa_search.run_rpa_search(tmp_path / "r", rpa_contract(), run=run)
    assert result.baseline == "chunk-512" and result.winner == "chunk-256"
    assert result.execution_orders[1] == ("chunk-256", "chunk-512")
    rows = {row.name: row for row in result.candidates}
    assert rows["chunk-256"].tile_n == 256 and 0.03 < rows["chunk-256"].improvement_over_baseline < 0.06


def test_the_reference_tile_search_contract_is_read_as_it_is():
    """The reference's own contract document (contracts/matmul-tile-search-tpu7x.json: mesh 8,
    1024 x 65536 x 1024, 20 + 200 calls, five rounds, square tiles of 128 / 256 / 512) has no field
    this backend does not know and needs none it lacks; what it does not say gets this backend's
    defaults. Tiles above the hardware tile are walked in hardware sub-tiles."""
    import json

    document = {
        "mesh_size": 8, "m": 1024, "k": 65536, "n": 1024, "warmup_iterations": 20, "measured_iterations": 200, "rounds": 5,
        "bootstrap_samples": 10000, "minimum_practical_improvement": 0.01,
        "candidates": [{"name": f"tile-{size}", "tile_m": size, "tile_n": size} for size in (128, 256, 512)],
    }
    contract = search.MatmulSearchContract.from_json(json.dumps(document))
    assert (contract.mesh_size, contract.m, contract.k, contract.n, contract.rounds) == (8, 1024, 65536, 1024, 5)
    assert [(c.name, c.tile_m, c.tile_n) for c in contract.candidates] == [("tile-128", 128, 128), ("tile-256", 256, 256), ("tile-512", 512, 512)]
    assert contract.collective_strategy == "p2p_fused_epilogue_bf16_transport" and contract.execution == "one-process-per-gpu"
