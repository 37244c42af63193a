"""Run bundles on the GPU: the fused-RPA runner (protocol, correctness gate, bundle re-check), the
matmul runner's trace / counters modes, and the three-phase bundle receipt."""

from __future__ import annotations

import json

import numpy as np
import pytest

from tpu_cake_b200 import receipt, rpa_runner, runner
from tpu_cake_b200.run_ledger import RunLedger, RunState

pytestmark = pytest.mark.gpu

HEADER = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'


def _row(index, kernel, metric="gpu__time_duration.sum", unit="ns", value="9000"):
    return f'"{index}","1","python","h","{kernel}","1","7","(384, 1, 1)","(148, 1, 1)","0","10.0","s","{metric}","{unit}","{value}"\n'


def test_fused_rpa_run_writes_a_bundle_that_verifies(cuda_device, tmp_path):
    """The predeclared protocol (seed 97, 5 + 50 calls) on the toy experiment: ledger CREATED ...
    TIMED, 50 samples, output within allclose(0.02, 0.02) of the expectation and the cache
    bit-exact; the bundle re-checks from its files, and a changed saved cache byte is refused."""
    out = tmp_path / "rpa"
    with pytest.raises(ValueError, match="predeclared benchmark protocol"):
        rpa_runner.run_fused_rpa(out, seed=97, warmup_iterations=1, measured_iterations=3)
    assert not out.exists()
    result = rpa_runner.run_fused_rpa(out)
    assert result.passed and result.preflight_passed and len(result.samples_ns) == 50 and result.median_ns > 0
    assert result.maximum_absolute_errors[0] <= 0.02 and result.maximum_absolute_errors[1] == 0.0
    for name in ("invocation.json", "profiler_config.json", "source_state.json", "source_diff.patch", "experiment.json", "physical.xdsl",
                 "lowered_cuda.py", "preflight.json", "kernel_manifest.json", "inputs/03-fused_cache.npy", "outputs/00-output.npy",
                 "outputs/01-updated_cache.npy", "oracle/01-updated_cache.npy", "ledger.sqlite", "result.json"):
        assert (out / name).exists(), name
    with RunLedger(out / "ledger.sqlite") as ledger:
        states = [event.state for event in ledger.history(result.run_id)]
    assert states == [RunState.CREATED, RunState.VERIFIED, RunState.LOWERED, RunState.COMPILED, RunState.CORRECT, RunState.TIMED]
    assert rpa_runner.validate_fused_rpa_bundle(out)["run_id"] == result.run_id
    cache_path = out / "outputs" / "01-updated_cache.npy"
    original = cache_path.read_bytes()
    tampered = bytearray(original)
    tampered[-1] ^= 1
    cache_path.write_bytes(bytes(tampered))
    with pytest.raises(ValueError, match="ARTIFACT_CHANGED path=outputs/01-updated_cache.npy"):
        rpa_runner.validate_fused_rpa_bundle(out)
    cache_path.write_bytes(original)
    rpa_runner.validate_fused_rpa_bundle(out)
    with pytest.raises(FileExistsError):
        rpa_runner.run_fused_rpa(out)


def test_fused_rpa_run_rejects_a_forged_cache_byte(cuda_device, tmp_path):
    """One flipped bit in the device's updated cache: the output still passes its tolerance, the
    exact cache comparison does not, and the run ends REJECTED."""
    out = tmp_path / "forged"
    with pytest.raises(ValueError, match="FUSED_RPA_CORRECTNESS_FAILED"):
        rpa_runner.run_fused_rpa(out, corrupt_device_cache_for_testing=True)
    with RunLedger(out / "ledger.sqlite") as ledger:
        events = ledger.history(_run_id_of(out))
    assert events[-1].state is RunState.REJECTED
    assert not (out / "result.json").exists()


def _run_id_of(out):
    import sqlite3

    with sqlite3.connect(out / "ledger.sqlite") as connection:
        return connection.execute("select run_id from events limit 1").fetchone()[0]


def test_rpa_trace_mode_ends_traced_without_host_timings(cuda_device, tmp_path):
    result = rpa_runner.run_fused_rpa(tmp_path / "trace", mode="trace")
    assert result.mode == "trace" and result.samples_ns == () and result.median_ns is None and result.passed
    config = json.loads((tmp_path / "trace" / "profiler_config.json").read_text())
    assert config["profiler"] == "ncu" and config["counters"] is False and "--clock-control" in config["arguments"]
    with RunLedger(tmp_path / "trace" / "ledger.sqlite") as ledger:
        assert ledger.history(result.run_id)[-1].state is RunState.TRACED


def test_three_phase_matmul_bundle(cuda_device, tmp_path):
    """timing / trace / counters runs of one invocation agree on every identity; with launch lists
    for the two profiled phases the bundle receipt is written. A trace capture that carries
    hardware counters, a counters capture without them, and a phase run with another shape are
    refused."""
    root = tmp_path / "bundle"
    common = dict(mesh_size=2, m=128, k=1024, n=1024, warmup_iterations=1, measured_iterations=3, collective_strategy="p2p_fused_epilogue",
                  emulate_on_one_gpu=True)
    results = {mode: runner.run_distributed_matmul(root / mode, mode=mode, **common) for mode in ("timing", "trace", "counters")}
    assert results["timing"].median_ns > 0 and results["trace"].samples_ns == () and results["counters"].median_ns is None
    assert len({r.output_sha256 for r in results.values()}) == 1 and len({r.run_id for r in results.values()}) == 3
    with RunLedger(root / "counters" / "ledger.sqlite") as ledger:
        assert ledger.history(results["counters"].run_id)[-1].state is RunState.COUNTERED
    gemm, reduce = "void cake::cake_matmul_rs_sm100<256, 0>(...)", "void cake::cake_reduce_slots_sm100(...)"
    trace = tmp_path / "trace.csv"
    trace.write_text(HEADER + _row(0, gemm) + _row(1, reduce))
    counters = tmp_path / "counters.csv"
    counters.write_text(HEADER + _row(0, gemm) + _row(0, gemm, "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "%", "61.5")
                        + _row(0, gemm, "dram__bytes_read.sum", "Mbyte", "2.1") + _row(0, gemm, "dram__bytes_write.sum", "Mbyte", "0.6") + _row(1, reduce))
    with pytest.raises(ValueError, match="PROFILE_CAPTURE_REJECTED phase=counters"):
        receipt.finalize_matmul_bundle(root, trace_profile=trace, counters_profile=trace)
    with pytest.raises(ValueError, match="PROFILER_CONTRACT_VIOLATION phase=trace"):
        receipt.finalize_matmul_bundle(root, trace_profile=counters, counters_profile=counters)
    document = receipt.finalize_matmul_bundle(root, trace_profile=trace, counters_profile=counters)
    assert set(document["run_ids"]) == {"timing", "trace", "counters"} and (root / "bundle.json").exists()
    assert document["profiles"]["counters"]["marker_launches"]["cake_matmul_rs_sm100"] == 1
    other = tmp_path / "other"
    for mode in ("timing", "trace"):
        runner.run_distributed_matmul(other / mode, mode=mode, **common)
    runner.run_distributed_matmul(other / "counters", mode="counters", **{**common, "n": 512})
    with pytest.raises(ValueError, match="BUNDLE_IDENTITY_MISMATCH phase=counters"):
        receipt.finalize_matmul_bundle(other, trace_profile=trace, counters_profile=counters)


def test_sharded_surface_protocol_emulated_on_one_gpu(cuda_device, tmp_path):
    """The 2 x 4 surface protocol with the eight positions run one after the other on this GPU: five
    seeds, two executions each, exact repeats, exact cache, output within 1e-3 / 6e-3 of the host
    definition; two chained timing rounds instead of sixteen. A single process must ask for the
    emulation explicitly."""
    from tpu_cake_b200 import rpa_surface_runner

    with pytest.raises(ValueError, match="MESH_NOT_AVAILABLE"):
        rpa_surface_runner.run_inkling_sharded_rpa_surface(tmp_path / "refused")
    result = rpa_surface_runner.run_inkling_sharded_rpa_surface(tmp_path / "surface", emulate_on_one_gpu=True, protocol={"timing_rounds": 2})
    assert result["passed"] and result["execution"] == "emulated" and len(result["correctness"]) == 5
    for observation in result["correctness"]:
        assert observation["repeated_output_exact"] and observation["repeated_cache_exact"] and observation["cache_exact"]
        assert observation["maximum_absolute_error"] <= 1e-3 and observation["relative_l2_error"] <= 6e-3
    assert len(result["round_medians_ns"]) == 2 and (tmp_path / "surface" / "correctness.json").is_file()
