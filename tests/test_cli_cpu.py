from __future__ import annotations

import json

from tpu_cake_b200 import cli


def test_verify_schedule_and_render(capsys):
    assert cli.main(["verify-schedule", "--mesh-size", "8", "--m", "128", "--k", "1024", "--n", "1024"]) == 0
    hashes = json.loads(capsys.readouterr().out)
    assert len(hashes["distributed_sha256"]) == 64 and len(hashes["physical_sha256"]) == 64
    assert cli.main(["render-workload", "--physical"]) == 0
    assert '"tpu_schedule.collective"' in capsys.readouterr().out


def test_estimate_large_configuration(capsys):
    assert cli.main(["estimate", "--mesh-size", "8", "--m", "8192", "--k", "16384", "--n", "8192", "--scatter-dimension", "M"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["operations_per_device"] == 2 * 8192 * 2048 * 8192 and report["limiting_resource"] == "compute"


def test_experiment_records(capsys, tmp_path):
    """``experiment inkling-rpa`` renders the prototype decode op's record (toy shapes, protocol 5 / 50,
    what a profile must show); ``--output`` writes the same text."""
    assert cli.main(["experiment", "inkling-rpa"]) == 0
    record = json.loads(capsys.readouterr().out)
    assert record["benchmark"] == {"warmup_iterations": 5, "measured_iterations": 50, "synchronization": "synchronize the device after every call",
                                   "statistic": "median wall duration"}
    assert [t["shape"] for t in record["workload"]["inputs"]] == [[4, 4, 32], [32, 16, 4, 32], [32, 16, 4, 32], [4, 8], [4], [4, 128]]
    assert record["profile"]["required_timed_hlo_markers"] == ["cake_rpa_decode_sm100"] and len(record["schedule_sha256"]) == 64
    target = tmp_path / "nested" / "experiment.json"
    assert cli.main(["experiment", "inkling-fused-rpa", "--output", str(target)]) == 0
    assert "EXPERIMENT_WRITTEN workload=inkling-fused-rpa" in capsys.readouterr().out
    assert json.loads(target.read_text())["workload"]["seed"] == 97
    assert cli.main(["experiment", "matmul"]) == 0
    assert json.loads(capsys.readouterr().out)["workload"]["mesh_size"] == 8


HEADER = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'


def _launch(index, kernel):
    return f'"{index}","1","python","h","{kernel}","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","s","gpu__time_duration.sum","ns","9000"\n'


def test_inspect_profile_exit_codes(capsys, tmp_path):
    """Exit code 0 for an accepted capture, 1 for a rejected one (src/tpu_cake/cli.py:572-601), with
    the contract read from JSON or TOML."""
    good = tmp_path / "good.csv"
    good.write_text(HEADER + _launch(0, "void cake::cake_rpa_decode_sm100(...)"))
    wrong = tmp_path / "wrong.csv"
    wrong.write_text(HEADER + _launch(0, "void flash_fwd_splitkv_kernel<...>(...)"))
    contract = tmp_path / "expectation.json"
    contract.write_text(json.dumps({"name": "rpa-decode", "require_tensor_core_activity": False,
                                    "required_timed_hlo_markers": ["cake_rpa_decode_sm100"], "forbidden_timed_hlo_fragments": ["flash_fwd"]}))
    toml = tmp_path / "expectation.toml"
    toml.write_text('name = "rpa-decode"\nrequire_tensor_core_activity = false\nrequired_timed_hlo_markers = ["cake_rpa_decode_sm100"]\n'
                    'forbidden_timed_hlo_fragments = ["flash_fwd"]\n')
    report = tmp_path / "report.json"
    assert cli.main(["inspect-profile", str(good), "--contract", str(contract), "--output", str(report)]) == 0
    assert "PROFILE_ACCEPTED contract=rpa-decode" in capsys.readouterr().out and json.loads(report.read_text())["accepted"]
    assert cli.main(["inspect-profile", str(wrong), "--contract", str(toml)]) == 1
    out = capsys.readouterr().out
    assert "PROFILE_REJECTED" in out and "REQUIRED_TIMED_MARKER_MISSING" in out and "FORBIDDEN_TIMED_FRAGMENT_PRESENT" in out
    assert cli.main(["inspect-profile", str(tmp_path / "absent.csv"), "--contract", str(contract)]) == 1


def test_profiler_contract_rules():
    """A timing run carries no profiler, a trace run no hardware counters, and every profiled run
    leaves the GPU clocks alone."""
    import pytest

    from tpu_cake_b200 import run_artifacts

    for mode in ("timing", "trace", "counters"):
        run_artifacts.validate_profiler_contract(run_artifacts.profiler_contract(mode))
    assert run_artifacts.profiler_contract("timing")["profiler"] is None
    trace = run_artifacts.profiler_contract("trace")
    assert "gpu__time_duration.sum" in " ".join(trace["arguments"]) and "dram__" not in " ".join(trace["arguments"])
    with pytest.raises(ValueError, match="PROFILER_CONTRACT_VIOLATION mode=trace"):
        run_artifacts.validate_profiler_contract({**trace, "arguments": [*trace["arguments"], "--metrics", "dram__bytes_read.sum"]})
    with pytest.raises(ValueError, match="PROFILER_CONTRACT_VIOLATION mode=timing"):
        run_artifacts.validate_profiler_contract({"mode": "timing", "profiler": "ncu", "arguments": []})
    counters = run_artifacts.profiler_contract("counters")
    with pytest.raises(ValueError, match="would lock the GPU clocks"):
        run_artifacts.validate_profiler_contract({**counters, "arguments": [a for a in counters["arguments"] if a not in ("--clock-control", "none")]})


def test_fused_rpa_protocol_inputs_and_expectation(golden_dir):
    """The runner's own pieces against the reference's vectors: the seeded toy inputs are the
    reference's bit for bit, and the expected result the correctness gate uses equals the
    reference oracle's output and updated cache bit for bit (seeds 0 and 7)."""
    import numpy as np
    import pytest

    from tpu_cake_b200 import rpa_runner, workloads

    vectors = np.load(golden_dir / "rpa_reference_vectors.npz")
    names = ("queries", "keys", "values", "cache", "kv_lengths", "page_indices", "cu_q_lens", "cu_kv_lens", "distribution",
             "relative_states", "relative_projection")
    for seed in (0, 7):
        inputs = workloads.inkling_fused_rpa_inputs(seed)
        for name, value in zip(names, inputs, strict=True):
            bits = value.view(np.uint16) if value.dtype.itemsize == 2 else value
            np.testing.assert_array_equal(bits, vectors[f"fused/seed{seed}/{name}"])
        output, cache = rpa_runner.expected_fused_rpa(inputs, softmax_scale=1.0 / 32)
        np.testing.assert_array_equal(output.view(np.uint16), vectors[f"fused/seed{seed}/output_bf16_bits"])
        np.testing.assert_array_equal(cache.view(np.uint16), vectors[f"fused/seed{seed}/updated_cache_bf16_bits"])
    rpa_runner.validate_fused_rpa_run_protocol(seed=97, warmup_iterations=5, measured_iterations=50)
    with pytest.raises(ValueError, match="predeclared benchmark protocol"):
        rpa_runner.validate_fused_rpa_run_protocol(seed=1, warmup_iterations=5, measured_iterations=50)


def test_reference_named_lowerings():
    """The names the reference's callers use resolve to the CUDA plans, with the reference's shapes."""
    from tpu_cake_b200 import rpa_cuda_lowering, workloads

    plan = rpa_cuda_lowering.lower_inkling_rpa_to_cuda(workloads.inkling_fused_rpa_schedule())
    assert plan.query_shape == (4, 4, 32) and plan.fused_cache_shape == (32, 16, 2, 2, 128) and plan.softmax_scale == 1.0 / 32
    sharded = rpa_cuda_lowering.lower_inkling_sharded_rpa_to_cuda(workloads.inkling_sharded_rpa_schedule())
    assert sharded.mesh_axes == ("data", "tensor") and sharded.mesh_shape == (2, 4)
    assert sharded.global_input_shapes[0] == (8, 32, 128) and sharded.global_input_shapes[3] == (7424, 1, 16, 2, 128)
    assert hasattr(sharded, "place_inputs") and hasattr(sharded, "build_executable")


def test_validate_saved_cuda_plan_replays_and_rejects(tmp_path):
    """The saved physical IR and lowered source of a run replay to the same plan; a changed byte in
    either, a stale hash, or a source that belongs to another workload is refused with the
    reference's error names (src/tpu_cake/pallas_lowering.py:850-947)."""
    import pytest

    from tpu_cake_b200 import cuda_lowering, dialects, ir, schedule_lowering, workloads
    from tpu_cake_b200.identity import text_sha256

    def save(mesh_size, n, implementation, folder):
        logical = workloads.distributed_matmul_schedule(mesh_size=mesh_size, m=128, k=1024, n=n, scatter_dimension="N")
        physical = schedule_lowering.lower_distributed_matmul(logical, collective_implementation=implementation)
        plan = cuda_lowering.lower_physical_matmul_to_cuda(physical)
        folder.mkdir()
        (folder / "physical.xdsl").write_text(ir.canonical_text(physical))
        (folder / "lowered_cuda.py").write_text(plan.render_executable_source())
        return plan, folder / "physical.xdsl", folder / "lowered_cuda.py"

    plan, physical_path, source_path = save(8, 1024, dialects.CollectiveImplementation.P2P_OWNER_PUSH_BF16, tmp_path / "a")
    hashes = {"schedule_sha256": plan.schedule_sha256, "source_sha256": plan.source_sha256()}
    assert cuda_lowering.validate_saved_cuda_plan(physical_path, source_path, **hashes) == plan
    with pytest.raises(ValueError, match="SAVED_PHYSICAL_IR_HASH_MISMATCH"):
        cuda_lowering.validate_saved_cuda_plan(physical_path, source_path, schedule_sha256="0" * 64, source_sha256=hashes["source_sha256"])
    with pytest.raises(ValueError, match="SAVED_CUDA_SOURCE_HASH_MISMATCH"):
        cuda_lowering.validate_saved_cuda_plan(physical_path, source_path, schedule_sha256=hashes["schedule_sha256"], source_sha256="0" * 64)
    # A physical IR edited after the run (hash re-recorded by the forger) no longer regenerates.
    forged = tmp_path / "forged.mlir"
    forged.write_text(physical_path.read_text().replace('reducer = "sum"', 'reducer = "max"'))
    with pytest.raises(ValueError, match="SAVED_PHYSICAL_IR_INVALID"):
        cuda_lowering.validate_saved_cuda_plan(forged, source_path, schedule_sha256=text_sha256(forged.read_text()), source_sha256=hashes["source_sha256"])
    # A source edited after the run: another tile than the plan of the saved IR gives.
    edited = tmp_path / "edited.py"
    edited.write_text(source_path.read_text().replace("tile = (128, 128, 256)", "tile = (128, 128, 128)"))
    with pytest.raises(ValueError, match="SAVED_CUDA_SOURCE_PLAN_MISMATCH"):
        cuda_lowering.validate_saved_cuda_plan(physical_path, edited, schedule_sha256=hashes["schedule_sha256"], source_sha256=text_sha256(edited.read_text()))
    commented = tmp_path / "commented.py"
    commented.write_text(source_path.read_text() + "# appended\n")
    with pytest.raises(ValueError, match="SAVED_CUDA_RENDERING_MISMATCH"):
        cuda_lowering.validate_saved_cuda_plan(physical_path, commented, schedule_sha256=hashes["schedule_sha256"], source_sha256=text_sha256(commented.read_text()))
    # The source of another workload beside this IR.
    _, _, other_source = save(8, 2048, dialects.CollectiveImplementation.P2P_OWNER_PUSH_BF16, tmp_path / "b")
    with pytest.raises(ValueError, match="SAVED_PHYSICAL_IR_INVALID|SAVED_CUDA_SOURCE_PLAN_MISMATCH"):
        cuda_lowering.validate_saved_cuda_plan(physical_path, other_source, schedule_sha256=hashes["schedule_sha256"], source_sha256=text_sha256(other_source.read_text()))


def test_sharded_surface_inputs_and_host_definition(golden_dir):
    """The surface's global inputs are the reference's (hashes of all eleven arrays for the contract's
    first correctness seed and a small seed), and the host definition of the result assembles the
    eight positions' shards into the global shapes."""
    import numpy as np

    from tpu_cake_b200 import identity, rpa_cuda_lowering, rpa_surface_runner, workloads

    wanted = json.loads((golden_dir / "sharded_surface_input_hashes.json").read_text())
    for seed, hashes in wanted.items():
        inputs = workloads.inkling_sharded_fused_rpa_inputs(int(seed))
        assert [identity.array_sha256(np.asarray(value)) for value in inputs] == hashes
    plan = rpa_cuda_lowering.lower_inkling_sharded_rpa_to_cuda(workloads.inkling_sharded_rpa_schedule())
    assert [tuple(np.asarray(v).shape) for v in inputs] == [tuple(shape) for shape in plan.global_input_shapes]
    output, cache = rpa_surface_runner.expected_surface(plan, inputs)
    assert output.shape == (8, 32, 128) and cache.shape == (7424, 1, 16, 2, 128)
    # Position (1, 2) alone: its shard through the single-position definition equals its block of the assembly.
    shard = tuple(np.ascontiguousarray(v) for v in plan.shard_inputs(inputs, (1, 2)))
    local_output, _ = rpa_surface_runner.expected_fused_rpa(shard, softmax_scale=plan.local_plan.softmax_scale)
    np.testing.assert_array_equal(local_output.view(np.uint16), output[4:8, 16:24].view(np.uint16))
    assert rpa_surface_runner.SURFACE_PROTOCOL["repeat_executions"] == 2 and len(rpa_surface_runner.SURFACE_PROTOCOL["correctness_seeds"]) == 5
    maximum, relative = rpa_surface_runner.surface_error_metrics(output, output)
    assert maximum == 0.0 and relative == 0.0
