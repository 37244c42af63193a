"""Command line of the CUDA backend: the hot-path subcommands of ``tpu-cake``
(src/tpu_cake/cli.py:154-425): ``run-matmul`` (:216-232), ``search-matmul``, ``render-workload`` and
``verify-schedule`` for the distributed matmul, ``estimate`` for its cost model, ``experiment``
(:150,212,667-676) for the experiment records of the matmul and the two Inkling RPA workloads,
``run-rpa`` (the device entry point, src/tpu_cake/rpa_device_main.py), ``inspect-profile``
(:187,572-601: exit code 1 when the capture is rejected) and the receipt commands.

    python -m torch.distributed.run --nproc-per-node 8 __graft_entry__.py cli run-matmul OUT \
        --mesh-size 8 --m 128 --k 1024 --n 1024 --collective-strategy p2p_fused_epilogue
    python __graft_entry__.py cli experiment inkling-rpa
    python __graft_entry__.py cli inspect-profile launches.csv --contract expectation.json
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict
from pathlib import Path


def _add_shape(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--mesh-size", type=int, default=4)
    parser.add_argument("--m", type=int, default=16)
    parser.add_argument("--k", type=int, default=32)
    parser.add_argument("--n", type=int, default=16)
    parser.add_argument("--scatter-dimension", choices=("M", "N"), default="N")


def main(argv: list[str] | None = None) -> int:
    from . import cost_model, cuda_lowering, ir, schedule_lowering, workloads

    parser = argparse.ArgumentParser(prog="cake-b200")
    commands = parser.add_subparsers(dest="command", required=True)
    run = commands.add_parser("run-matmul", help="run the distributed matmul on the CUDA backend and write a run bundle")
    run.add_argument("output_dir", type=Path)
    _add_shape(run)
    run.add_argument("--warmup-iterations", type=int, default=3)
    run.add_argument("--measured-iterations", type=int, default=10)
    run.add_argument("--tile-m", type=int)
    run.add_argument("--tile-n", type=int)
    run.add_argument("--collective-strategy", choices=[s.value for s in cuda_lowering.MatmulCollectiveStrategy], default="nccl_reduce_scatter")
    run.add_argument("--output-dtype", choices=("f32", "bf16"), default="f32")
    run.add_argument("--mode", choices=("timing", "trace", "counters"), default="timing",
                     help="trace / counters: run the measured calls untimed for the ncu invocation profiler_config.json names")
    run.add_argument("--from-physical", type=Path, metavar="PHYSICAL.XDSL",
                     help="run the kernel a saved physical schedule holds (one this backend or the reference wrote): mesh, shapes, tile, "
                          "scatter dimension, target and collective come from the file and the shape options are ignored")
    run.add_argument("--emulate-on-one-gpu", action="store_true",
                     help="without one process per GPU: run every mesh position on this GPU (correctness only, not a multi-GPU timing)")
    run_rpa = commands.add_parser("run-rpa", help="run the fused Inkling RPA experiment (seed 97, 5 warm-up, 50 measured) and write a run bundle")
    run_rpa.add_argument("output_dir", type=Path)
    run_rpa.add_argument("--mode", choices=("timing", "trace", "counters"), default="timing")
    run_rpa.add_argument("--kv-chunk-tokens", type=int, default=0)
    run_rpa.add_argument("--from-physical", type=Path, metavar="PHYSICAL.XDSL",
                         help="run the kernel a saved physical schedule holds instead of this backend's own schedule of the experiment")
    surface = commands.add_parser("run-rpa-surface", help="run the 2 x 4 sharded RPA surface protocol (five seeds, two executions each, exact repeats and cache; chained timing rounds)")
    surface.add_argument("output_dir", type=Path)
    surface.add_argument("--emulate-on-one-gpu", action="store_true", help="run the eight mesh positions one after the other on this GPU (they exchange nothing); recorded as emulated")
    surface.add_argument("--timing-rounds", type=int, default=None, help="fewer timing rounds than the contract's 16 (the record says so)")
    verify_rpa = commands.add_parser("verify-rpa-bundle", help="re-check a finished RPA run bundle from its files")
    verify_rpa.add_argument("root", type=Path)
    experiment = commands.add_parser("experiment", help="print (or write) the experiment record of a workload")
    experiment.add_argument("workload", choices=("matmul", "inkling-rpa", "inkling-fused-rpa"))
    experiment.add_argument("--output", type=Path)
    inspect = commands.add_parser("inspect-profile", help="assess an ncu --csv launch list against a profile expectation; exit 1 if rejected")
    inspect.add_argument("capture", type=Path)
    inspect.add_argument("--contract", type=Path, required=True, help="ProfileExpectation as JSON or TOML")
    inspect.add_argument("--output", type=Path)
    bundle = commands.add_parser("finalize-matmul-bundle", help="check a timing / trace / counters triple of runs and write the bundle receipt")
    bundle.add_argument("root", type=Path, help="directory holding timing/, trace/ and counters/ run bundles")
    bundle.add_argument("--trace-profile", type=Path, required=True)
    bundle.add_argument("--counters-profile", type=Path, required=True)
    render = commands.add_parser("render-workload", help="print the canonical text of the logical or physical schedule")
    _add_shape(render)
    render.add_argument("--physical", action="store_true")
    verify = commands.add_parser("verify-schedule", help="verify a saved physical schedule (the reference's physical.xdsl text), or build, verify and hash the matmul schedules")
    verify.add_argument("schedule", type=Path, nargs="?", help="canonical text of a physical kernel; without it the schedules of the shape options are built")
    _add_shape(verify)
    estimate_cost = commands.add_parser("estimate-physical-cost", help="static resource report of a saved physical kernel, written as JSON")
    estimate_cost.add_argument("schedule", type=Path)
    estimate_cost.add_argument("--output", required=True, type=Path)
    verify_cost = commands.add_parser("verify-physical-cost", help="derive the report of a saved physical kernel again and compare it with a saved report")
    verify_cost.add_argument("report", type=Path)
    verify_cost.add_argument("--schedule", required=True, type=Path)
    search = commands.add_parser("search-matmul", help="tile search: run every candidate of a contract in alternating rounds and pick a winner")
    search.add_argument("contract", type=Path)
    search.add_argument("output_dir", type=Path)
    rpa_search_cmd = commands.add_parser("search-rpa", help="search over the decode kernel's split-KV chunk size")
    rpa_search_cmd.add_argument("contract", type=Path)
    rpa_search_cmd.add_argument("output_dir", type=Path)
    finalize = commands.add_parser("finalize-matmul-run", help="check a finished run bundle and write its receipt and roofline artifacts")
    finalize.add_argument("root", type=Path)
    finalize.add_argument("--profile", type=Path, help="ncu --csv launch list of the same run")
    verify_bundle = commands.add_parser("verify-matmul-bundle", help="re-derive everything a bundle's receipt states")
    verify_bundle.add_argument("root", type=Path)
    estimate = commands.add_parser("estimate", help="cost model of the lowered plan")
    _add_shape(estimate)
    estimate.add_argument("--collective-strategy", choices=[s.value for s in cuda_lowering.MatmulCollectiveStrategy], default="p2p_fused_epilogue_bf16_transport")
    estimate.add_argument("--physical-kernel", choices=("matmul", "inkling-rpa", "inkling-fused-rpa", "inkling-sharded-rpa"), default=None,
                          help="print the static resource report of this workload's physical kernel instead of the matmul plan's counts")
    args = parser.parse_args(argv)

    if args.command == "experiment":
        return _experiment(args.workload, args.output)
    if args.command == "inspect-profile":
        return _inspect_profile(args.capture, args.contract, args.output)
    if args.command == "run-rpa":
        from . import rpa_runner

        saved = [] if args.from_physical is None else ["--from-physical", str(args.from_physical)]
        return rpa_runner.rpa_device_main([str(args.output_dir), "--mode", args.mode, "--kv-chunk-tokens", str(args.kv_chunk_tokens), *saved])
    if args.command == "run-rpa-surface":
        from . import rpa_surface_runner
        from .mesh import ProcessMesh

        mesh = ProcessMesh.from_environment()  # one process per GPU under torch.distributed.run, else a single position
        protocol = {"timing_rounds": args.timing_rounds} if args.timing_rounds else None
        result = rpa_surface_runner.run_inkling_sharded_rpa_surface(args.output_dir, emulate_on_one_gpu=args.emulate_on_one_gpu, protocol=protocol)
        if mesh.rank == 0:
            print(f"INKLING_SHARDED_RPA_SURFACE_{'PASSED' if result['passed'] else 'FAILED'} run_id={result['run_id']} "
                  f"execution={result['execution']} median_ns={result['median_ns']:.0f}")
        return 0
    if args.command == "verify-rpa-bundle":
        from . import rpa_runner

        result = rpa_runner.validate_fused_rpa_bundle(args.root)
        print(f"FUSED_RPA_BUNDLE_VERIFIED run_id={result['run_id']} mode={result['mode']}")
        return 0
    if args.command == "finalize-matmul-bundle":
        from . import receipt as receipt_module

        document = receipt_module.finalize_matmul_bundle(args.root, trace_profile=args.trace_profile, counters_profile=args.counters_profile)
        print(json.dumps({"bundle_id": document["bundle_id"], "run_ids": document["run_ids"]}))
        return 0
    if args.command in ("finalize-matmul-run", "verify-matmul-bundle"):
        from . import receipt as receipt_module

        document = (receipt_module.finalize_matmul_run(args.root, profile_csv=args.profile) if args.command == "finalize-matmul-run"
                    else receipt_module.validate_receipt(args.root))
        print(json.dumps({"receipt_id": document["receipt_id"], "run_id": document["run_id"], **document["metrics"]}))
        return 0
    if args.command == "verify-schedule" and args.schedule is not None:
        # The reference's command (src/tpu_cake/cli.py:432-436): parse the file, verify, accept.
        from . import xdsl_text

        module = xdsl_text.parse_reference_module(args.schedule.read_text())
        module.verify()
        print(f"SCHEDULE_ACCEPTED path={args.schedule} schedule_sha256={ir.schedule_sha256(module)}")
        return 0
    if args.command in ("estimate-physical-cost", "verify-physical-cost"):
        # The reference's commands (src/tpu_cake/cli.py:439-469) on this backend's rate model.
        from . import physical_cost_model, xdsl_text

        module = xdsl_text.parse_reference_physical_kernel(args.schedule.read_text())
        module.verify()
        report = physical_cost_model.analyze_physical_kernel(module)
        document = json.dumps(report.to_json(), indent=2, sort_keys=True) + "\n"
        if args.command == "estimate-physical-cost":
            args.output.write_text(document)
            word = "PHYSICAL_COST_DERIVED"
        else:
            if json.loads(args.report.read_text()) != json.loads(document):
                raise ValueError("PHYSICAL_COST_REPORT_MISMATCH the saved report is not what the schedule derives")
            word = "PHYSICAL_COST_REPLAYED"
        print(f"{word} schedule_sha256={report.physical_schedule_sha256} mxu_regions={len(report.mxu_regions)} "
              f"limiting_priced_resource={report.predicted_limiting_priced_resource}")
        return 0
    if args.command == "search-rpa":
        from . import rpa_search

        contract = rpa_search.RpaSearchContract.from_json(args.contract.read_text())
        result = rpa_search.run_rpa_search(args.output_dir, contract)
        print(json.dumps({"search_id": result.search_id, "baseline": result.baseline, "winner": result.winner,
                          "medians_ns": {row.name: row.median_ns for row in result.candidates}}))
        return 0
    if args.command == "search-matmul":
        from . import search as search_module

        contract = search_module.MatmulSearchContract.from_json(args.contract.read_text())
        result = search_module.run_matmul_search(args.output_dir, contract)
        print(json.dumps({"search_id": result.search_id, "baseline": result.baseline, "winner": result.winner,
                          "medians_ns": {row.name: row.median_ns for row in result.candidates}}))
        return 0
    shape = dict(mesh_size=args.mesh_size, m=args.m, k=args.k, n=args.n, scatter_dimension=args.scatter_dimension)
    if args.command == "run-matmul":
        from . import runner

        if (args.tile_m is None) != (args.tile_n is None):
            parser.error("--tile-m and --tile-n come together")
        tile = schedule_lowering.MatmulTile(args.tile_m, args.tile_n) if args.tile_m is not None else None
        what = dict(mesh_size=args.mesh_size, m=args.m, k=args.k, n=args.n, tile=tile, collective_strategy=args.collective_strategy,
                    scatter_dimension=args.scatter_dimension)
        if args.from_physical is not None:
            what = runner.invocation_of_saved_schedule(args.from_physical)
        result = runner.run_distributed_matmul(
            args.output_dir, warmup_iterations=args.warmup_iterations, measured_iterations=args.measured_iterations,
            output_dtype=args.output_dtype, mode=args.mode, emulate_on_one_gpu=args.emulate_on_one_gpu, **what,
        )
        print(f"run {result.run_id[:12]} mode={result.mode} passed={result.passed} median_ns={result.median_ns} execution={result.execution}")
        return 0
    logical = workloads.distributed_matmul_schedule(**shape)
    physical = schedule_lowering.lower_distributed_matmul(logical)
    if args.command == "render-workload":
        sys.stdout.write(ir.canonical_text(physical if args.physical else logical))
        return 0
    if args.command == "verify-schedule":
        logical.verify()
        physical.verify()
        print(json.dumps({"distributed_sha256": ir.schedule_sha256(logical), "physical_sha256": ir.schedule_sha256(physical)}))
        return 0
    strategy = cuda_lowering.MatmulCollectiveStrategy(args.collective_strategy)
    if args.physical_kernel is not None:
        from . import physical_cost_model
        from .runner import _IMPLEMENTATION

        kernel = {
            "matmul": lambda: schedule_lowering.lower_distributed_matmul(logical, collective_implementation=_IMPLEMENTATION[strategy] if args.mesh_size > 1 else None),
            "inkling-rpa": workloads.paged_attention_schedule, "inkling-fused-rpa": workloads.inkling_fused_rpa_schedule,
            "inkling-sharded-rpa": workloads.inkling_sharded_rpa_schedule,
        }[args.physical_kernel]()
        print(json.dumps(physical_cost_model.analyze_physical_kernel(kernel).to_json(), indent=2))
        return 0
    plan = cuda_lowering.plan_distributed_matmul(
        mesh_size=args.mesh_size, m=args.m, k=args.k, n=args.n, scatter_dimension=0 if args.scatter_dimension == "M" else 1,
        collective_implementation=strategy if args.mesh_size > 1 else None,
    )
    report = cost_model.estimate_distributed_matmul(plan)
    print(json.dumps({**asdict(report.counts), "compute_ns": float(report.compute_ns), "memory_ns": float(report.memory_ns),
                      "communication_ns": float(report.communication_ns), "limiting_resource": report.limiting_resource}, indent=2))
    return 0


def experiment_document(workload: str) -> dict:
    """The experiment record of a workload: what is run, on what, under which protocol, and what a
    profile of it must show."""
    from . import ir, run_artifacts, schedule_lowering, workloads

    protocol = workloads.FUSED_RPA_BENCHMARK_PROTOCOL
    if workload == "matmul":
        logical = workloads.distributed_matmul_schedule(mesh_size=8, m=128, k=1024, n=1024)
        physical = schedule_lowering.lower_distributed_matmul(logical)
        return run_artifacts.experiment_record(
            workload={"name": "distributed-matmul-reduce-scatter", "mesh_size": 8, "m": 128, "k": 1024, "n": 1024, "input_dtype": "bf16",
                      "accumulate": "f32", "identity": workloads.distributed_matmul_workload_identity(8, 128, 1024, 1024)},
            schedule_sha256=ir.schedule_sha256(physical), warmup_iterations=3, measured_iterations=10,
            profile_expectation={"name": "matmul-reduce-scatter", "required_timed_hlo_markers": ["cake_matmul_rs_sm100"],
                                 "forbidden_timed_hlo_fragments": [], "require_tensor_core_activity": True},
            tolerance={"reference": "bf16(lhs).astype(f32) @ bf16(rhs).astype(f32)", "absolute_tolerance": 1e-3, "relative_tolerance": 1e-3},
        )
    if workload == "inkling-rpa":
        # The prototype decode op over separate caches with the reference's toy shapes
        # (src/tpu_cake/workloads/inkling_rpa.py:693-722, 937-964).
        schedule = workloads.paged_attention_schedule()
        tensors = (("query", (4, 4, 32), "bf16"), ("key_cache", (32, 16, 4, 32), "bf16"), ("value_cache", (32, 16, 4, 32), "bf16"),
                   ("page_table", (4, 8), "i32"), ("sequence_lengths", (4,), "i32"), ("relative_bias", (4, 128), "bf16"))
        return run_artifacts.experiment_record(
            workload={"name": "inkling-ragged-paged-relative-bias-attention", "stage": "steady_decode",
                      "inputs": [{"name": n, "shape": list(shape), "dtype": dtype} for n, shape, dtype in tensors],
                      "outputs": [{"name": "output", "shape": [4, 4, 32], "dtype": "bf16"}]},
            schedule_sha256=ir.schedule_sha256(schedule), warmup_iterations=protocol["warmup_iterations"],
            measured_iterations=protocol["measured_iterations"],
            profile_expectation={"name": "inkling-rpa-steady-decode", "required_timed_hlo_markers": ["cake_rpa_decode_sm100"],
                                 "forbidden_timed_hlo_fragments": ["flash_fwd", "paged_attention_v", "BatchDecode"],
                                 "require_tensor_core_activity": False},
            tolerance={"reference": "softmax(q.k / D + bias) v in float32 per request", "absolute_tolerance": 0.02, "relative_tolerance": 0.02},
        )
    schedule = workloads.inkling_fused_rpa_schedule()
    return run_artifacts.experiment_record(
        workload={"name": "inkling-fused-ragged-paged-attention", "stage": "steady_decode", "seed": protocol["seed"]},
        schedule_sha256=ir.schedule_sha256(schedule), warmup_iterations=protocol["warmup_iterations"],
        measured_iterations=protocol["measured_iterations"],
        profile_expectation={"name": "inkling-fused-rpa-steady-decode", "required_timed_hlo_markers": ["cake_rpa_decode_sm100"],
                             "forbidden_timed_hlo_fragments": ["flash_fwd", "paged_attention_v", "BatchDecode"],
                             "require_tensor_core_activity": False},
        tolerance={"absolute_tolerance": 0.02, "relative_tolerance": 0.02, "cache": "bit-exact"},
    )


def _experiment(workload: str, output: Path | None) -> int:
    from .identity import semantic_sha256

    document = experiment_document(workload)
    rendered = json.dumps(document, indent=2, sort_keys=True) + "\n"
    if output is None:
        sys.stdout.write(rendered)
    else:
        output.parent.mkdir(parents=True, exist_ok=True)
        output.write_text(rendered)
        print(f"EXPERIMENT_WRITTEN workload={workload} id={semantic_sha256('experiment', rendered)} path={output}")
    return 0


def load_profile_expectation(path: Path):
    """A ProfileExpectation from JSON, or from TOML as the reference's contracts are written."""
    from . import profile_evidence

    text = path.read_text()
    if path.suffix == ".toml":
        import tomllib

        raw = tomllib.loads(text)
    else:
        raw = json.loads(text)
    unknown = set(raw) - set(profile_evidence.ProfileExpectation.__dataclass_fields__)
    if unknown:
        raise ValueError(f"unknown profile expectation fields {sorted(unknown)}")
    for key in ("required_timed_hlo_markers", "forbidden_timed_hlo_fragments"):
        if key in raw:
            raw[key] = tuple(raw[key])
    return profile_evidence.ProfileExpectation(**raw)


def _inspect_profile(capture: Path, contract_path: Path, output: Path | None) -> int:
    from . import profile_evidence

    expectation = load_profile_expectation(contract_path)
    assessment = profile_evidence.assess_capture(capture, expectation)
    print(f"PROFILE_{'ACCEPTED' if assessment.accepted else 'REJECTED'} contract={expectation.name}")
    for finding in assessment.findings:
        print(f"ERROR {finding.code}: {finding.message}" + (f" ({', '.join(finding.evidence)})" if finding.evidence else ""))
    print("EVIDENCE " + " ".join(f"{marker}={count}launches/{assessment.marker_time_ns.get(marker, 0.0):.0f}ns"
                                 for marker, count in assessment.marker_launches.items()))
    if output is not None:
        output.parent.mkdir(parents=True, exist_ok=True)
        output.write_text(json.dumps({"accepted": assessment.accepted, "contract": expectation.name,
                                      "findings": [asdict(f) for f in assessment.findings], "marker_launches": assessment.marker_launches,
                                      "marker_time_ns": assessment.marker_time_ns}, indent=2) + "\n")
    return 0 if assessment.accepted else 1


if __name__ == "__main__":
    raise SystemExit(main())
