"""Command line of the CUDA backend: the hot-path subcommands of ``tpu-cake``
(src/tpu_cake/cli.py:154-425): ``run-matmul`` (:216-232), ``render-workload`` and
``verify-schedule`` for the distributed matmul, and ``estimate`` for its cost model.

    python __graft_entry__.py cli run-matmul OUT --mesh-size 8 --m 128 --k 1024 --n 1024
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
    render = commands.add_parser("render-workload", help="print the canonical text of the logical or physical schedule")
    _add_shape(render)
    render.add_argument("--physical", action="store_true")
    verify = commands.add_parser("verify-schedule", help="build, verify and hash the schedules")
    _add_shape(verify)
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
    args = parser.parse_args(argv)

    if args.command in ("finalize-matmul-run", "verify-matmul-bundle"):
        from . import receipt as receipt_module

        document = (receipt_module.finalize_matmul_run(args.root, profile_csv=args.profile) if args.command == "finalize-matmul-run"
                    else receipt_module.validate_receipt(args.root))
        print(json.dumps({"receipt_id": document["receipt_id"], "run_id": document["run_id"], **document["metrics"]}))
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
        result = runner.run_distributed_matmul(
            args.output_dir, mesh_size=args.mesh_size, m=args.m, k=args.k, n=args.n, warmup_iterations=args.warmup_iterations,
            measured_iterations=args.measured_iterations, tile=tile, collective_strategy=args.collective_strategy,
            scatter_dimension=args.scatter_dimension, output_dtype=args.output_dtype,
        )
        print(f"run {result.run_id[:12]} passed={result.passed} median_ns={result.median_ns} execution={result.execution}")
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
    plan = cuda_lowering.plan_distributed_matmul(
        mesh_size=args.mesh_size, m=args.m, k=args.k, n=args.n, scatter_dimension=0 if args.scatter_dimension == "M" else 1,
        collective_implementation=strategy if args.mesh_size > 1 else None,
    )
    report = cost_model.estimate_distributed_matmul(plan)
    print(json.dumps({**asdict(report.counts), "compute_ns": float(report.compute_ns), "memory_ns": float(report.memory_ns),
                      "communication_ns": float(report.communication_ns), "limiting_resource": report.limiting_resource}, indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
