"""Benchmark of the hot path on N B200s of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      (the CPU path on host cores)

Headline: the large K-sharded BF16 matmul + reduce-scatter, A[8192,16384] x B[16384,8192], K split
over the N ranks, result reduce-scattered along M into bf16 [8192/N, 8192] per GPU. One step = one
pass of cake_matmul_rs_sm100 (+ cake_reduce_slots_sm100 when N > 1). The total work is fixed, so
scaling is "strong". A second object, "rpa_decode", reports the ragged-paged-attention decode
(HBM-bound): 64 sequences on one GPU, or the 256-sequence configuration with KV heads sharded over
the ranks and outputs all-gathered ("rpa_decode_sharded", at every N including 1, so its curve has
its own anchor). A third object at N = 1, "rpa_mixed", reports the mixed batch (8 prefill + 120
decode sequences): the whole step, and its decode and prefill parts alone.

Parity: outside the timed regions every rank compares sampled rows of its local matmul output with
the oracle's split-K reduce-scatter (plus the row-sum identity over the whole local output), and
sampled sequences of the attention result -- the gathered buffer when sharded -- with the oracle,
three different steps in a row; the line carries "parity" objects and the exit code is non-zero if
any rank disagrees.

Timing: CUDA events on the stream the kernels are launched on, one event pair per step, a write of
a buffer larger than L2 between steps, barrier + synchronize on both sides of the timed region,
maximum over ranks. Clocks and throttle reasons are sampled with nvidia-smi during the region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__  # noqa: E402

M, K, N = 8192, 16384, 8192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/: cake_matmul_rs_sm100<256> on 8192x16384x8192 (2.276 GB read + 0.129 GB written) and
# cake_rpa_decode_sm100 on the 64-sequence decode configuration (1.090 GB read + 0.012 GB written).
MEASURED_TRAFFIC_BYTES = {"matmul_n1": 2_405_254_744, "rpa_decode_64": 1_102_643_400}


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    QUERY = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.process: subprocess.Popen | None = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.process = None
        time.sleep(0.3)  # let nvidia-smi start sampling before the GPU work begins

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(self.NAMES, parts[3:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


def reduce_max(mesh, value: float) -> float:
    if mesh.world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=mesh.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=mesh.group)
    return float(t.item())


def all_ranks_ok(mesh, ok: bool) -> bool:
    return reduce_max(mesh, 0.0 if ok else 1.0) == 0.0


def matmul_config(world: int, collective: str) -> dict:
    """The workload description both arms print (the reference arm names the same configuration)."""
    return {
        "workload": f"K-sharded bf16 matmul {M}x{K}x{N} + reduce-scatter along M to bf16 [{M // world},{N}] per GPU",
        "m": M, "k": K, "n": N, "mesh": world, "accumulate": "f32", "collective": collective,
        "l2": "256 MiB flush between steps",
    }


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


class blas_threads:
    """Runs the numpy oracle on every host core this process may use, whatever OMP_NUM_THREADS the
    launcher exported (torch.distributed.run sets it to 1), and reports the count actually in use."""

    def __init__(self):
        self.used = 1
        self._limit = None

    def __enter__(self):
        try:
            import threadpoolctl

            self._limit = threadpoolctl.threadpool_limits(limits=host_threads())
            self._limit.__enter__()
            pools = [pool for pool in threadpoolctl.threadpool_info() if pool.get("user_api") == "blas"]
            self.used = max([int(pool.get("num_threads", 1)) for pool in pools] or [1])
        except Exception:  # noqa: BLE001 - threadpoolctl absent or no BLAS pool: single-threaded numpy
            self.used = 1
        return self

    def __exit__(self, *exc):
        if self._limit is not None:
            self._limit.__exit__(*exc)
        return False


def timed_steps(mesh, step, steps: int, warmup: int, flush) -> tuple[float, list[float]]:
    """Runs ``warmup`` untimed and ``steps`` timed calls of ``step``; returns (total ms = max over
    ranks of the sum of per-step device times, this rank's per-step ms)."""
    import torch

    for _ in range(warmup):
        flush()
        step()
    mesh.barrier()
    torch.cuda.synchronize(mesh.device)
    pairs = []
    for _ in range(steps):
        flush()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        step()
        stop.record()
        pairs.append((start, stop))
    torch.cuda.synchronize(mesh.device)
    mesh.barrier()
    per_step = [a.elapsed_time(b) for a, b in pairs]
    return reduce_max(mesh, sum(per_step)), per_step


def cpu_matmul_sample(rows: int) -> dict:
    """Times the oracle (numpy float32 matmul on bf16-valued inputs) on ``rows`` lhs rows of the
    headline shape, on every host core this process may use."""
    from oracle import matmul_rs

    generator = np.random.default_rng(0)
    lhs = matmul_rs.quantize_bf16(generator.normal(scale=K**-0.5, size=(rows, K)).astype(np.float32))
    rhs = matmul_rs.quantize_bf16(generator.normal(scale=K**-0.5, size=(K, N)).astype(np.float32))
    with blas_threads() as pool:
        matmul_rs.matmul_reference(lhs[:64], rhs)
        best = float("inf")
        repeats = 0
        budget_started = time.perf_counter()
        while repeats < 3 or (time.perf_counter() - budget_started < 10.0 and repeats < 20):
            started = time.perf_counter()
            matmul_rs.matmul_reference(lhs, rhs)
            best = min(best, time.perf_counter() - started)
            repeats += 1
    return {
        "value": 2.0 * rows * K * N / best / 1e12,
        "unit": "TFLOP/s",
        "cores": pool.used,
        "kind": "port",
        "sample": f"{rows} of {M} lhs rows of the {M}x{K}x{N} product, numpy float32 matmul, best of {repeats}",
        "seconds": best,
    }


def cpu_rpa_sample(lengths: np.ndarray, table: np.ndarray, config, sequences: int) -> dict:
    from oracle import rpa
    from tpu_cake_b200 import workloads

    generator = np.random.default_rng(1)
    order = np.argsort(lengths)[:: max(1, len(lengths) // sequences)][:sequences]
    total_bytes, seconds = 0, 0.0
    pool = blas_threads().__enter__()
    for s in order:
        count = -(-int(lengths[s]) // config.page_size)
        keys = generator.standard_normal((count, config.page_size, config.kv_heads, config.head_dim), dtype=np.float32)
        values = generator.standard_normal((count, config.page_size, config.kv_heads, config.head_dim), dtype=np.float32)
        query = generator.standard_normal((1, config.q_heads, config.head_dim), dtype=np.float32)
        started = time.perf_counter()
        rpa.rpa_separate(query, keys, values, np.arange(count, dtype=np.int32)[None, :], lengths[s : s + 1], None, scale=config.softmax_scale)
        seconds += time.perf_counter() - started
        total_bytes += workloads.decode_algorithmic_bytes(lengths[s : s + 1], config.q_heads, config.kv_heads, config.head_dim, config.page_size)
    pool.__exit__(None, None, None)
    return {
        "value": total_bytes / seconds / 1e9,
        "unit": "GB/s",
        "cores": pool.used,
        "kind": "port",
        "sample": f"{len(order)} of {len(lengths)} sequences of {config.name}, numpy oracle, algorithmic bf16 bytes / wall time",
        "seconds": seconds,
    }


# ----------------------------------------------------------------------------------------- ours


def bench_matmul(mesh, args, peaks, peak_kind) -> dict:
    import torch

    from tpu_cake_b200 import cuda_lowering

    world = mesh.world
    strategy = {
        "p2p_bf16": cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT,
        "p2p_f32": cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE,
        "nccl": cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER,
    }[args.strategy]
    plan = cuda_lowering.plan_distributed_matmul(
        mesh_size=world, m=M, k=K, n=N, scatter_dimension=0, output_dtype="bf16", tile_n=256,
        collective_implementation=strategy if world > 1 else None,
    )
    executable, _ = plan.build(mesh=mesh)
    k_local = K // world
    # Every rank draws the whole operands from the same seed and keeps its K slice; what the parity
    # check needs of the whole (sampled lhs rows, rhs, the row-sum identity) is taken before the rest
    # is freed.
    generator = torch.Generator(device=mesh.device).manual_seed(20261125)
    lhs_full = (torch.randn((M, K), generator=generator, device=mesh.device) * K**-0.5).to(torch.bfloat16)
    lhs = lhs_full[:, mesh.rank * k_local : (mesh.rank + 1) * k_local].contiguous()
    rhs_full = (torch.randn((K, N), generator=generator, device=mesh.device) * K**-0.5).to(torch.bfloat16)
    rhs = rhs_full[mesh.rank * k_local : (mesh.rank + 1) * k_local].contiguous()
    local_rows = M // world
    sampled = sorted({0, 1, 127, 128, local_rows // 2, local_rows - 129, local_rows - 2, local_rows - 1})
    sampled_rows = torch.tensor(sampled, device=mesh.device)
    parity_inputs = {
        "rows": sampled,
        "lhs_rows": lhs_full[mesh.rank * local_rows + sampled_rows].float().cpu().numpy(),
        "rhs": rhs_full.float().cpu().numpy(),
        # C 1 = A (B 1): the row sums this rank's local output must have, in float64.
        "row_sums": lhs_full[mesh.rank * local_rows : (mesh.rank + 1) * local_rows].double() @ rhs_full.double().sum(dim=1),
    }
    del lhs_full, rhs_full
    out = torch.empty(plan.output_local_shape, dtype=torch.bfloat16, device=mesh.device)
    flush_buffer = torch.empty(256 << 20, dtype=torch.uint8, device=mesh.device)

    def flush():
        flush_buffer.fill_(1)

    def step():
        executable(lhs, rhs, out)

    sampler = ClockSampler(mesh.device.index)
    sampler.start()
    total_ms, per_step = timed_steps(mesh, step, args.steps, args.warmup, flush)
    clocks = sampler.stop()
    executable.status()
    parity = matmul_parity(mesh, plan, out, parity_inputs)
    del parity_inputs
    launches = executable.launches_per_call * args.steps
    flops_total = 2.0 * M * N * K
    ms_per_step = total_ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # Roofline of the dominant kernel: at N = 1 the step is exactly one cake_matmul_rs_sm100
    # launch; at N > 1 the event pair also spans the slot reduction, so the figure is conservative.
    kernel_ms = statistics.mean(per_step)
    achieved = (flops_total / world) / (kernel_ms * 1e-3) / 1e12
    peak = float(peaks["bf16_tflops"])
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "traffic": MEASURED_TRAFFIC_BYTES["matmul_n1"] if world == 1 else None,
        "peak_source": f"{peak_kind}: cuBLAS bf16 burst", "frac_of_sustained": achieved / float(peaks["bf16_tflops_sustained"]),
        "kernel": "cake_matmul_rs_sm100<256>", "kernel_ms": kernel_ms,
    }

    # How much of the step is communication that the contraction does not hide: the same kernel,
    # tiles and transport dtype with the partial left in local memory ("pushes disabled"), and the
    # two halves of the peer-to-peer step timed separately.
    phases = None
    if world > 1 and strategy is not cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER:
        twin = cuda_lowering.MatmulRsExecutable(plan, mesh, contraction_only=True)
        only_ms, _ = timed_steps(mesh, lambda: twin(lhs, rhs), args.steps, 3, flush)
        twin.close()
        push_ms, reduce_ms = 0.0, 0.0
        mesh.barrier()
        for _ in range(args.steps):
            flush()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            executable.push(lhs, rhs)
            e1.record()
            executable.reduce(out)
            e2.record()
            torch.cuda.synchronize(mesh.device)
            push_ms += e0.elapsed_time(e1)
            reduce_ms += e1.elapsed_time(e2)
        mesh.barrier()
        executable.status()
        only_ms /= args.steps
        phases = {
            "contraction_only_ms": only_ms,
            "push_kernel_ms": reduce_max(mesh, push_ms / args.steps),
            "reduce_kernel_ms": reduce_max(mesh, reduce_ms / args.steps),
            "exposed_communication": max(0.0, (ms_per_step - only_ms) / ms_per_step),
            "link_egress_bytes_per_gpu": plan.collective_resources.remote_payload_bytes,
        }
        # Roofline of the fused step: the slower of the contraction at the measured bf16 burst and the
        # link egress at the measured peer-copy rate of one direction (770 GB/s).
        tensor_ms = flops_total / world / (peak * 1e12) * 1e3
        link_ms = phases["link_egress_bytes_per_gpu"] / 770e9 * 1e3
        phases["fused_target"] = {
            "tensor_ms": tensor_ms, "link_ms": link_ms, "link_peak_gbs": 770.0, "bound": "tensor" if tensor_ms >= link_ms else "link",
            "frac": max(tensor_ms, link_ms) / ms_per_step,
        }

    # End to end through the C ABI with host buffers (pinned): H2D of both operands, the kernels,
    # D2H of the local output, inside the timed region.
    e2e = None
    if strategy is not cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER or world == 1:
        lhs_host = lhs.cpu().view(torch.uint16).pin_memory().numpy()
        rhs_host = rhs.cpu().view(torch.uint16).pin_memory().numpy()
        out_host = torch.empty(plan.output_local_shape, dtype=torch.uint16).pin_memory().numpy()
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            executable.run_host(lhs_host, rhs_host, out_host)
        mesh.barrier()
        torch.cuda.synchronize(mesh.device)
        started = time.perf_counter()
        for _ in range(e2e_steps):
            executable.run_host(lhs_host, rhs_host, out_host)
        torch.cuda.synchronize(mesh.device)
        elapsed = reduce_max(mesh, time.perf_counter() - started)
        mesh.barrier()
        executable.status()
        # The host-buffer call may cut the matrix into blocks of rows; its bits must not differ.
        same = bool(np.array_equal(out_host, out.cpu().view(torch.uint16).numpy()))
        if not all_ranks_ok(mesh, same):
            raise SystemExit("PARITY_FAILED: cake_matmul_rs_run_host and the device-buffer call disagree")
        e2e = {
            "bit_identical_to_device_call": True,
            "value": flops_total / (elapsed / e2e_steps) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(lhs_host.nbytes + rhs_host.nbytes), "d2h_bytes_per_step": int(out_host.nbytes),
            "ms_per_step": elapsed / e2e_steps * 1e3, "steps": e2e_steps, "api": "cake_matmul_rs_run_host",
        }
    executable.close()
    del lhs, rhs, out, flush_buffer
    torch.cuda.empty_cache()
    return {
        "value": value, "ms_per_step": ms_per_step, "roofline": roofline, "e2e": e2e, "clocks": clocks,
        "gpu_launches": launches, "strategy": args.strategy if world > 1 else "single", "phases": phases,
        "parity": parity,
    }


def bench_matmul_c1_latency(mesh, calls: int = 200) -> dict:
    """The reference's CPU-runnable case on the GPUs it names: mesh 8, A[128,1024] x B[1024,1024]
    (K = 128 per GPU), partials reduce-scattered along N in f32 -- 33.5 MFLOP and 458,752 bytes of
    egress per GPU, so the step is latency: launch, one tile's contraction, the push across the
    link, the flag round trip and the slot reduction. Median of ``calls`` device-timed calls; the
    output is checked with the reference's allclose(1e-3, 1e-3) first."""
    import torch

    from oracle import matmul_rs
    from tpu_cake_b200 import cuda_lowering, workloads

    world = mesh.world
    m, k, n = 128, 1024, 1024
    plan = cuda_lowering.plan_distributed_matmul(
        mesh_size=world, m=m, k=k, n=n, scatter_dimension=1, output_dtype="f32", tile_n=128,
        collective_implementation=cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE,
    )
    executable, _ = plan.build(mesh=mesh)
    lhs, rhs = workloads.distributed_matmul_inputs(world, m, k, n)
    lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, world, mesh.rank)
    lhs_d = torch.from_numpy(np.ascontiguousarray(lhs_r).view(np.uint16).copy()).view(torch.bfloat16).to(mesh.device)
    rhs_d = torch.from_numpy(np.ascontiguousarray(rhs_r).view(np.uint16).copy()).view(torch.bfloat16).to(mesh.device)
    out = torch.empty(plan.output_local_shape, dtype=torch.float32, device=mesh.device)
    for _ in range(10):
        executable(lhs_d, rhs_d, out)
    torch.cuda.synchronize(mesh.device)
    expected = matmul_rs.matmul_reduce_scatter(lhs.astype(np.float32), rhs.astype(np.float32), world=world, scatter_dimension=1)[mesh.rank]
    ok = all_ranks_ok(mesh, bool(np.allclose(out.cpu().numpy(), expected, atol=1e-3, rtol=1e-3)))
    mesh.barrier()
    pairs = []
    for _ in range(calls):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        executable(lhs_d, rhs_d, out)
        stop.record()
        pairs.append((start, stop))
    torch.cuda.synchronize(mesh.device)
    executable.status()
    samples = sorted(a.elapsed_time(b) * 1e3 for a, b in pairs)
    median_us = reduce_max(mesh, samples[len(samples) // 2])
    p90_us = reduce_max(mesh, samples[int(len(samples) * 0.9)])
    executable.close()
    return {
        "metric": "matmul_c1_latency_us", "value": median_us, "unit": "us", "higher_is_better": False, "p90_us": p90_us, "calls": calls,
        "config": {"workload": f"run-matmul --mesh-size {world} --m {m} --k {k} --n {n}: bf16 inputs, f32 partials reduce-scattered along N",
                   "collective": "p2p_f32", "launch": "stream, back to back"},
        "note": "latency-bound (tens of MFLOP and a few hundred KB of link egress per GPU): a roofline fraction would be meaningless",
        "flops_per_gpu": 2 * m * (k // world) * n, "link_egress_bytes_per_gpu": (world - 1) * m * (n // world) * 4,
        "parity": {"checked": "the local [128, 128] output of every rank against the oracle, allclose(1e-3, 1e-3)", "ok": ok},
        "gpu_launches": calls,
    }


def matmul_parity(mesh, plan, out, inputs) -> dict:
    """This rank's local output of the last timed step against the oracle: the sampled rows must
    equal the rank-ordered sum of the W split-K partials (rounded to the transport and output dtypes
    as the device does) within max-abs 2e-2 and relative-L2 1e-2, and every row's sum must satisfy
    C 1 = A (B 1) within 2e-2 (the accumulated bf16 rounding of 8192 outputs of magnitude ~1/128).
    All ranks check; the verdict is the logical AND, the errors the maxima over ranks."""
    import torch

    from oracle import matmul_rs

    expected = matmul_rs.reduced_rows(inputs["lhs_rows"], inputs["rhs"], world=mesh.world,
                                      transport_dtype=plan.transport_dtype if mesh.world > 1 else "f32", out_dtype=plan.output_dtype)
    rows = torch.tensor(inputs["rows"], device=out.device)
    actual = out[rows].float().cpu().numpy()
    max_abs = matmul_rs.max_abs_error(actual, expected)
    rel_l2 = matmul_rs.relative_l2_error(actual, expected)
    row_sum_error = float((out.double().sum(dim=1) - inputs["row_sums"]).abs().max().item())
    finite = bool(torch.isfinite(out.float()).all().item())
    ok = finite and max_abs <= 2e-2 and rel_l2 <= 1e-2 and row_sum_error <= 2e-2
    return {
        "checked": f"{len(inputs['rows'])} rows x {out.shape[1]} columns per rank against the oracle's split-K reduce-scatter, "
                   f"and the row-sum identity over all {out.shape[0]} local rows, on every rank",
        "max_abs": reduce_max(mesh, max_abs), "rel_l2": reduce_max(mesh, rel_l2), "row_sum_max_abs": reduce_max(mesh, row_sum_error),
        "tolerance": {"max_abs": 2e-2, "rel_l2": 1e-2, "row_sum_max_abs": 2e-2}, "ok": all_ranks_ok(mesh, ok),
    }


def bench_rpa(mesh, args, peaks, peak_kind, config) -> dict:
    """Decode step of ``config`` with its KV heads sharded over the mesh (world 1: all heads here, no
    collective)."""
    import torch

    from tpu_cake_b200 import rpa_cuda_lowering, workloads

    world = mesh.world
    if args.rpa_pool_pages:
        import dataclasses

        config = dataclasses.replace(config, total_pages=args.rpa_pool_pages)
    lengths, table = workloads.decode_metadata(config)
    local_kv = config.kv_heads // world
    local_q = config.q_heads // world
    generator = torch.Generator(device=mesh.device).manual_seed(1000 + mesh.rank)
    shape = (config.total_pages, config.page_size, local_kv, 2, config.head_dim)
    cache = torch.empty(shape, dtype=torch.bfloat16, device=mesh.device)
    block = 4096
    for start in range(0, config.total_pages, block):
        stop = min(config.total_pages, start + block)
        cache[start:stop] = torch.randn((stop - start, *shape[1:]), generator=generator, device=mesh.device).to(torch.bfloat16)
    query = torch.randn((config.num_seqs, local_q, config.head_dim), generator=generator, device=mesh.device).to(torch.bfloat16)
    table_d = torch.from_numpy(table).to(mesh.device)
    lengths_d = torch.from_numpy(lengths).to(mesh.device)
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name=config.name, schedule_sha256="0" * 64, query_shape=(config.num_seqs, local_q, config.head_dim),
        cache_shape=(config.total_pages, config.page_size, local_kv, config.head_dim), page_table_shape=table.shape,
        bias_shape=None, softmax_scale=config.softmax_scale, cache_layout="fused", kv_chunk_tokens=args.kv_chunk,
    )
    executable = plan.build(mesh.device)
    out = torch.empty_like(query)
    gathered = gather_buffer = gather_flags = None
    if world > 1 and args.rpa_gather == "nccl":
        gathered = torch.empty((world, config.num_seqs, local_q, config.head_dim), dtype=torch.bfloat16, device=mesh.device)
    elif world > 1:
        # Outputs are written straight into every rank's gathered buffer over peer memory.
        from tpu_cake_b200.mesh import SymmetricBuffer

        # two halves: call n fills half n & 1, so a rank one call ahead never disturbs a peer's reader
        gather_buffer = SymmetricBuffer(mesh, 2 * world * config.num_seqs * local_q * config.head_dim * 2)
        gather_flags = SymmetricBuffer(mesh, 64)
        gather_view = gather_buffer.as_tensor(torch.bfloat16, (2, world, config.num_seqs, local_q, config.head_dim))
    flush_buffer = torch.empty(256 << 20, dtype=torch.uint8, device=mesh.device)

    def flush():
        flush_buffer.fill_(1)

    last_half = [0]

    def step():
        if gather_buffer is not None:
            last_half[0] = executable.enqueue_allgather(query, cache, None, lengths_d, table_d, gather_buffer.pointers,
                                                        gather_flags.pointers, world, mesh.rank)
            return
        plan.invoke(executable, query, cache, None, table_d, lengths_d, out=out)
        if world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(gathered, out, group=mesh.group)

    def result_rows(sample):
        """[n, all query heads, head_dim] of the sequences in ``sample`` from the step just enqueued."""
        if gather_buffer is not None:
            return gather_view[last_half[0]][:, sample].permute(1, 0, 2, 3).reshape(len(sample), config.q_heads, config.head_dim)
        if gathered is not None:
            return gathered[:, sample].permute(1, 0, 2, 3).reshape(len(sample), config.q_heads, config.head_dim)
        return out[sample]

    steps = max(args.steps, 10)
    launch_mode = "stream"
    if world == 1 and not args.no_graph:
        # The step is three short kernels: replaying them from a CUDA graph removes the launch gaps.
        step()
        torch.cuda.synchronize(mesh.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            plan.invoke(executable, query, cache, None, table_d, lengths_d, out=out)
        eager_step = step

        def step():
            graph.replay()

        launch_mode = "cuda-graph"
    total_ms, per_step = timed_steps(mesh, step, steps, max(args.warmup, 3), flush)
    executable.status()
    parity = rpa_parity(mesh, config, lengths, table, cache, query, step, result_rows)
    executable.status()
    bytes_total = workloads.decode_algorithmic_bytes(lengths, config.q_heads, config.kv_heads, config.head_dim, config.page_size)
    ms_per_step = total_ms / steps
    value = bytes_total / (ms_per_step * 1e-3) / 1e9
    achieved = (bytes_total / world) / (statistics.mean(per_step) * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    result = {
        "metric": "rpa_decode_hbm_gbs", "value": value, "unit": "GB/s", "ms_per_step": ms_per_step, "steps": steps,
        "config": {
            "workload": config.name, "num_seqs": config.num_seqs, "q_heads": config.q_heads, "kv_heads": config.kv_heads,
            "head_dim": config.head_dim, "page_size": config.page_size, "total_pages": config.total_pages,
            "kv_tokens": int(lengths.astype(np.int64).sum()), "sharding": f"kv_heads/{world}" if world > 1 else "none",
            "collective": ("none" if world == 1 else "nccl all_gather of outputs" if gather_buffer is None else "peer-to-peer stores into every rank's gathered buffer + flag barrier"), "l2": "256 MiB flush between steps",
            "launch": launch_mode,
        },
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": MEASURED_TRAFFIC_BYTES["rpa_decode_64"] if (world == 1 and config.num_seqs == 64) else None,
            "peak_source": f"{peak_kind}: device copy bandwidth", "kernel": "cake_rpa_decode_sm100 (+plan, combine)",
            "algorithmic_bytes": bytes_total // world,
        },
        "gpu_launches": executable.launches_per_call * steps,
        "parity": parity,
    }
    # End to end: per-step inputs (queries, lengths, page table) come from pinned host memory and the
    # outputs go back; the KV pool is resident state, as in serving.
    q_host = query.cpu().pin_memory()
    table_host = table_d.cpu().pin_memory()
    lengths_host = lengths_d.cpu().pin_memory()
    result_device = out if gather_buffer is None else gather_view[0]
    if gathered is not None:
        result_device = gathered
    out_host = torch.empty(result_device.shape, dtype=result_device.dtype).pin_memory()
    e2e_steps = 10
    mesh.barrier()
    torch.cuda.synchronize(mesh.device)
    started = time.perf_counter()
    for _ in range(e2e_steps):
        query.copy_(q_host, non_blocking=True)
        table_d.copy_(table_host, non_blocking=True)
        lengths_d.copy_(lengths_host, non_blocking=True)
        step()
        out_host.copy_(result_device if gather_buffer is None else gather_view[last_half[0]], non_blocking=True)
        torch.cuda.synchronize(mesh.device)
    elapsed = reduce_max(mesh, time.perf_counter() - started)
    result["e2e"] = {
        "value": bytes_total / (elapsed / e2e_steps) / 1e9, "unit": "GB/s",
        "h2d_bytes_per_step": int(q_host.nbytes + table_host.nbytes + lengths_host.nbytes), "d2h_bytes_per_step": int(out_host.nbytes),
        "ms_per_step": elapsed / e2e_steps * 1e3,
    }
    if world == 1 and mesh.rank == 0 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_rpa_sample(lengths, table, config, 32 if config.num_seqs <= 64 else 8)
    executable.close()
    for buffer in (gather_buffer, gather_flags):
        if buffer is not None:
            buffer.close()
    return result


def rpa_parity(mesh, config, lengths, table, cache, query, step, result_rows) -> dict:
    """Three steps in a row with three different query tensors (the timed one, its negative, its
    half) and no host synchronisation between them; after each, the rows of four sampled sequences
    (shortest, longest, two between) are copied from where the step left its result -- the gathered
    buffer of all ranks' heads when the decode is sharded. Every rank compares all query heads of
    those rows with the oracle: each rank runs the oracle on the KV heads it holds and the expected
    rows are exchanged over torch.distributed. Tolerance: max-abs 2e-2, relative-L2 1e-2."""
    import torch

    from oracle import matmul_rs, rpa

    order = np.argsort(lengths)
    count = len(order)
    sample = sorted({int(order[0]), int(order[count // 3]), int(order[2 * count // 3]), int(order[-1])})
    sample_device = torch.tensor(sample, device=mesh.device)
    base = query.clone()
    factors = (1.0, -1.0, 0.5)
    snapshots = []
    for factor in factors:
        query.copy_((base.float() * factor).to(torch.bfloat16))
        step()
        snapshots.append(result_rows(sample_device).clone())
    query.copy_(base)
    torch.cuda.synchronize(mesh.device)
    pages_of = {}
    for s in sample:
        pages = -(-int(lengths[s]) // config.page_size)
        index = torch.from_numpy(table[s, :pages].astype(np.int64)).to(mesh.device)
        pages_of[s] = cache[index].float().cpu().numpy()  # [pages, page_size, local KV heads, 2, head_dim]
    max_abs, rel_l2, finite = 0.0, 0.0, True
    for factor, snapshot in zip(factors, snapshots):
        expected_local = np.zeros((len(sample), query.shape[1], config.head_dim), dtype=np.float32)
        for i, s in enumerate(sample):
            rows = pages_of[s]
            q = (base[s : s + 1].float() * factor).to(torch.bfloat16).float().cpu().numpy()
            expected_local[i] = rpa.rpa_separate(q, rows[:, :, :, 0, :], rows[:, :, :, 1, :], np.arange(rows.shape[0], dtype=np.int32)[None, :],
                                                 lengths[s : s + 1], None, scale=config.softmax_scale)[0]
        if mesh.world > 1:
            import torch.distributed as dist

            mine = torch.from_numpy(expected_local).to(mesh.device)
            everyone = torch.empty((mesh.world,) + tuple(mine.shape), dtype=mine.dtype, device=mesh.device)
            dist.all_gather_into_tensor(everyone, mine, group=mesh.group)
            expected = everyone.permute(1, 0, 2, 3).reshape(len(sample), config.q_heads, config.head_dim).cpu().numpy()
        else:
            expected = expected_local
        actual = snapshot.float().cpu().numpy()
        finite = finite and bool(np.isfinite(actual).all())
        max_abs = max(max_abs, matmul_rs.max_abs_error(actual, expected))
        rel_l2 = max(rel_l2, matmul_rs.relative_l2_error(actual, expected))
    ok = finite and max_abs <= 2e-2 and rel_l2 <= 1e-2
    return {
        "checked": f"{len(sample)} sequences x {config.q_heads} query heads, 3 steps in a row, "
                   f"{'the gathered buffer on every rank' if mesh.world > 1 else 'the output buffer'} against the oracle",
        "max_abs": reduce_max(mesh, max_abs), "rel_l2": reduce_max(mesh, rel_l2),
        "tolerance": {"max_abs": 2e-2, "rel_l2": 1e-2}, "ok": all_ranks_ok(mesh, ok),
    }


def bench_rpa_mixed(mesh, args, peaks, peak_kind) -> dict:
    """Mixed batch (8 prefill + 120 decode sequences) on one GPU: the whole step, then the decode
    sequences alone and the prefill sequences alone, so that each part can be held against the
    bound that governs it (HBM bandwidth for decode, tensor throughput for prefill)."""
    import torch

    from tpu_cake_b200 import rpa_cuda_lowering, workloads

    config = workloads.MIXED_8_120
    if args.case == "rpa-prefill":
        import dataclasses

        # Small case for profiler captures: the prefill sequences' distributions without the decode
        # sequences (about 0.2 GB of KV pages instead of 8 GB).
        config = dataclasses.replace(config, decode_seqs=0, name=config.name + "-prefill-part")
    meta = workloads.mixed_metadata(config)
    device = mesh.device
    generator = torch.Generator(device=device).manual_seed(2000)
    tokens = meta.num_tokens
    cache = torch.empty((meta.total_pages, config.page_size, config.kv_heads, 2, config.head_dim), dtype=torch.bfloat16, device=device)
    for start in range(0, meta.total_pages, 8192):
        block = cache[start : start + 8192]
        block.copy_(torch.randn(block.shape, generator=generator, device=device))
    q = torch.randn((tokens, config.q_heads, config.head_dim), generator=generator, device=device).to(torch.bfloat16)
    new_k = torch.randn((tokens, config.kv_heads, config.head_dim), generator=generator, device=device).to(torch.bfloat16)
    new_v = torch.randn((tokens, config.kv_heads, config.head_dim), generator=generator, device=device).to(torch.bfloat16)
    out = torch.empty_like(q)
    flush_buffer = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def flush():
        flush_buffer.fill_(1)

    def part(first: int, last: int, decode_end: int):
        """Executable and arguments for sequences [first, last) of the batch."""
        count = last - first
        tok0, tok1 = int(meta.cu_q_lens[first]), int(meta.cu_q_lens[last])
        page0 = int(meta.cu_kv_lens[first]) // config.page_size
        pages = meta.page_indices[page0:]
        plan = rpa_cuda_lowering.CudaMixedRpaPlan(
            name=config.name, schedule_sha256="0" * 64, query_shape=(tok1 - tok0, config.q_heads, config.head_dim),
            key_shape=(tok1 - tok0, config.kv_heads, config.head_dim), fused_cache_shape=tuple(cache.shape), sequences=count,
            page_indices_shape=tuple(pages.shape), softmax_scale=config.softmax_scale, kv_chunk_tokens=args.kv_chunk,
        )
        executable = plan.build(device)
        inputs = (
            q[tok0:tok1], new_k[tok0:tok1], new_v[tok0:tok1], cache, torch.from_numpy(meta.kv_lens[first:last].copy()).to(device),
            torch.from_numpy(pages.copy()).to(device), torch.from_numpy((meta.cu_q_lens[first : last + 1] - tok0).astype(np.int32)).to(device),
            torch.from_numpy((meta.cu_kv_lens[first : last + 1] - meta.cu_kv_lens[first]).astype(np.int32)).to(device),
            np.array([decode_end, count, count], dtype=np.int32), None, None,
        )
        result = out[tok0:tok1]

        def call():
            plan.invoke(executable, *inputs, out=result)

        return executable, call

    decode_count = int(meta.distribution[0])
    total = len(meta.kv_lens)
    steps = max(args.steps, 10)
    timings = {}
    launches = 0
    parts = {"whole": (0, total, decode_count), "decode_only": (0, decode_count, decode_count), "prefill_only": (decode_count, total, 0)}
    if decode_count == 0:
        parts = {"whole": parts["whole"]}
    for label, (first, last, decode_end) in parts.items():
        executable, call = part(first, last, decode_end)
        step = call
        if not args.no_graph:
            call()
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                call()
            step = graph.replay
        total_ms, per_step = timed_steps(mesh, step, steps, max(args.warmup, 3), flush)
        executable.status()
        timings[label] = total_ms / steps
        if label == "whole":
            launches = executable.launches_per_call * steps
        executable.close()
    work = workloads.mixed_algorithmic_work(meta, config.q_heads, config.kv_heads, config.head_dim)
    update_bytes = tokens * config.kv_heads * config.head_dim * 2 * 2 * 2  # new K/V read and written into the cache
    bytes_total = work["bytes"] + update_bytes
    hbm_peak, tensor_peak = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
    bound_hbm_ms = bytes_total / (hbm_peak * 1e9) * 1e3
    bound_tensor_ms = work["prefill_flops"] / (tensor_peak * 1e12) * 1e3
    ms = timings["whole"]
    timings.setdefault("prefill_only", ms)
    decode_ms = timings.get("decode_only")
    return {
        "metric": "rpa_mixed_step_ms", "value": ms, "unit": "ms", "higher_is_better": False, "steps": steps,
        "config": {
            "workload": config.name, "decode_seqs": config.decode_seqs, "prefill_seqs": config.prefill_seqs, "query_tokens": tokens,
            "kv_tokens": int(meta.kv_lens.astype(np.int64).sum()), "q_heads": config.q_heads, "kv_heads": config.kv_heads,
            "head_dim": config.head_dim, "page_size": config.page_size, "total_pages": meta.total_pages, "causal": True,
            "cache_update": True, "l2": "256 MiB flush between steps", "launch": "stream" if args.no_graph else "cuda-graph",
        },
        "hbm_gbs": bytes_total / (ms * 1e-3) / 1e9,
        "attention_tflops": work["flops"] / (ms * 1e-3) / 1e12,
        "roofline": {
            "bound": "hbm (decode sequences) then tensor (prefill sequences): the kernels run one after the other, so the bounds add",
            "bound_ms": bound_hbm_ms + bound_tensor_ms, "hbm_bound_ms": bound_hbm_ms, "tensor_bound_ms": bound_tensor_ms,
            "frac": (bound_hbm_ms + bound_tensor_ms) / ms, "algorithmic_bytes": bytes_total, "prefill_flops": work["prefill_flops"],
            "peak_source": f"{peak_kind}: device copy bandwidth and cuBLAS bf16 burst",
        },
        "parts": {
            "decode_only_ms": decode_ms, "decode_only_gbs": work["decode_bytes"] / (decode_ms * 1e-3) / 1e9 if decode_ms else None,
            "decode_only_frac_of_hbm_peak": work["decode_bytes"] / (decode_ms * 1e-3) / 1e9 / hbm_peak if decode_ms else None,
            "prefill_only_ms": timings["prefill_only"], "prefill_only_tflops": work["prefill_flops"] / (timings["prefill_only"] * 1e-3) / 1e12,
            "prefill_only_frac_of_bf16_peak": work["prefill_flops"] / (timings["prefill_only"] * 1e-3) / 1e12 / tensor_peak,
            "kernel": "cake_rpa_prefill_sm100 (tcgen05, TMEM accumulators) for prefill; cake_rpa_decode_sm100 for decode",
        },
        "gpu_launches": launches,
    }


def run_ours(args) -> None:
    import torch

    __graft_entry__.load_package()
    from tpu_cake_b200 import workloads
    from tpu_cake_b200.mesh import ProcessMesh

    mesh = ProcessMesh.from_environment()
    if mesh.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {mesh.world}: launch with torch.distributed.run")
    peaks, peak_kind = measured_peaks()
    if args.case == "rpa-mixed" or args.case == "rpa-prefill":
        # Small cases for profiler captures (the commands recorded under profiles/).
        if mesh.rank == 0:
            print(json.dumps(bench_rpa_mixed(mesh, args, peaks, peak_kind)), flush=True)
        return
    if args.case == "rpa-decode":
        result = bench_rpa(mesh, args, peaks, peak_kind, workloads.DECODE_64)
        if mesh.rank == 0:
            print(json.dumps(result), flush=True)
        return
    rpa = sharded = mixed = None
    if not args.no_rpa:
        if mesh.world == 1:
            rpa = bench_rpa(mesh, args, peaks, peak_kind, workloads.DECODE_64)
            mixed = None if args.no_mixed else bench_rpa_mixed(mesh, args, peaks, peak_kind)
        sharded = bench_rpa(mesh, args, peaks, peak_kind, workloads.DECODE_SHARDED_256)
        sharded["metric"] = "rpa_decode_sharded_hbm_gbs"
    matmul = bench_matmul(mesh, args, peaks, peak_kind)
    c1 = bench_matmul_c1_latency(mesh) if mesh.world == 8 else None
    line = {
        "metric": "matmul_reduce_scatter_tflops", "value": matmul["value"], "unit": "TFLOP/s", "n_gpus": mesh.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": matmul["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": matmul_config(mesh.world, matmul["strategy"]),
        "roofline": matmul["roofline"], "e2e": matmul["e2e"], "gpu_launches": matmul["gpu_launches"], "clocks": matmul["clocks"],
        "parity": matmul["parity"],
    }
    if matmul["phases"] is not None:
        line["communication"] = matmul["phases"]
    if mesh.rank == 0 and mesh.world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_matmul_sample(args.cpu_rows)
    # "rpa_decode": the 64-sequence decode on one GPU; at N > 1 the sharded 256-sequence decode (the
    # key earlier runs used for it). "rpa_decode_sharded": the 256-sequence decode at every N.
    if sharded is not None:
        line["rpa_decode_sharded"] = sharded
        line["rpa_decode"] = rpa if rpa is not None else sharded
        line["gpu_launches"] += sharded["gpu_launches"] + (rpa["gpu_launches"] if rpa is not None else 0)
    if mixed is not None:
        line["rpa_mixed"] = mixed
        line["gpu_launches"] += mixed["gpu_launches"]
    if c1 is not None:
        line["matmul_c1_latency"] = c1
        line["gpu_launches"] += c1["gpu_launches"]
    ok = line["parity"]["ok"] and all(part is None or part["parity"]["ok"] for part in (rpa, sharded, c1))
    if mesh.rank == 0:
        print(json.dumps(line), flush=True)
    if mesh.world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("PARITY_FAILED: a rank's result disagrees with the oracle (see the parity objects of the line)")


# ------------------------------------------------------------------------------------ reference


def run_reference(args) -> None:
    """The reference's CPU path for the same metric and config. The reference's own JAX program
    cannot run on this machine (jax and xDSL are not installed and cannot be), so this arm times the
    oracle port, which restates the numpy oracle the reference itself checks against, in the form
    the reference's device program has: ``mesh`` split-K partial products summed in rank order and
    sliced along M (src/tpu_cake/pallas_lowering.py:446-464). Each step is a bounded sample of the
    workload (``--cpu-rows`` of the 8192 lhs rows); rank 0 alone runs it, on every host core it may use."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = args.gpus
    rows = max(world, args.cpu_rows // world * world)
    from oracle import matmul_rs

    generator = np.random.default_rng(0)
    lhs = matmul_rs.quantize_bf16(generator.normal(scale=K**-0.5, size=(rows, K)).astype(np.float32))
    rhs = matmul_rs.quantize_bf16(generator.normal(scale=K**-0.5, size=(K, N)).astype(np.float32))

    def step():
        return matmul_rs.matmul_reduce_scatter(lhs, rhs, world=world, scatter_dimension=0, transport_dtype="f32", out_dtype="bf16")

    with blas_threads() as pool:
        for _ in range(args.warmup):
            step()
        started = time.perf_counter()
        for _ in range(args.steps):
            step()
        elapsed = time.perf_counter() - started
    value = 2.0 * rows * K * N * args.steps / elapsed / 1e12
    sample = (f"{rows} of {M} lhs rows of the {M}x{K}x{N} product per step: {world} split-K partial products (numpy float32 "
              f"matmul on bf16-valued inputs), summed in rank order, sliced along M, rounded to bf16")
    baseline = {"value": value, "unit": "TFLOP/s", "cores": pool.used, "threads_used": pool.used, "host_cores": host_threads(),
                "kind": "port", "sample": sample}
    line = {
        "impl": "reference", "metric": "matmul_reduce_scatter_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": matmul_config(world, "p2p_bf16" if world > 1 else "single"),
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_rpa:
        # The attention objects' CPU side: the numpy oracle on a bounded sample of each configuration.
        __graft_entry__.load_package()
        from tpu_cake_b200 import workloads

        for key, config, sequences in (("rpa_decode", workloads.DECODE_64, 32), ("rpa_decode_sharded", workloads.DECODE_SHARDED_256, 8)):
            lengths, table = workloads.decode_metadata(config)
            sampled = cpu_rpa_sample(lengths, table, config, sequences)
            line[key] = {"metric": "rpa_decode_hbm_gbs" if key == "rpa_decode" else "rpa_decode_sharded_hbm_gbs",
                         "value": sampled["value"], "unit": "GB/s", "config": {"workload": config.name}, "cpu_baseline": sampled}
    print(json.dumps(line), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--strategy", choices=("p2p_bf16", "p2p_f32", "nccl"), default="p2p_bf16")
    parser.add_argument("--kv-chunk", type=int, default=0)
    parser.add_argument("--cpu-rows", type=int, default=8192, help="lhs rows of the CPU legs' sample (the whole product by default)")
    parser.add_argument("--no-rpa", action="store_true")
    parser.add_argument("--rpa-gather", choices=("p2p", "nccl"), default="p2p", help="how the sharded decode's outputs are all-gathered")
    parser.add_argument("--no-graph", action="store_true", help="launch the attention step kernel by kernel instead of replaying a CUDA graph")
    parser.add_argument("--no-mixed", action="store_true", help="skip the mixed prefill/decode batch")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--case", choices=("all", "rpa-decode", "rpa-mixed", "rpa-prefill"), default="all",
                        help="one part of the bench alone, sized for a profiler capture: rpa-decode = the 64-sequence decode "
                             "(with --rpa-pool-pages to shrink the page pool), rpa-mixed = the mixed batch, rpa-prefill = its "
                             "prefill sequences on a small pool")
    parser.add_argument("--rpa-pool-pages", type=int, default=0,
                        help="with --case rpa-decode: shrink the KV page pool (same sequences and lengths)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
