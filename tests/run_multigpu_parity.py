"""Multi-GPU parity of the matmul + reduce-scatter strategies, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port 29533 tests/run_multigpu_parity.py

Not collected by pytest (the GPU test tier runs on one GPU, where all ranks are emulated on that
GPU instead, tests/test_gpu_matmul.py). Every rank checks its own local output against the CPU
oracle and rank 0 prints one line per case; the exit code is non-zero if any rank saw a mismatch.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import __graft_entry__  # noqa: E402

__graft_entry__.load_package()

from oracle import matmul_rs as oracle  # noqa: E402
from tests.helpers import bf16_to_torch  # noqa: E402
from tpu_cake_b200 import cuda_lowering, workloads  # noqa: E402
from tpu_cake_b200.mesh import ProcessMesh  # noqa: E402

STRATEGIES = {
    "nccl_reduce_scatter": ("f32", cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER),
    "p2p_fused_epilogue": ("f32", cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE),
    "p2p_fused_epilogue_bf16_transport": ("bf16", cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT),
}


def main() -> int:
    mesh = ProcessMesh.from_environment()
    failures = 0
    cases = [(128, 1024, 1024, 128), (1024, 4096, 2048, 256)]
    for m, k, n, tile_n in cases:
        lhs, rhs = workloads.distributed_matmul_inputs(mesh.world, m, k, n, scale=1.0 if m == 128 else k**-0.5)
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, mesh.world, mesh.rank)
        lhs_d, rhs_d = bf16_to_torch(lhs_r, mesh.device), bf16_to_torch(rhs_r, mesh.device)
        lhs32, rhs32 = lhs.astype(np.float32), rhs.astype(np.float32)
        for scatter_dimension in (0, 1):
            for name, (transport, strategy) in STRATEGIES.items():
                for output_dtype in ("f32", "bf16"):
                    plan = cuda_lowering.plan_distributed_matmul(
                        mesh_size=mesh.world, m=m, k=k, n=n, scatter_dimension=scatter_dimension,
                        output_dtype=output_dtype, tile_n=tile_n, collective_implementation=strategy,
                    )
                    executable, _ = plan.build(mesh=mesh)
                    mesh.barrier()
                    outputs = []
                    for _ in range(3):
                        outputs.append(executable(lhs_d, rhs_d).float().cpu().numpy())
                    if name != "nccl_reduce_scatter":
                        executable.status()
                    expected = oracle.matmul_reduce_scatter(
                        lhs32, rhs32, world=mesh.world, scatter_dimension=scatter_dimension,
                        transport_dtype=transport, out_dtype=output_dtype,
                    )[mesh.rank]
                    if transport == "f32" and output_dtype == "f32":
                        ok = bool(np.allclose(outputs[0], expected, atol=1e-3, rtol=1e-3))
                    else:
                        ok = oracle.relative_l2_error(outputs[0], expected) < 4e-3
                    if name != "nccl_reduce_scatter":
                        ok = ok and all(np.array_equal(outputs[0], later) for later in outputs[1:])
                    flag = torch.tensor([0 if ok else 1], device=mesh.device)
                    if mesh.world > 1:
                        import torch.distributed as dist

                        dist.all_reduce(flag, group=mesh.group)
                    failures += int(flag.item())
                    if mesh.rank == 0:
                        print(
                            f"{'PASS' if flag.item() == 0 else 'FAIL'} {m}x{k}x{n} W={mesh.world} scatter={scatter_dimension} "
                            f"{name} out={output_dtype} rel_l2={oracle.relative_l2_error(outputs[0], expected):.2e}",
                            flush=True,
                        )
                    executable.close()
    failures += sharded_decode_case(mesh)
    if mesh.world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 1 if failures else 0


def sharded_decode_case(mesh) -> int:
    """Decode with KV heads sharded over the ranks and the outputs all-gathered through peer memory:
    every rank checks the whole gathered result against the oracle, three calls in a row."""
    import math

    from oracle import rpa as rpa_oracle
    from tests.helpers import BF16, to_device, torch_to_bf16
    from tpu_cake_b200 import rpa_cuda_lowering
    from tpu_cake_b200.mesh import SymmetricBuffer

    world = mesh.world
    generator = np.random.default_rng(77)
    lengths = np.array([33, 900, 1700, 512, 64, 2049], dtype=np.int32)
    count, kv_heads, group, page_size = len(lengths), 8, 4, 32
    q_heads = kv_heads * group
    pages_per = -(-lengths.astype(np.int64) // page_size)
    pool = int(pages_per.sum()) + 5
    query = generator.normal(size=(count, q_heads, 128)).astype(np.float32).astype(BF16)
    keys = generator.normal(size=(pool, page_size, kv_heads, 128)).astype(np.float32).astype(BF16)
    values = generator.normal(size=(pool, page_size, kv_heads, 128)).astype(np.float32).astype(BF16)
    table = np.zeros((count, int(pages_per.max())), dtype=np.int32)
    permutation = generator.permutation(pool)
    cursor = 0
    for s in range(count):
        table[s, : pages_per[s]] = permutation[cursor : cursor + pages_per[s]]
        cursor += int(pages_per[s])
    expected = rpa_oracle.rpa_separate(query, keys, values, table, lengths, None, scale=1.0 / math.sqrt(128))
    local_kv, local_q = kv_heads // world, q_heads // world
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name="sharded", schedule_sha256="0" * 64, query_shape=(count, local_q, 128), cache_shape=(pool, page_size, local_kv, 128),
        page_table_shape=table.shape, bias_shape=None, softmax_scale=1.0 / math.sqrt(128), cache_layout="fused",
    )
    executable = plan.build(mesh.device)
    heads = slice(mesh.rank * local_kv, (mesh.rank + 1) * local_kv)
    cache = to_device(rpa_oracle.fused_cache_from_separate(keys[:, :, heads], values[:, :, heads]), mesh.device)
    q_local = to_device(np.ascontiguousarray(query[:, mesh.rank * local_q : (mesh.rank + 1) * local_q]), mesh.device)
    gathered = SymmetricBuffer(mesh, 2 * world * count * local_q * 128 * 2)
    flags = SymmetricBuffer(mesh, 64)
    table_d, lengths_d = to_device(table, mesh.device), to_device(lengths, mesh.device)
    view = gathered.as_tensor(torch.bfloat16, (2, world, count, local_q, 128))
    # Three calls back to back with no host barrier between them, each followed on the stream by its
    # consumer (a copy of the half it filled): the halves alternate, so a rank that is already in
    # the next call cannot disturb a peer's consumer of this one. Queries differ per call (scaled),
    # so a stale or overwritten half would not pass.
    factors = (1.0, -1.0, 0.5)
    snapshots = []
    for factor in factors:
        half = executable.enqueue_allgather((q_local.float() * factor).to(torch.bfloat16), cache, None, lengths_d, table_d,
                                            gathered.pointers, flags.pointers, world, mesh.rank)
        snapshots.append(view[half].clone())
    executable.status()
    ok = True
    for factor, snapshot in zip(factors, snapshots):
        full = torch_to_bf16(snapshot).astype(np.float32)
        assembled = np.concatenate([full[r] for r in range(world)], axis=1)
        wanted = rpa_oracle.rpa_separate((query.astype(np.float32) * factor).astype(BF16), keys, values, table, lengths, None,
                                         scale=1.0 / math.sqrt(128))
        ok = ok and oracle.max_abs_error(assembled, wanted) <= 2e-2 and oracle.relative_l2_error(assembled, wanted) <= 1e-2
    mesh.barrier()
    flag = torch.tensor([0 if ok else 1], device=mesh.device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(flag, group=mesh.group)
    if mesh.rank == 0:
        print(f"{'PASS' if flag.item() == 0 else 'FAIL'} sharded decode W={world} with peer-to-peer all-gather", flush=True)
    executable.close()
    gathered.close()
    flags.close()
    return int(flag.item())


if __name__ == "__main__":
    raise SystemExit(main())
