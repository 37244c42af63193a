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
    if mesh.world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 1 if failures else 0


if __name__ == "__main__":
    raise SystemExit(main())
