"""Algorithmic cost of the two hot-path kernels on B200.

``estimate_distributed_matmul`` keeps the reference's counting convention for the unfused program
(src/tpu_cake/cost_model.py:127-180: the f32 partial is written to and re-read from HBM between the
contraction and the collective, link bytes are ``2 * partial * (W-1)/W`` "bidirectional"), so its
integers reproduce the reference's known-answer test, and adds the counts of what the CUDA backend
actually does (fused epilogue: no partial round trip; link egress in the transport dtype). The
reference's physical cost model refuses all three RPA ops (src/tpu_cake/physical_cost_model.py:800-812);
``estimate_rpa_decode`` is the byte / FLOP convention this backend reports against.
"""

from __future__ import annotations

from dataclasses import dataclass
from decimal import Decimal

from .cuda_lowering import CudaMatmulRsPlan, MatmulCollectiveStrategy


@dataclass(frozen=True)
class HardwareRateModel:
    name: str
    compute_flops_per_second: int
    hbm_bytes_per_second: int
    ici_bytes_per_second: int  # per direction per device


# Denominators measured on B200 (device copy bandwidth, cuBLAS bf16 burst throughput) and the nominal
# NVLink 5 rate per direction; the reference's TPU7x model is 1153.5 TFLOP/s, 3690 GB/s, 600 GB/s
# (src/tpu_cake/cost_model.py:95-106).
B200_MEASURED = HardwareRateModel("b200-measured", 1_628_900_000_000_000, 6_459_000_000_000, 900_000_000_000)


@dataclass(frozen=True)
class MatmulPhysicalCounts:
    operations_per_device: int
    hbm_read_bytes_per_device: int
    hbm_write_bytes_per_device: int
    ici_bidirectional_bytes_per_device: int
    fused_hbm_read_bytes_per_device: int
    fused_hbm_write_bytes_per_device: int
    link_egress_bytes_per_device: int
    receive_slot_bytes_per_device: int


@dataclass(frozen=True)
class CostModelReport:
    counts: MatmulPhysicalCounts
    compute_ns: Decimal
    memory_ns: Decimal
    communication_ns: Decimal
    lower_bound_ns: Decimal
    serial_ns: Decimal
    limiting_resource: str


def matmul_counts(plan: CudaMatmulRsPlan) -> MatmulPhysicalCounts:
    m, local_k = plan.lhs_local_shape
    _, n = plan.rhs_local_shape
    output_elements = plan.output_local_shape[0] * plan.output_local_shape[1]
    partial_bytes = 4 * plan.partial_local_shape[0] * plan.partial_local_shape[1]
    operand_bytes = 2 * (m * local_k + local_k * n)
    out_size = 4 if plan.output_dtype == "f32" else 2
    resources = plan.collective_resources
    peer_to_peer = plan.mesh_size > 1 and plan.collective_implementation is not MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER
    return MatmulPhysicalCounts(
        operations_per_device=2 * m * local_k * n,
        hbm_read_bytes_per_device=operand_bytes + partial_bytes,
        hbm_write_bytes_per_device=partial_bytes + 4 * output_elements,
        ici_bidirectional_bytes_per_device=2 * partial_bytes * (plan.mesh_size - 1) // plan.mesh_size,
        fused_hbm_read_bytes_per_device=operand_bytes + (resources.reduce_read_bytes if peer_to_peer else 0),
        fused_hbm_write_bytes_per_device=out_size * output_elements + (resources.reduce_read_bytes // plan.mesh_size if peer_to_peer else 0),
        link_egress_bytes_per_device=resources.remote_payload_bytes if peer_to_peer else partial_bytes * (plan.mesh_size - 1) // plan.mesh_size,
        receive_slot_bytes_per_device=resources.receive_slot_bytes,
    )


def estimate_distributed_matmul(plan: CudaMatmulRsPlan, *, hardware: HardwareRateModel = B200_MEASURED) -> CostModelReport:
    counts = matmul_counts(plan)
    billion = Decimal(1_000_000_000)
    compute_ns = Decimal(counts.operations_per_device) * billion / Decimal(hardware.compute_flops_per_second)
    memory_ns = Decimal(counts.fused_hbm_read_bytes_per_device + counts.fused_hbm_write_bytes_per_device) * billion / Decimal(hardware.hbm_bytes_per_second)
    bandwidth = hardware.ici_bytes_per_second
    if plan.collective_link_bandwidths:
        bandwidth = min(bandwidth, min(b for _, b in plan.collective_link_bandwidths))
    communication_ns = Decimal(counts.link_egress_bytes_per_device) * billion / Decimal(bandwidth)
    floors = (("compute", compute_ns), ("hbm", memory_ns), ("ici", communication_ns))
    return CostModelReport(
        counts=counts, compute_ns=compute_ns, memory_ns=memory_ns, communication_ns=communication_ns,
        lower_bound_ns=max(v for _, v in floors), serial_ns=sum(v for _, v in floors),
        limiting_resource=max(floors, key=lambda kv: kv[1])[0],
    )


@dataclass(frozen=True)
class RpaDecodeCounts:
    kv_bytes: int
    query_and_output_bytes: int
    metadata_bytes: int
    flops: int

    @property
    def hbm_bytes(self) -> int:
        return self.kv_bytes + self.query_and_output_bytes + self.metadata_bytes


def estimate_rpa_decode(kv_lens, *, q_heads: int, kv_heads: int, head_dim: int, page_size: int, elem_bytes: int = 2) -> RpaDecodeCounts:
    """Valid K and V tokens once per KV head, the query read and the output write, one table entry
    per page and one length per sequence; FLOPs = 4 * head_dim * q_heads per valid token."""
    total_tokens = int(sum(int(v) for v in kv_lens))
    pages = int(sum(-(-int(v) // page_size) for v in kv_lens))
    count = len(kv_lens)
    return RpaDecodeCounts(
        kv_bytes=total_tokens * kv_heads * head_dim * elem_bytes * 2,
        query_and_output_bytes=count * q_heads * head_dim * elem_bytes * 2,
        metadata_bytes=pages * 4 + 8 * count,
        flops=4 * head_dim * q_heads * total_tokens,
    )
