"""Static resource report of any physical kernel of this backend's dialect subset, for target ``b200``.

Counterpart of ``analyze_physical_kernel`` (src/tpu_cake/physical_cost_model.py:774): it walks the
operations of one ``tpu_schedule.kernel`` as declared -- nothing is executed -- and reports the MXU
regions with their tile grids (:73-114), the memory ledger (external HBM footprints, explicit DMA
bytes, allocated and peak live on-chip bytes, :131-149), the collectives with the reference's
payload and ring-equivalent bytes (:587-611), per-stage activity (:198-211), capacity peaks
(:214-227) and priced time floors with the limiting resource (:313-320).

Differences that the target forces: NVSwitch gives every GPU its full link rate to every peer, so
besides the ring-equivalent figure a collective carries ``switch_egress_bytes_per_device`` (what one
GPU sends: ``payload * (g - 1) / g``), which is what the ICI floor prices; and the ragged paged
attention ops, which the reference's model refuses for want of a work convention (:800-812), are
priced with this backend's convention at the capacity the declared buffers allow (every page-table
slot full), flagged as an upper bound. Vector / pipeline-loop schedules (the Seqax kernels) are not
in this dialect subset.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from decimal import Decimal

from .cost_model import B200_MEASURED, HardwareRateModel
from .ir import BufferType, Module, Operation, schedule_sha256

SCHEMA = "physical-kernel-resource-b200-v1"
_RPA_OPS = ("tpu_schedule.ragged_paged_attention", "tpu_schedule.fused_ragged_paged_attention")


class UnsupportedPhysicalCostModelError(ValueError):
    """The kernel holds an operation the model has no work convention for."""


@dataclass(frozen=True)
class PhysicalMxuRegion:
    region_index: int
    operation: str
    input_dtype: str
    stage: int
    m: int
    k: int
    n: int
    tile_m: int
    tile_k: int
    tile_n: int
    grid: tuple[int, int, int]
    tile_programs: int
    flops: int
    accumulator_bytes: int


@dataclass(frozen=True)
class PhysicalMemoryLedger:
    external_hbm_input_footprint_bytes_per_device: int
    external_hbm_output_footprint_bytes_per_device: int
    explicit_hbm_dma_read_bytes_per_device: int
    explicit_hbm_dma_write_bytes_per_device: int
    allocated_vmem_bytes_per_device: int
    allocated_smem_bytes_per_device: int
    peak_live_vmem_bytes_per_device: int
    peak_live_vmem_stage: int
    peak_live_smem_bytes_per_device: int
    peak_live_smem_stage: int


@dataclass(frozen=True)
class PhysicalCollectiveTraffic:
    kind: str
    stage: int
    mesh_axis: str
    group_size: int
    implementation: str | None
    payload_bytes_per_device: int
    ring_equivalent_bidirectional_bytes_per_device: Decimal
    switch_egress_bytes_per_device: Decimal
    link_bandwidth_bytes_per_second: int


@dataclass(frozen=True)
class PhysicalAttentionWork:
    operation: str
    stage: int
    sequences: int
    q_heads: int
    kv_heads: int
    head_dim: int
    token_capacity: int
    hbm_bytes_upper_bound: int
    flops_upper_bound: int


@dataclass(frozen=True)
class PhysicalStageRecord:
    stage: int
    operations: tuple[str, ...]
    active_dma: int
    active_mxu: int
    active_ici: int
    active_attention: int
    live_vmem_bytes_per_device: int
    live_smem_bytes_per_device: int


@dataclass(frozen=True)
class PhysicalResourcePeak:
    resource: str
    observed: int
    capacity: int
    stage: int


@dataclass(frozen=True)
class PhysicalKernelResourceReport:
    schema_version: str
    physical_schedule_sha256: str
    kernel_name: str
    target: str
    topology_authority: str
    mesh_axes: tuple[tuple[str, int], ...]
    device_count: int
    canonical_operation_inventory: tuple[tuple[str, int], ...]
    hardware: HardwareRateModel
    mxu_regions: tuple[PhysicalMxuRegion, ...]
    memory: PhysicalMemoryLedger
    collectives: tuple[PhysicalCollectiveTraffic, ...]
    attention: tuple[PhysicalAttentionWork, ...]
    stages: tuple[PhysicalStageRecord, ...]
    resource_peaks: tuple[PhysicalResourcePeak, ...]
    priced_compute_time_floor_ns: Decimal
    priced_hbm_time_floor_ns: Decimal
    priced_ici_time_floor_ns: Decimal
    collective_ring_equivalent_time_scenario_ns: Decimal
    priced_overlapped_resource_scenario_ns: Decimal
    priced_serial_resource_scenario_ns: Decimal
    predicted_limiting_priced_resource: str
    assumptions: tuple[str, ...] = field(default_factory=tuple)
    omissions: tuple[str, ...] = field(default_factory=tuple)

    def to_json(self) -> dict:
        def plain(value):
            if isinstance(value, Decimal):
                return str(value)
            if isinstance(value, dict):
                return {k: plain(v) for k, v in value.items()}
            if isinstance(value, (list, tuple)):
                return [plain(v) for v in value]
            return value

        return plain(asdict(self))


def _buffer(op: Operation, index: int) -> BufferType:
    type_ = op.operands[index].type
    if not isinstance(type_, BufferType):
        raise UnsupportedPhysicalCostModelError(f"{op.name}: operand {index} is not a buffer")
    return type_


def _live_bytes(buffers: list[BufferType], space: str, stage: int) -> int:
    return sum(b.nbytes() for b in buffers if b.memory == space and b.lifetime[0] <= stage <= b.lifetime[1])


def _collective(op: Operation, topology: dict[str, int], hardware: HardwareRateModel) -> PhysicalCollectiveTraffic:
    source, destination = _buffer(op, 0), _buffer(op, 1)
    kind, group = op.properties["kind"], int(op.properties["group_size"])
    if kind == "reduce_scatter":
        payload = source.nbytes()
    elif kind == "all_gather":
        payload = destination.nbytes()
    else:
        raise UnsupportedPhysicalCostModelError(f"unsupported collective kind {kind}")
    implementation = op.properties.get("implementation")
    # What one GPU sends through the switch; the bf16 owner-push halves the f32 partial's bytes.
    egress = Decimal(payload * (group - 1)) / Decimal(group)
    if implementation == "p2p_owner_push_bf16":
        egress /= 2
    axis = op.properties["mesh_axis"]
    return PhysicalCollectiveTraffic(
        kind=kind, stage=int(op.properties["stage"]), mesh_axis=axis, group_size=group, implementation=implementation,
        payload_bytes_per_device=payload, ring_equivalent_bidirectional_bytes_per_device=Decimal(2 * payload * (group - 1)) / Decimal(group),
        switch_egress_bytes_per_device=egress, link_bandwidth_bytes_per_second=min(topology.get(axis, hardware.ici_bytes_per_second), hardware.ici_bytes_per_second),
    )


def _attention(op: Operation) -> PhysicalAttentionWork:
    """Capacity pricing of a decode attention op: every page-table slot of every sequence holds
    a full page; bytes and FLOPs by ``cost_model.estimate_rpa_decode``'s convention."""
    query = _buffer(op, 0)
    if op.name == "tpu_schedule.ragged_paged_attention":
        cache, table = _buffer(op, 1), _buffer(op, 3)
        page_size, kv_heads = cache.shape[1], cache.shape[2]
        token_capacity = table.shape[0] * table.shape[1] * page_size
        pages = table.shape[0] * table.shape[1]
    else:
        cache, indices = _buffer(op, 3), _buffer(op, 5)
        page_size, kv_heads = cache.shape[1], cache.shape[2] * cache.shape[3] // 2
        token_capacity = min(indices.shape[0], cache.shape[0]) * page_size
        pages = min(indices.shape[0], cache.shape[0])
    sequences, q_heads, head_dim = query.shape
    element = 2
    kv_bytes = token_capacity * kv_heads * head_dim * element * 2
    return PhysicalAttentionWork(
        operation=op.name, stage=int(op.properties["stage"]), sequences=sequences, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
        token_capacity=token_capacity, hbm_bytes_upper_bound=kv_bytes + sequences * q_heads * head_dim * element * 2 + pages * 4 + 8 * sequences,
        flops_upper_bound=4 * head_dim * q_heads * token_capacity,
    )


def analyze_physical_kernel(module: Module, *, hardware: HardwareRateModel = B200_MEASURED) -> PhysicalKernelResourceReport:
    """Static report of the module's single physical kernel. Raises
    ``UnsupportedPhysicalCostModelError`` for operations outside the dialect subset."""
    module.verify()
    kernels = [op for op in module.ops if op.name == "tpu_schedule.kernel"]
    if len(kernels) != 1:
        raise UnsupportedPhysicalCostModelError("the module must hold exactly one tpu_schedule.kernel")
    kernel = kernels[0]
    properties = kernel.properties
    mesh_axes = tuple(zip(properties["mesh_axis_names"], properties["mesh_axis_sizes"], strict=True))
    topology = {entry.split(":")[0]: int(entry.split(":")[1]) for entry in properties["topology"]}
    device_count = 1
    for _, size in mesh_axes:
        device_count *= size

    inventory: dict[str, int] = {}
    locals_: list[BufferType] = []
    regions: list[PhysicalMxuRegion] = []
    collectives: list[PhysicalCollectiveTraffic] = []
    attention: list[PhysicalAttentionWork] = []
    dma_read = dma_write = 0
    by_stage: dict[int, list[Operation]] = {}
    for op in kernel.body.ops:
        inventory[op.name] = inventory.get(op.name, 0) + 1
        stage = op.properties.get("stage")
        if stage is not None:
            by_stage.setdefault(int(stage), []).append(op)
        if op.name == "tpu_schedule.alloc":
            locals_.append(op.result.type)
        elif op.name == "tpu_schedule.dma_start":
            source, destination = _buffer(op, 0), _buffer(op, 1)
            if source.memory == "hbm":
                dma_read += source.nbytes()
            if destination.memory == "hbm":
                dma_write += destination.nbytes()
        elif op.name == "tpu_schedule.mxu_matmul":
            lhs, rhs, accumulator = _buffer(op, 0), _buffer(op, 1), _buffer(op, 2)
            m, k = lhs.shape
            n = rhs.shape[1]
            tile_m, tile_k, tile_n = (int(op.properties[name]) for name in ("tile_m", "tile_k", "tile_n"))
            grid = (m // tile_m, n // tile_n, k // tile_k)
            regions.append(PhysicalMxuRegion(
                region_index=len(regions), operation=op.name, input_dtype=lhs.element_type, stage=int(op.properties["stage"]), m=m, k=k, n=n,
                tile_m=tile_m, tile_k=tile_k, tile_n=tile_n, grid=grid, tile_programs=grid[0] * grid[1] * grid[2], flops=2 * m * k * n,
                accumulator_bytes=accumulator.nbytes()))
        elif op.name == "tpu_schedule.collective":
            collectives.append(_collective(op, topology, hardware))
        elif op.name in _RPA_OPS:
            attention.append(_attention(op))
        elif op.name not in ("tpu_schedule.semaphore_alloc", "tpu_schedule.dma_wait", "tpu_schedule.yield", "tpu_schedule.cuda_rpa_decode"):
            raise UnsupportedPhysicalCostModelError(f"no work convention for {op.name}")

    external = [value.type for value in kernel.body.args if isinstance(value.type, BufferType)]
    written = {id(op.operands[1]) for op in kernel.body.ops if op.name == "tpu_schedule.dma_start"}
    outputs_footprint = sum(value.type.nbytes() for value in kernel.body.args if isinstance(value.type, BufferType) and id(value) in written)
    last_stage = max(by_stage) if by_stage else 0
    live = {space: [(_live_bytes(locals_, space, stage), stage) for stage in range(last_stage + 1)] for space in ("vmem", "smem")}
    peak_vmem, peak_vmem_stage = max(live["vmem"], default=(0, 0))
    peak_smem, peak_smem_stage = max(live["smem"], default=(0, 0))
    memory = PhysicalMemoryLedger(
        external_hbm_input_footprint_bytes_per_device=sum(b.nbytes() for b in external) - outputs_footprint,
        external_hbm_output_footprint_bytes_per_device=outputs_footprint,
        explicit_hbm_dma_read_bytes_per_device=dma_read, explicit_hbm_dma_write_bytes_per_device=dma_write,
        allocated_vmem_bytes_per_device=sum(b.nbytes() for b in locals_ if b.memory == "vmem"),
        allocated_smem_bytes_per_device=sum(b.nbytes() for b in locals_ if b.memory == "smem"),
        peak_live_vmem_bytes_per_device=peak_vmem, peak_live_vmem_stage=peak_vmem_stage,
        peak_live_smem_bytes_per_device=peak_smem, peak_live_smem_stage=peak_smem_stage,
    )
    stages = tuple(
        PhysicalStageRecord(
            stage=stage, operations=tuple(op.name for op in ops),
            active_dma=sum(op.name in ("tpu_schedule.dma_start", "tpu_schedule.dma_wait") for op in ops),
            active_mxu=sum(op.name == "tpu_schedule.mxu_matmul" for op in ops),
            active_ici=sum(op.name == "tpu_schedule.collective" for op in ops),
            active_attention=sum(op.name in _RPA_OPS for op in ops),
            live_vmem_bytes_per_device=_live_bytes(locals_, "vmem", stage), live_smem_bytes_per_device=_live_bytes(locals_, "smem", stage))
        for stage, ops in sorted(by_stage.items()))
    peaks = (
        PhysicalResourcePeak("vmem_bytes", peak_vmem, int(properties["vmem_capacity_bytes"]), peak_vmem_stage),
        PhysicalResourcePeak("smem_bytes", peak_smem, int(properties["smem_capacity_bytes"]), peak_smem_stage),
    )
    for peak in peaks:
        if peak.observed > peak.capacity:
            raise ValueError("PHYSICAL_RESOURCE_CAPACITY_EXCEEDED")

    billion = Decimal(1_000_000_000)
    flops = sum(r.flops for r in regions) + sum(a.flops_upper_bound for a in attention)
    hbm_bytes = dma_read + dma_write + sum(a.hbm_bytes_upper_bound for a in attention)
    compute_ns = Decimal(flops) * billion / Decimal(hardware.compute_flops_per_second)
    hbm_ns = Decimal(hbm_bytes) * billion / Decimal(hardware.hbm_bytes_per_second)
    ici_ns = sum((c.switch_egress_bytes_per_device * billion / Decimal(c.link_bandwidth_bytes_per_second) for c in collectives), Decimal(0))
    ring_ns = sum((c.ring_equivalent_bidirectional_bytes_per_device * billion / Decimal(2 * c.link_bandwidth_bytes_per_second) for c in collectives), Decimal(0))
    floors = (("compute", compute_ns), ("hbm", hbm_ns), ("ici", ici_ns))
    limiting = max(floors, key=lambda kv: kv[1])
    assumptions = ["rates are the measured B200 copy bandwidth and cuBLAS bf16 burst throughput, and the nominal NVLink 5 rate per direction",
                   "a collective is priced by what one GPU sends through the switch, every peer at full rate"]
    if attention:
        assumptions.append("attention is priced at the capacity of its declared page table: an upper bound on bytes and FLOPs")
    return PhysicalKernelResourceReport(
        schema_version=SCHEMA, physical_schedule_sha256=schedule_sha256(module), kernel_name=properties["sym_name"], target=properties["target"],
        topology_authority=properties["topology_authority"], mesh_axes=mesh_axes, device_count=device_count,
        canonical_operation_inventory=tuple(sorted(inventory.items())), hardware=hardware, mxu_regions=tuple(regions), memory=memory,
        collectives=tuple(collectives), attention=tuple(attention), stages=stages, resource_peaks=peaks,
        priced_compute_time_floor_ns=compute_ns, priced_hbm_time_floor_ns=hbm_ns, priced_ici_time_floor_ns=ici_ns,
        collective_ring_equivalent_time_scenario_ns=ring_ns, priced_overlapped_resource_scenario_ns=limiting[1],
        priced_serial_resource_scenario_ns=sum(v for _, v in floors),
        predicted_limiting_priced_resource=limiting[0] if limiting[1] > 0 else "none",
        assumptions=tuple(assumptions),
        omissions=("launch latency and kernel tails", "L2 re-reads of operand tiles", "vector / pipeline-loop work: not in this dialect subset"),
    )
