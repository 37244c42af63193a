"""Mid-level lowering: logical distributed matmul program -> physical kernel for a target.

Same entry point and result as the reference's ``lower_distributed_matmul``
(src/tpu_cake/lowering.py:77-269): it accepts exactly ``einsum_local -> reduce_scatter -> return``
on rank-2 ``lhs[M,K]`` / ``rhs[K,N]`` bf16 inputs with f32 accumulation and emits the 16-operation
physical kernel (4 allocs, 3 semaphores, 2 loads, matmul, collective, store) whose shape the
backend pattern-matches.

Target semantics for ``b200``: the schedule's ``vmem`` space is the device-resident staging of one
rank's local operands and partial (HBM backed by the 126 MB L2), so its capacity is a share of the
180 GB of HBM; the real on-chip tiling (shared-memory ring of 128 x 64 / 64 x BN tiles, TMEM
accumulators) is a property of the CUDA plan, not of the schedule, because the dialect's
``mxu_matmul`` requires ``tile_k`` to equal the whole local contraction extent.
"""

from __future__ import annotations

from dataclasses import dataclass

from .dialects import CollectiveImplementation, KernelBuilder, buffer, program_mesh
from .ir import DTensorType, Module, Operation


class UnsupportedLoweringError(ValueError):
    pass


@dataclass(frozen=True)
class LoweringTarget:
    name: str
    vmem_capacity_bytes: int
    smem_capacity_bytes: int
    ici_bandwidth_bytes_per_second: int

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("lowering target needs a name")
        if min(self.vmem_capacity_bytes, self.smem_capacity_bytes, self.ici_bandwidth_bytes_per_second) <= 0:
            raise ValueError("lowering target memory and interconnect capacities must be positive")


B200_TARGET = LoweringTarget(
    name="b200",
    vmem_capacity_bytes=160 << 30,  # device-resident staging (see module docstring)
    smem_capacity_bytes=227 << 10,  # shared memory one CTA can own
    ici_bandwidth_bytes_per_second=900_000_000_000,  # NVLink 5, one direction, any peer through NVSwitch
)


@dataclass(frozen=True)
class MatmulTile:
    m: int
    n: int

    def __post_init__(self) -> None:
        if self.m <= 0 or self.n <= 0:
            raise ValueError("matmul tile dimensions must be positive")


def _reject(operation: Operation | None, message: str) -> UnsupportedLoweringError:
    if operation is None:
        return UnsupportedLoweringError(message)
    return UnsupportedLoweringError(f"{message}: {operation.name} at {operation.location}")


def _local_shape(tensor: DTensorType, mesh: dict[str, int]) -> tuple[int, ...]:
    shape = []
    for (_, size), axes in zip(tensor.logical_shape(), tensor.sharding_axes(), strict=True):
        divisor = 1
        for axis in axes:
            divisor *= mesh[axis]
        shape.append(size // divisor)
    return tuple(shape)


def lower_distributed_matmul(
    module: Module,
    *,
    target: LoweringTarget = B200_TARGET,
    tile: MatmulTile | None = None,
    collective_implementation: CollectiveImplementation | None = None,
) -> Module:
    module.verify()
    if len(module.ops) != 1 or module.ops[0].name != "dtensor.program":
        raise _reject(module.ops[0] if module.ops else None, "expected one distributed program")
    program = module.ops[0]
    operations = list(program.body.ops)
    allowed = ("dtensor.einsum_local", "dtensor.reduce_scatter", "dtensor.return")
    if len(operations) != 3:
        unexpected = next((op for op in operations if op.name not in allowed), program)
        raise _reject(unexpected, "only einsum, reduce-scatter, and return are supported")
    einsum, collective, terminator = operations
    if einsum.name != "dtensor.einsum_local":
        raise _reject(einsum, "the first operation must be a local einsum")
    if collective.name != "dtensor.reduce_scatter":
        raise _reject(collective, "the second operation must be a reduce-scatter")
    if terminator.name != "dtensor.return":
        raise _reject(terminator, "the final operation must be a return")
    if collective.operands[0].owner is not einsum:
        raise _reject(collective, "reduce-scatter must consume the einsum result")
    if len(terminator.operands) != 1 or terminator.operands[0].owner is not collective:
        raise _reject(terminator, "the program must return the reduce-scatter result")
    if len(program.body.args) != 2:
        raise _reject(program, "distributed matmul needs exactly two inputs")
    lhs_type, rhs_type = (value.type for value in program.body.args)
    partial_type, result_type = einsum.result.type, collective.result.type
    if lhs_type.element_type != "bf16" or rhs_type.element_type != "bf16":
        raise _reject(einsum, "the first lowerer supports bf16 inputs only")
    if partial_type.element_type != "f32" or result_type.element_type != "f32":
        raise _reject(einsum, "the first lowerer supports f32 accumulation only")
    lhs_names = [name for name, _ in lhs_type.logical_shape()]
    rhs_names = [name for name, _ in rhs_type.logical_shape()]
    contraction = einsum.properties["contracting_dimension"]
    if len(lhs_names) != 2 or len(rhs_names) != 2 or lhs_names[1] != contraction or rhs_names[0] != contraction:
        raise _reject(einsum, "the first lowerer requires rank-2 lhs[M,K] and rhs[K,N] orientation")
    axes, dimensions = collective.properties["axes"], collective.properties["scatter_dimensions"]
    if len(axes) != 1 or len(dimensions) != 1 or collective.properties["reducer"] != "sum":
        raise _reject(collective, "the first lowerer supports one sum reduce-scatter axis")
    mesh = program_mesh(program)
    mesh_axis = axes[0]
    partial_names = [name for name, _ in partial_type.logical_shape()]
    scatter_index = partial_names.index(dimensions[0])

    def sharding(tensor_type: DTensorType) -> tuple[str, ...]:
        return tuple("/".join(axes_) for axes_ in tensor_type.sharding_axes())

    def names(tensor_type: DTensorType) -> tuple[str, ...]:
        return tuple(name for name, _ in tensor_type.logical_shape())

    lhs_shape, rhs_shape = _local_shape(lhs_type, mesh), _local_shape(rhs_type, mesh)
    partial_shape, result_shape = _local_shape(partial_type, mesh), _local_shape(result_type, mesh)
    external = {"memory": "hbm", "ownership": "external", "lifetime": (0, 5)}
    inputs = (
        buffer(lhs_shape, names(lhs_type), "bf16", sharding=sharding(lhs_type), **external),
        buffer(rhs_shape, names(rhs_type), "bf16", sharding=sharding(rhs_type), **external),
        buffer(result_shape, names(result_type), "f32", sharding=sharding(result_type), **external),
    )
    builder = KernelBuilder(
        f"{program.properties['sym_name']}_physical", target.name, inputs,
        vmem_capacity_bytes=target.vmem_capacity_bytes, smem_capacity_bytes=target.smem_capacity_bytes, mesh=mesh,
        interconnect_bandwidth_bytes_per_second={axis: target.ici_bandwidth_bytes_per_second for axis in mesh},
    )
    lhs = builder.alloc(buffer(lhs_shape, names(lhs_type), "bf16", memory="vmem", sharding=sharding(lhs_type), lifetime=(0, 2)), "lhs_tile")
    rhs = builder.alloc(buffer(rhs_shape, names(rhs_type), "bf16", memory="vmem", sharding=sharding(rhs_type), lifetime=(0, 2)), "rhs_tile")
    partial = builder.alloc(buffer(partial_shape, names(partial_type), "f32", memory="vmem", lifetime=(2, 3)), "partial_accumulator")
    reduced = builder.alloc(buffer(result_shape, names(result_type), "f32", memory="vmem", sharding=sharding(result_type), lifetime=(3, 5)), "reduced_output")
    lhs_semaphore, rhs_semaphore, output_semaphore = builder.semaphore(), builder.semaphore(), builder.semaphore()
    lhs_dma = builder.dma_start(builder.inputs[0], lhs, lhs_semaphore, stage=0)
    rhs_dma = builder.dma_start(builder.inputs[1], rhs, rhs_semaphore, stage=0)
    builder.dma_wait(lhs_dma, stage=1)
    builder.dma_wait(rhs_dma, stage=1)
    matmul = builder.matmul(
        lhs, rhs, partial, stage=2,
        tile_m=tile.m if tile is not None else lhs_shape[0], tile_k=lhs_shape[1],
        tile_n=tile.n if tile is not None else rhs_shape[1],
    )
    matmul.location = einsum.location
    physical_collective = builder.collective_reduce_scatter(
        partial, reduced, stage=3, mesh_axis=mesh_axis, group_size=mesh[mesh_axis], scatter_dimension=scatter_index,
        implementation=collective_implementation,
    )
    physical_collective.location = collective.location
    output_dma = builder.dma_start(reduced, builder.inputs[2], output_semaphore, stage=4)
    builder.dma_wait(output_dma, stage=5)
    return builder.module()
