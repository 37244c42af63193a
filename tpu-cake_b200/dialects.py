"""Builders and verifiers for the subset of ``dtensor.*`` and ``tpu_schedule.*`` the matmul path uses.

Logical dialect (src/tpu_cake/dialects/distributed_tensor.py): ``program``, ``einsum_local``
(:1020-1093), ``reduce_scatter`` (:1202-1254), ``return``. Physical dialect
(src/tpu_cake/dialects/tpu_schedule.py): ``kernel`` (:3230-3296), ``alloc``, ``semaphore_alloc``,
``dma_start`` / ``dma_wait``, ``mxu_matmul`` (:952-1015), ``collective`` (:1748-1969), ``yield``.
The verifier rules restated here are the ones the 16-op physical matmul kernel exercises: operand
placement and liveness, tile divisibility with ``tile_k == K``, the reduce-scatter shape and
sharding transition, one wait per DMA, and live on-chip bytes within the target's capacity.
"""

from __future__ import annotations

from enum import StrEnum

from .ir import Block, BufferType, DTensorType, Module, OpaqueType, Operation, SourceLocation, Value, VerifyException


class CollectiveImplementation(StrEnum):
    """How a physical collective is carried out. The reference has ``pallas_bidirectional_ring``
    (tpu_schedule.py:89-104) beside the compiler's collective; the B200 backend has the NCCL
    collective and the owner-push epilogue with f32 or bf16 transport."""

    NCCL = "nccl"
    P2P_OWNER_PUSH = "p2p_owner_push"
    P2P_OWNER_PUSH_BF16 = "p2p_owner_push_bf16"


DMA_TOKEN = OpaqueType("tpu_schedule.dma_token")
SEMAPHORE = OpaqueType("tpu_schedule.semaphore")


# ------------------------------------------------------------------------------ logical dialect


def tensor(element_type: str, dimensions, *, sharding: dict | None = None, pending_reductions: dict | None = None) -> DTensorType:
    """``tensor(bf16, (("M", m), ("K", k)), sharding={"K": ("t",)})`` as in distributed_frontend.py."""
    sharding = sharding or {}
    names = [name for name, _ in dimensions]
    unknown = set(sharding) - set(names)
    if unknown:
        raise VerifyException(f"sharding names unknown dimensions {sorted(unknown)}")
    return DTensorType(
        element_type=element_type,
        dimensions=tuple((name, int(size)) for name, size in dimensions),
        sharding=tuple(tuple(sharding.get(name, ())) for name in names),
        pending_reductions=tuple(sorted((pending_reductions or {}).items())),
    )


class DistributedProgramBuilder:
    """Builds one ``dtensor.program`` (distributed_frontend.py:75-570, the three methods used)."""

    def __init__(self, name: str, mesh: dict[str, int], inputs: tuple[DTensorType, ...]):
        if list(mesh) != sorted(mesh):
            raise VerifyException("mesh axes must be lexically sorted")
        self.block = Block(args=[Value(t) for t in inputs])
        for index, value in enumerate(self.block.args):
            value.owner, value.index = self.block, index
        self.program = Operation(
            "dtensor.program",
            properties={"sym_name": name, "mesh_axis_names": tuple(mesh), "mesh_axis_sizes": tuple(mesh.values())},
            body=self.block,
        )
        self.inputs = tuple(self.block.args)

    def einsum_local(self, lhs: Value, rhs: Value, result: DTensorType, *, contracting_dimension: str, source: SourceLocation | None = None) -> Value:
        op = Operation("dtensor.einsum_local", [lhs, rhs], [result], {"contracting_dimension": contracting_dimension}, location=source)
        self.block.ops.append(op)
        return op.result

    def reduce_scatter(self, value: Value, result: DTensorType, *, axes: tuple[str, ...], scatter_dimensions: tuple[str, ...], reducer: str = "sum", source: SourceLocation | None = None) -> Value:
        op = Operation(
            "dtensor.reduce_scatter", [value], [result],
            {"axes": tuple(axes), "scatter_dimensions": tuple(scatter_dimensions), "reducer": reducer}, location=source,
        )
        self.block.ops.append(op)
        return op.result

    def module(self, *results: Value) -> Module:
        self.block.ops.append(Operation("dtensor.return", list(results)))
        module = Module([self.program])
        module.verify()
        return module


def program_mesh(program: Operation) -> dict[str, int]:
    return dict(zip(program.properties["mesh_axis_names"], program.properties["mesh_axis_sizes"], strict=True))


# ----------------------------------------------------------------------------- physical dialect


def buffer(shape, logical_shape, element_type: str, *, memory: str = "hbm", sharding=None, ownership: str = "local", lifetime=(0, 0)) -> BufferType:
    return BufferType(
        shape=tuple(int(v) for v in shape), logical_shape=tuple(logical_shape), element_type=element_type, memory=memory,
        sharding=tuple(sharding) if sharding is not None else ("",) * len(tuple(shape)), ownership=ownership,
        lifetime=(int(lifetime[0]), int(lifetime[1])),
    )


class KernelBuilder:
    """Builds one ``tpu_schedule.kernel`` (frontend.py:75-630, the methods the matmul lowering uses)."""

    def __init__(self, name: str, target: str, inputs: tuple[BufferType, ...], *, vmem_capacity_bytes: int, smem_capacity_bytes: int,
                 mesh: dict[str, int], interconnect_bandwidth_bytes_per_second: dict[str, int]):
        self.block = Block(args=[Value(t) for t in inputs])
        for index, value in enumerate(self.block.args):
            value.owner, value.index = self.block, index
        self.kernel = Operation(
            "tpu_schedule.kernel",
            properties={
                "sym_name": name, "target": target, "vmem_capacity_bytes": int(vmem_capacity_bytes),
                "smem_capacity_bytes": int(smem_capacity_bytes), "mesh_axis_names": tuple(mesh),
                "mesh_axis_sizes": tuple(mesh.values()),
                "topology": tuple(f"{axis}:{interconnect_bandwidth_bytes_per_second[axis]}" for axis in mesh),
                "physical_schema": "static-topology-v3", "topology_authority": "static-cost-model-only",
            },
            body=self.block,
        )
        self.inputs = tuple(self.block.args)

    def _append(self, op: Operation) -> Operation:
        self.block.ops.append(op)
        return op

    def alloc(self, type_: BufferType, role: str) -> Value:
        return self._append(Operation("tpu_schedule.alloc", [], [type_], {"role": role})).result

    def semaphore(self) -> Value:
        return self._append(Operation("tpu_schedule.semaphore_alloc", [], [SEMAPHORE])).result

    def dma_start(self, source: Value, destination: Value, semaphore: Value, *, stage: int) -> Value:
        return self._append(Operation("tpu_schedule.dma_start", [source, destination, semaphore], [DMA_TOKEN], {"stage": stage})).result

    def dma_wait(self, token: Value, *, stage: int) -> None:
        self._append(Operation("tpu_schedule.dma_wait", [token], [], {"stage": stage}))

    def matmul(self, lhs: Value, rhs: Value, accumulator: Value, *, stage: int, tile_m: int, tile_k: int, tile_n: int) -> Operation:
        return self._append(Operation("tpu_schedule.mxu_matmul", [lhs, rhs, accumulator], [], {"stage": stage, "tile_m": tile_m, "tile_k": tile_k, "tile_n": tile_n}))

    def collective_reduce_scatter(self, source: Value, destination: Value, *, stage: int, mesh_axis: str, group_size: int,
                                  scatter_dimension: int, implementation: CollectiveImplementation | None = None) -> Operation:
        properties = {
            "kind": "reduce_scatter", "stage": stage, "mesh_axis": mesh_axis, "group_size": group_size,
            "split_dimension": scatter_dimension, "concat_dimension": -1, "reducer": "sum", "collective_plan": f"axis:{mesh_axis}",
        }
        if implementation is not None:
            properties["implementation"] = CollectiveImplementation(implementation).value
        return self._append(Operation("tpu_schedule.collective", [source, destination], [], properties))

    def module(self) -> Module:
        self._append(Operation("tpu_schedule.yield"))
        module = Module([self.kernel])
        module.verify()
        return module


# ------------------------------------------------------------------------------------ verifiers


def _fail(op: Operation, message: str) -> VerifyException:
    where = f" at {op.location}" if op.location else ""
    return VerifyException(f"{op.name}: {message}{where}")


def _buffer(op: Operation, value: Value, role: str) -> BufferType:
    if not isinstance(value.type, BufferType):
        raise _fail(op, f"{role} must be a buffer")
    return value.type


def _live(buffer_type: BufferType, stage: int) -> bool:
    return buffer_type.lifetime[0] <= stage <= buffer_type.lifetime[1]


def _verify_program(op: Operation) -> None:
    names, sizes = op.properties["mesh_axis_names"], op.properties["mesh_axis_sizes"]
    if len(names) != len(sizes) or any(size <= 0 for size in sizes):
        raise _fail(op, "mesh axes need positive sizes")
    if list(names) != sorted(names):
        raise _fail(op, "mesh axes must be lexically sorted")
    mesh = dict(zip(names, sizes))
    for value in list(op.body.args) + [r for inner in op.body.ops for r in inner.results]:
        tensor_type = value.type
        if not isinstance(tensor_type, DTensorType):
            raise _fail(op, "program values must be distributed tensors")
        for (name, size), axes in zip(tensor_type.dimensions, tensor_type.sharding, strict=True):
            divisor = 1
            for axis in axes:
                if axis not in mesh:
                    raise _fail(op, f"dimension {name} is sharded over unknown mesh axis {axis}")
                divisor *= mesh[axis]
            if size % divisor:
                raise _fail(op, f"dimension {name}={size} is not divisible by its sharding {axes}")
    if not op.body.ops or op.body.ops[-1].name != "dtensor.return":
        raise _fail(op, "program must end with dtensor.return")


def _verify_einsum_local(op: Operation) -> None:
    lhs, rhs, out = op.operands[0].type, op.operands[1].type, op.result.type
    contraction = op.properties["contracting_dimension"]
    lhs_dims, rhs_dims, out_dims = dict(lhs.dimensions), dict(rhs.dimensions), dict(out.dimensions)
    if contraction not in lhs_dims or contraction not in rhs_dims or lhs_dims[contraction] != rhs_dims[contraction]:
        raise _fail(op, f"contracting dimension {contraction} must appear with equal extent in both operands")
    if contraction in out_dims:
        raise _fail(op, "contracting dimension must not appear in the result")
    for name, size in out.dimensions:
        source = lhs_dims.get(name, rhs_dims.get(name))
        if source != size:
            raise _fail(op, f"result dimension {name} does not match its operand")
    lhs_axes = lhs.sharding[[n for n, _ in lhs.dimensions].index(contraction)]
    rhs_axes = rhs.sharding[[n for n, _ in rhs.dimensions].index(contraction)]
    if lhs_axes != rhs_axes:
        raise _fail(op, "both operands must shard the contracting dimension identically")
    pending = dict(out.pending_reductions)
    if set(pending) != set(lhs_axes) or any(v != "sum" for v in pending.values()):
        raise _fail(op, "a contraction over a sharded dimension leaves a pending sum over exactly those axes")


def _verify_reduce_scatter(op: Operation) -> None:
    source, out = op.operands[0].type, op.result.type
    axes, dims, reducer = op.properties["axes"], op.properties["scatter_dimensions"], op.properties["reducer"]
    if len(axes) != len(dims) or not axes:
        raise _fail(op, "one scatter dimension per reduced axis")
    pending = dict(source.pending_reductions)
    for axis in axes:
        if pending.get(axis) != reducer:
            raise _fail(op, f"axis {axis} has no pending {reducer} reduction")
    if dict(out.pending_reductions) != {k: v for k, v in pending.items() if k not in axes}:
        raise _fail(op, "result must drop exactly the reduced axes from the pending reductions")
    if [d for d in out.dimensions] != [d for d in source.dimensions] or out.element_type != source.element_type:
        raise _fail(op, "reduce-scatter keeps logical shape and element type")
    names = [n for n, _ in source.dimensions]
    for axis, dim in zip(axes, dims):
        if dim not in names:
            raise _fail(op, f"unknown scatter dimension {dim}")
        i = names.index(dim)
        if out.sharding[i] != source.sharding[i] + (axis,):
            raise _fail(op, f"dimension {dim} must gain mesh axis {axis} in its sharding")


def _verify_matmul(op: Operation) -> None:
    stage = op.properties["stage"]
    lhs, rhs, acc = (_buffer(op, v, r) for v, r in zip(op.operands, ("lhs", "rhs", "accumulator")))
    for role, b in (("lhs", lhs), ("rhs", rhs), ("accumulator", acc)):
        if b.memory != "vmem":
            raise _fail(op, f"{role} must be in on-chip memory")
        if not _live(b, stage):
            raise _fail(op, f"{role} is not live at stage {stage}")
        if len(b.shape) != 2:
            raise _fail(op, f"{role} must have rank 2")
    if lhs.shape[1] != rhs.shape[0] or acc.shape != (lhs.shape[0], rhs.shape[1]):
        raise _fail(op, "shapes must be M x K . K x N -> M x N")
    if lhs.element_type not in ("bf16", "f16") or lhs.element_type != rhs.element_type:
        raise _fail(op, "inputs must share a bf16 or f16 element type")
    if acc.element_type != "f32":
        raise _fail(op, "accumulator must be f32")
    tile_m, tile_k, tile_n = op.properties["tile_m"], op.properties["tile_k"], op.properties["tile_n"]
    if min(tile_m, tile_k, tile_n) <= 0 or lhs.shape[0] % tile_m or rhs.shape[1] % tile_n:
        raise _fail(op, "tiles must be positive and divide the operands")
    if tile_k != lhs.shape[1]:
        raise _fail(op, "tile_k must equal the full local contraction extent")


def _verify_collective(op: Operation) -> None:
    if op.properties["kind"] != "reduce_scatter":
        raise _fail(op, "only reduce_scatter is lowered by this backend")
    source, destination = _buffer(op, op.operands[0], "source"), _buffer(op, op.operands[1], "destination")
    group, split = op.properties["group_size"], op.properties["split_dimension"]
    if group <= 1:
        raise _fail(op, "group_size must exceed 1")
    if not 0 <= split < len(source.shape) or source.shape[split] % group:
        raise _fail(op, "split dimension must exist and be divisible by the group size")
    expected = list(source.shape)
    expected[split] //= group
    if tuple(expected) != destination.shape or destination.element_type != source.element_type:
        raise _fail(op, f"destination must be {tuple(expected)} {source.element_type}")
    axis = op.properties["mesh_axis"]
    previous = source.sharding[split]
    wanted = f"{previous}/{axis}" if previous else axis
    if destination.sharding[split] != wanted:
        raise _fail(op, f"destination dimension {split} must be sharded over {wanted}")
    implementation = op.properties.get("implementation")
    if implementation is not None:
        CollectiveImplementation(implementation)
        if op.properties["reducer"] != "sum" or source.element_type != "f32":
            raise _fail(op, "owned collective implementations reduce f32 sums")


def _verify_kernel(op: Operation) -> None:
    names = op.properties["mesh_axis_names"]
    if list(names) != sorted(names):
        raise _fail(op, "mesh axes must be lexically sorted")
    if not op.body.ops or op.body.ops[-1].name != "tpu_schedule.yield":
        raise _fail(op, "kernel must end with tpu_schedule.yield")
    pending_tokens: dict[int, Operation] = {}
    busy_semaphores: set[int] = set()
    local_buffers: list[BufferType] = []
    last_stage = 0
    for inner in op.body.ops:
        stage = inner.properties.get("stage")
        if stage is not None:
            if stage < 0:
                raise _fail(inner, "stage must be non-negative")
            last_stage = max(last_stage, stage)
        if inner.name == "tpu_schedule.alloc":
            local_buffers.append(inner.result.type)
        elif inner.name == "tpu_schedule.dma_start":
            source, destination = _buffer(inner, inner.operands[0], "source"), _buffer(inner, inner.operands[1], "destination")
            if source.shape != destination.shape or source.element_type != destination.element_type:
                raise _fail(inner, "DMA source and destination must agree in shape and element type")
            if not _live(source, stage) or not _live(destination, stage):
                raise _fail(inner, f"DMA operands must be live at stage {stage}")
            semaphore = id(inner.operands[2])
            if semaphore in busy_semaphores:
                raise _fail(inner, "semaphore reused before its DMA was waited on")
            busy_semaphores.add(semaphore)
            pending_tokens[id(inner.result)] = inner
        elif inner.name == "tpu_schedule.dma_wait":
            start = pending_tokens.pop(id(inner.operands[0]), None)
            if start is None:
                raise _fail(inner, "DMA token waited on twice or never started")
            if stage < start.properties["stage"]:
                raise _fail(inner, "DMA waited on before it starts")
            busy_semaphores.discard(id(start.operands[2]))
    if pending_tokens:
        raise _fail(op, "every DMA must be waited on before the kernel ends")
    for capacity_key, space in (("vmem_capacity_bytes", "vmem"), ("smem_capacity_bytes", "smem")):
        capacity = op.properties[capacity_key]
        for stage in range(last_stage + 1):
            live = sum(b.nbytes() for b in local_buffers if b.memory == space and _live(b, stage))
            if live > capacity:
                raise _fail(op, f"{live} live {space} bytes at stage {stage} exceed the capacity {capacity}")


_VERIFIERS = {
    "dtensor.program": _verify_program,
    "dtensor.einsum_local": _verify_einsum_local,
    "dtensor.reduce_scatter": _verify_reduce_scatter,
    "tpu_schedule.kernel": _verify_kernel,
    "tpu_schedule.mxu_matmul": _verify_matmul,
    "tpu_schedule.collective": _verify_collective,
}


def verify_operation(op: Operation) -> None:
    verifier = _VERIFIERS.get(op.name)
    if verifier is not None:
        verifier(op)
