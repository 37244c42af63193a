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


FUSED_RPA_UPSTREAM_AUTHORITY = "opaque-upstream-wrapper"  # the reference's only authority: decode, scale = 1/head_dim
FUSED_RPA_CUDA_AUTHORITY = "cake-b200-sm100-kernels"       # this backend: any positive scale, ragged query runs
B200_SHARED_MEMORY_PER_CTA = 232448


class CollectiveImplementation(StrEnum):
    """How a physical collective is carried out. The reference has ``pallas_bidirectional_ring``
    (tpu_schedule.py:89-104) beside the compiler's collective; the B200 backend has the NCCL
    collective and the owner-push epilogue with f32 or bf16 transport."""

    NCCL = "nccl"
    P2P_OWNER_PUSH = "p2p_owner_push"
    P2P_OWNER_PUSH_BF16 = "p2p_owner_push_bf16"
    P2P_PEER_STORE = "p2p_peer_store"  # all-gather: the producing kernel stores its rows into every rank's buffer


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

    def collective_all_gather(self, source: Value, destination: Value, *, stage: int, mesh_axis: str, group_size: int,
                              concat_dimension: int, implementation: CollectiveImplementation | None = None) -> Operation:
        """All-gather along ``concat_dimension`` (tpu_schedule.py:1914-1923): the collective of the
        decode sharded by KV head, whose per-rank outputs are gathered along the head dimension."""
        properties = {
            "kind": "all_gather", "stage": stage, "mesh_axis": mesh_axis, "group_size": group_size,
            "split_dimension": -1, "concat_dimension": concat_dimension, "reducer": "none", "collective_plan": f"axis:{mesh_axis}",
        }
        if implementation is not None:
            properties["implementation"] = CollectiveImplementation(implementation).value
        return self._append(Operation("tpu_schedule.collective", [source, destination], [], properties))

    def ragged_paged_attention(self, query: Value, key_cache: Value, value_cache: Value, page_table: Value, sequence_lengths: Value,
                               bias: Value, output: Value, *, stage: int, query_block_size: int, kv_block_size: int) -> Operation:
        """The prototype decode op (tpu_schedule.py:2003-2103): separate caches, 2-D page table, dense bias."""
        return self._append(Operation(
            "tpu_schedule.ragged_paged_attention", [query, key_cache, value_cache, page_table, sequence_lengths, bias, output], [],
            {"stage": stage, "query_block_size": query_block_size, "kv_block_size": kv_block_size},
        ))

    def fused_ragged_paged_attention(self, operands: tuple[Value, ...], *, stage: int, softmax_scale: str, causal: int = 1,
                                     softmax_dtype: str = "float32", sliding_window: int = 0, query_block_size: int = 8,
                                     kv_block_size: int = 128, query_cluster_size: int = 8, kv_cluster_size: int = 128,
                                     vmem_limit_bytes: int = 1 << 20, execution_authority: str = FUSED_RPA_UPSTREAM_AUTHORITY,
                                     donated_operand_indices: tuple[int, ...] = (0, 1, 2, 3)) -> Operation:
        """The fused-cache op (tpu_schedule.py:2107-2349): 11 inputs + the two aliased outputs."""
        if len(operands) != 13:
            raise ValueError("fused RPA takes 11 inputs followed by the output and the updated cache")
        return self._append(Operation(
            "tpu_schedule.fused_ragged_paged_attention", list(operands), [],
            {"stage": stage, "causal": causal, "softmax_scale": softmax_scale, "softmax_dtype": softmax_dtype,
             "sliding_window": sliding_window, "query_block_size": query_block_size, "kv_block_size": kv_block_size,
             "query_cluster_size": query_cluster_size, "kv_cluster_size": kv_cluster_size, "vmem_limit_bytes": vmem_limit_bytes,
             "execution_authority": execution_authority, "donated_operand_indices": tuple(donated_operand_indices)},
        ))

    def cuda_rpa_decode(self, attention: Operation, *, stage: int, kv_chunk_tokens: int, warps_per_cta: int, ring_stages: int,
                        stage_tokens: int, shared_memory_bytes: int, workspace_bytes: int) -> Operation:
        """Static resource contract of the sm_100a decode kernel for one attention op of this kernel:
        the sibling of the reference's rpa_decode_core (tpu_schedule.py:2357-2885), whose VMEM / DMA
        semaphore shapes do not transfer to a GPU."""
        return self._append(Operation(
            "tpu_schedule.cuda_rpa_decode", list(attention.operands), [],
            {"stage": stage, "kv_chunk_tokens": kv_chunk_tokens, "warps_per_cta": warps_per_cta, "ring_stages": ring_stages,
             "stage_tokens": stage_tokens, "shared_memory_bytes": shared_memory_bytes, "workspace_bytes": workspace_bytes,
             "attention": attention.name, "backend": "cake-b200/sm_100a"},
        ))

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
    """Rules of the reference's collective (tpu_schedule.py:1867-1960) for the two kinds this backend
    lowers: reduce-scatter (the matmul's) and all-gather (the sharded decode's)."""
    kind = op.properties["kind"]
    if kind not in ("reduce_scatter", "all_gather"):
        raise _fail(op, "only reduce_scatter and all_gather are lowered by this backend")
    source, destination = _buffer(op, op.operands[0], "source"), _buffer(op, op.operands[1], "destination")
    group, split, concat = op.properties["group_size"], op.properties["split_dimension"], op.properties["concat_dimension"]
    if group <= 1:
        raise _fail(op, "group_size must exceed 1")
    if len(source.shape) != len(destination.shape):
        raise _fail(op, "collectives cannot change rank")
    axis = op.properties["mesh_axis"]
    implementation = op.properties.get("implementation")
    if implementation is not None:
        implementation = CollectiveImplementation(implementation)
    expected = list(source.shape)
    if kind == "reduce_scatter":
        if concat != -1 or op.properties["reducer"] == "none":
            raise _fail(op, "reduce-scatter needs a reducer and one split dimension")
        if not 0 <= split < len(source.shape) or source.shape[split] % group:
            raise _fail(op, "split dimension must exist and be divisible by the group size")
        expected[split] //= group
        previous = source.sharding[split]
        dimension, wanted = split, (f"{previous}/{axis}" if previous else axis)
        if implementation is CollectiveImplementation.P2P_PEER_STORE:
            raise _fail(op, "peer stores carry an all-gather, not a reduction")
        if implementation is not None and (op.properties["reducer"] != "sum" or source.element_type != "f32"):
            raise _fail(op, "owned collective implementations reduce f32 sums")
    else:
        if split != -1 or op.properties["reducer"] != "none":
            raise _fail(op, "all-gather needs one concat dimension and no reducer")
        if not 0 <= concat < len(source.shape):
            raise _fail(op, "collective dimension is out of range")
        parts = source.sharding[concat].split("/") if source.sharding[concat] else []
        if not parts or parts[-1] != axis:
            raise _fail(op, "all-gather must remove its mesh axis from the gathered dimension")
        expected[concat] *= group
        dimension, wanted = concat, "/".join(parts[:-1])
        if implementation not in (None, CollectiveImplementation.NCCL, CollectiveImplementation.P2P_PEER_STORE):
            raise _fail(op, "an all-gather is carried by NCCL or by peer stores")
    if tuple(expected) != destination.shape or destination.element_type != source.element_type:
        raise _fail(op, f"destination must be {tuple(expected)} {source.element_type}")
    if destination.sharding[dimension] != wanted:
        raise _fail(op, f"destination dimension {dimension} must be sharded over {wanted!r}")


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


def _verify_paged_attention(op: Operation) -> None:
    """Rules and messages of RaggedPagedAttentionOp.verify_ (tpu_schedule.py:2039-2103)."""
    stage = op.properties["stage"]
    names = ("query", "key_cache", "value_cache", "page_table", "sequence_lengths", "bias", "output")
    query, key_cache, value_cache, page_table, lengths, bias, output = (_buffer(op, v, n) for v, n in zip(op.operands, names))
    for name, b in zip(names, (query, key_cache, value_cache, page_table, lengths, bias, output)):
        if not _live(b, stage):
            raise _fail(op, f"{name} is not live at stage {stage}")
    if query.memory != "vmem" or output.memory != "vmem":
        raise _fail(op, "RPA query and output must be resident in VMEM")
    if bias.memory != "vmem":
        raise _fail(op, "RPA relative-position bias must be resident in VMEM")
    if any(b.memory != "hbm" for b in (key_cache, value_cache, page_table, lengths)):
        raise _fail(op, "RPA cache and page metadata must reside in HBM")
    if len(query.shape) != 3 or len(key_cache.shape) != 4 or len(value_cache.shape) != 4 or len(output.shape) != 3:
        raise _fail(op, "RPA expects query/output [batch, heads, dim] and caches [pages, page, heads, dim]")
    batch, query_heads, query_dimension = query.shape
    key_pages, page_size, key_heads, key_dimension = key_cache.shape
    value_pages, value_page_size, value_heads, value_dimension = value_cache.shape
    if (key_pages, page_size) != (value_pages, value_page_size):
        raise _fail(op, "RPA key and value caches must share pages and page size")
    if query_dimension != key_dimension:
        raise _fail(op, "RPA query and key head dimensions must match")
    if key_heads <= 0 or value_heads <= 0:
        raise _fail(op, "RPA key and value head counts must be positive")
    if query_heads % key_heads or query_heads % value_heads:
        raise _fail(op, "RPA query heads must divide evenly across key and value heads")
    if output.shape != (batch, query_heads, value_dimension):
        raise _fail(op, "RPA output must use batch/query heads and value dimension")
    if len(page_table.shape) != 2 or len(bias.shape) != 2:
        raise _fail(op, "RPA page table and bias must be rank 2")
    if page_table.shape[0] != batch or lengths.shape != (batch,):
        raise _fail(op, "RPA page metadata batch dimensions must match query")
    if bias.shape[0] != query_heads:
        raise _fail(op, "RPA bias head dimension must match query")
    if bias.shape[1] < page_table.shape[1] * page_size:
        raise _fail(op, "RPA bias extent must cover every addressable cache position")
    if op.properties["kv_block_size"] <= 0 or page_size % op.properties["kv_block_size"]:
        raise _fail(op, "RPA KV block size must be positive and divide page size")
    if op.properties["query_block_size"] <= 0:
        raise _fail(op, "RPA query block size must be positive")


def _verify_fused_paged_attention(op: Operation) -> None:
    """Rules and messages of FusedRaggedPagedAttentionOp.verify_ (tpu_schedule.py:2195-2349). Under the
    reference's authority the strict decode contract holds (tokens == sequences, scale * dim == 1);
    under this backend's authority the scale is any positive decimal and sequences may own query runs."""
    from decimal import Decimal, InvalidOperation

    names = ("queries", "keys", "values", "fused_cache", "kv_lengths", "page_indices", "cumulative_query_lengths",
             "cumulative_kv_lengths", "distribution", "relative_states", "relative_projection", "output", "updated_cache")
    buffers = [_buffer(op, v, n) for v, n in zip(op.operands, names)]
    if any(b.memory != "hbm" for b in buffers):
        raise _fail(op, "fused RPA wrapper operands must reside in HBM")
    stage = op.properties["stage"]
    if any(not _live(b, stage) for b in buffers):
        raise _fail(op, f"fused RPA operands must be live at stage {stage}")
    q, k, v, cache, lens, pages, cu_q, cu_kv, dist, states, projection, output, updated = buffers
    if len(q.shape) != 3 or len(k.shape) != 3 or len(v.shape) != 3:
        raise _fail(op, "fused RPA Q/K/V must have [tokens, heads, dim] shape")
    if len(cache.shape) != 5:
        raise _fail(op, "fused RPA cache must have [pages, page, packed_heads, packing, dim] shape")
    if any(extent <= 0 for extent in (*q.shape, *k.shape, *v.shape, *cache.shape)):
        raise _fail(op, "fused RPA Q/K/V/cache dimensions must be positive")
    if any(b.element_type != "bf16" for b in (q, k, v, cache, states, projection, output, updated)):
        raise _fail(op, "Inkling fused RPA data buffers must use bf16")
    if any(b.element_type != "i32" for b in (lens, pages, cu_q, cu_kv, dist)):
        raise _fail(op, "fused RPA metadata buffers must use i32")
    tokens, query_heads, dimension = q.shape
    if (k.shape[0], v.shape[0]) != (tokens, tokens):
        raise _fail(op, "fused RPA Q/K/V token counts must match")
    if k.shape[1] != v.shape[1] or query_heads % k.shape[1]:
        raise _fail(op, "fused RPA requires equal K/V heads dividing query heads")
    if (k.shape[2], v.shape[2]) != (dimension, dimension):
        raise _fail(op, "fused RPA Q/K/V head dimensions must match")
    _, _, packed_heads, packing, cache_dimension = cache.shape
    if cache_dimension != -(-dimension // 128) * 128:
        raise _fail(op, "fused RPA cache head dimension must be padded to a multiple of 128")
    if packing != 2 or packed_heads * packing != 2 * k.shape[1]:
        raise _fail(op, "fused RPA cache must interleave one K and V per KV head")
    if output.shape != q.shape:
        raise _fail(op, "fused RPA output shape must match queries")
    if updated.shape != cache.shape:
        raise _fail(op, "fused RPA updated cache shape must match its input cache")
    if len(lens.shape) != 1 or not lens.shape[0]:
        raise _fail(op, "fused RPA KV lengths must be nonempty rank 1")
    if len(pages.shape) != 1:
        raise _fail(op, "fused RPA page indices must be rank 1")
    sequences = lens.shape[0]
    authority = op.properties["execution_authority"]
    if authority not in (FUSED_RPA_UPSTREAM_AUTHORITY, FUSED_RPA_CUDA_AUTHORITY):
        raise _fail(op, "fused RPA must declare delegated execution authority")
    strict = authority == FUSED_RPA_UPSTREAM_AUTHORITY
    if strict and tokens != sequences:
        raise _fail(op, "Inkling fused decode RPA requires one query token per sequence")
    if not strict and tokens < sequences:
        raise _fail(op, "fused RPA needs at least one query token per sequence")
    if strict and pages.shape[0] % sequences:
        raise _fail(op, "fused RPA flat page indices must divide across sequences")
    if cu_q.shape != (sequences + 1,) or cu_kv.shape != (sequences + 1,):
        raise _fail(op, "fused RPA cumulative lengths must have sequences + 1 entries")
    if dist.shape != (3,):
        raise _fail(op, "fused RPA distribution must contain three boundaries")
    if len(states.shape) != 3 or len(projection.shape) != 2:
        raise _fail(op, "fused RPA relative states/projection must be rank 3/rank 2")
    if states.shape[:2] != (tokens, query_heads):
        raise _fail(op, "fused RPA relative states must match query tokens and heads")
    if states.shape[2] != projection.shape[0]:
        raise _fail(op, "fused RPA relative dimensions must match")
    if op.properties["causal"] != 1:
        raise _fail(op, "Inkling fused RPA adapter requires causal attention without a custom mask")
    try:
        scale = Decimal(op.properties["softmax_scale"])
    except (InvalidOperation, TypeError) as error:
        raise _fail(op, "fused RPA softmax scale must be decimal") from error
    if not scale.is_finite() or scale <= 0:
        raise _fail(op, "fused RPA softmax scale must be positive and finite")
    if strict and scale * dimension != Decimal(1):
        raise _fail(op, "Inkling fused RPA softmax scale must equal 1 / head dimension")
    if op.properties["softmax_dtype"] != "float32":
        raise _fail(op, "Inkling fused RPA softmax must use float32")
    if op.properties["sliding_window"] < 0:
        raise _fail(op, "fused RPA sliding window cannot be negative")
    block_keys = ("query_block_size", "kv_block_size", "query_cluster_size", "kv_cluster_size", "vmem_limit_bytes")
    if any(op.properties[key] <= 0 for key in block_keys):
        raise _fail(op, "fused RPA block sizes and VMEM limit must be positive")
    if tuple(op.properties["donated_operand_indices"]) != (0, 1, 2, 3):
        raise _fail(op, "fused RPA must donate Q, K, V, and fused cache")
    if op.operands[11] is not op.operands[0] or op.operands[12] is not op.operands[3]:
        raise _fail(op, "fused RPA output/cache destinations must alias query/cache inputs")
    page_size = cache.shape[1]
    if (op.properties["query_block_size"] % op.properties["query_cluster_size"] or op.properties["kv_block_size"] % op.properties["kv_cluster_size"]
            or op.properties["kv_block_size"] % page_size):
        raise _fail(op, "fused RPA blocks must divide into clusters and KV blocks must align to pages")


def _verify_cuda_rpa_decode(op: Operation) -> None:
    """Resource contract of the sm_100a decode kernel: what one CTA holds in shared memory must match
    what the declared ring needs and fit a B200 CTA; chunks are whole stages."""
    props = op.properties
    if props["stage_tokens"] not in (16, 32):
        raise _fail(op, "a stage is one or two 16-token MMA groups")
    if props["kv_chunk_tokens"] <= 0 or props["kv_chunk_tokens"] % props["stage_tokens"]:
        raise _fail(op, "kv_chunk_tokens must be a positive multiple of the stage size")
    if props["warps_per_cta"] <= 0 or props["ring_stages"] < 2:
        raise _fail(op, "the kernel needs at least one worker warp and a two-stage ring")
    row_bytes = 256  # one token of one head: 128 bf16
    needed = props["warps_per_cta"] * (props["ring_stages"] * props["stage_tokens"] * 2 * row_bytes + 8 * row_bytes) + 1024 + 256
    if props["shared_memory_bytes"] != needed:
        raise _fail(op, f"shared_memory_bytes must be {needed} for this ring")
    if needed > B200_SHARED_MEMORY_PER_CTA:
        raise _fail(op, f"{needed} bytes of shared memory exceed the {B200_SHARED_MEMORY_PER_CTA} a B200 CTA may use")
    if props["workspace_bytes"] <= 0:
        raise _fail(op, "split-KV workspace must be declared")
    if props["attention"] not in ("tpu_schedule.ragged_paged_attention", "tpu_schedule.fused_ragged_paged_attention"):
        raise _fail(op, "cuda_rpa_decode refines an attention op of the same kernel")


_VERIFIERS = {
    "dtensor.program": _verify_program,
    "dtensor.einsum_local": _verify_einsum_local,
    "dtensor.reduce_scatter": _verify_reduce_scatter,
    "tpu_schedule.kernel": _verify_kernel,
    "tpu_schedule.mxu_matmul": _verify_matmul,
    "tpu_schedule.collective": _verify_collective,
    "tpu_schedule.ragged_paged_attention": _verify_paged_attention,
    "tpu_schedule.fused_ragged_paged_attention": _verify_fused_paged_attention,
    "tpu_schedule.cuda_rpa_decode": _verify_cuda_rpa_decode,
}


def verify_operation(op: Operation) -> None:
    verifier = _VERIFIERS.get(op.name)
    if verifier is not None:
        verifier(op)
