"""CUDA backend lowering of the physical matmul + reduce-scatter kernel.

Mirror of the reference's Pallas backend (src/tpu_cake/pallas_lowering.py): ``CudaMatmulRsPlan``
carries the same fields as ``PallasMatmulPlan`` (:335-351) and offers the same surface --
``global_*_shape`` (:353-363), ``build()`` (:417-476), ``render_executable_source()`` /
``source_sha256()`` (:554-606). ``build()`` returns an executable bound to this process's GPU and
mesh position instead of a jitted ``shard_map``: each mesh position is its own process.

Collective strategies (the reference's are ``xla_reduce_scatter`` and
``pallas_bidirectional_ring``, src/tpu_cake/runner.py:60-72):
  nccl_reduce_scatter                 the kernel writes the partial owner-major and NCCL reduces it
  p2p_fused_epilogue                  the kernel's epilogue pushes f32 partial tiles to the owner
  p2p_fused_epilogue_bf16_transport   same with bf16 partial tiles (half the NVLink bytes)
"""

from __future__ import annotations

import ast
import ctypes
from dataclasses import dataclass, field, replace
from enum import StrEnum
from pathlib import Path

import numpy as np
import torch

from . import _native
from .identity import text_sha256
from .mesh import ProcessMesh, SymmetricBuffer


class UnsupportedLoweringError(ValueError):
    """The schedule cannot be expressed by the CUDA backend (same name as lowering.py:23-24)."""


class MatmulCollectiveStrategy(StrEnum):
    NCCL_REDUCE_SCATTER = "nccl_reduce_scatter"
    P2P_FUSED_EPILOGUE = "p2p_fused_epilogue"
    P2P_FUSED_EPILOGUE_BF16_TRANSPORT = "p2p_fused_epilogue_bf16_transport"


SUPPORTED_TILE_M = (128,)
SUPPORTED_TILE_N = (64, 128, 256)
_TORCH_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16}
_CAKE_DTYPE = {"f32": _native.CAKE_DTYPE_F32, "bf16": _native.CAKE_DTYPE_BF16}


@dataclass(frozen=True)
class P2pCollectiveResources:
    """Static resources of the owner-push reduce-scatter, the counterpart of
    ``pallas_bidirectional_ring_resources`` (src/tpu_cake/dialects/tpu_schedule.py:89-104)."""

    receive_slot_bytes: int  # 2 parities x W sources x local output (padded to 128 B), in the transport dtype
    arrival_flag_bytes: int  # one 32-bit call number per source rank and quarter tile (32 rows x tile_n)
    remote_payload_bytes: int  # bytes this rank sends to other ranks per call
    reduce_read_bytes: int  # bytes the slot reduction reads per call


@dataclass(frozen=True)
class CudaMatmulRsPlan:
    name: str
    schedule_sha256: str
    mesh_axis: str
    mesh_size: int
    lhs_local_shape: tuple[int, int]
    rhs_local_shape: tuple[int, int]
    partial_local_shape: tuple[int, int]
    output_local_shape: tuple[int, int]
    lhs_sharding: tuple[str, str]
    rhs_sharding: tuple[str, str]
    output_sharding: tuple[str, str]
    scatter_dimension: int
    tile_m: int
    tile_k: int
    tile_n: int
    collective_link_bandwidths: tuple[tuple[str, int], ...] = ()
    collective_implementation: MatmulCollectiveStrategy | None = None
    output_dtype: str = "f32"

    def __post_init__(self) -> None:
        m, k_local = self.lhs_local_shape
        k_rhs, n = self.rhs_local_shape
        if k_local != k_rhs or self.partial_local_shape != (m, n):
            raise UnsupportedLoweringError(
                f"inconsistent local shapes lhs={self.lhs_local_shape} rhs={self.rhs_local_shape} "
                f"partial={self.partial_local_shape}"
            )
        if self.scatter_dimension not in (0, 1):
            raise UnsupportedLoweringError(f"scatter dimension must be 0 or 1, got {self.scatter_dimension}")
        expected = list(self.partial_local_shape)
        if expected[self.scatter_dimension] % self.mesh_size:
            raise UnsupportedLoweringError("scatter dimension is not divisible by the mesh size")
        expected[self.scatter_dimension] //= self.mesh_size
        if tuple(expected) != self.output_local_shape:
            raise UnsupportedLoweringError(
                f"output local shape {self.output_local_shape} does not match reduce-scatter of "
                f"{self.partial_local_shape} along {self.scatter_dimension}"
            )
        if self.tile_m not in SUPPORTED_TILE_M or self.tile_n not in SUPPORTED_TILE_N:
            raise UnsupportedLoweringError(
                f"sm_100a matmul tiles are {SUPPORTED_TILE_M} x {SUPPORTED_TILE_N}, got {self.tile_m} x {self.tile_n}"
            )
        if self.tile_k != k_local:
            raise UnsupportedLoweringError("tile_k must equal the local contraction extent (tpu_schedule.py:1014-1015)")
        if self.output_dtype not in _TORCH_DTYPE:
            raise UnsupportedLoweringError(f"output dtype must be f32 or bf16, got {self.output_dtype}")
        if self.mesh_size > 1 and self.collective_implementation is None:
            object.__setattr__(self, "collective_implementation", MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER)

    # ------------------------------------------------------------------ shapes
    def _global_shape(self, shape: tuple[int, int], sharding: tuple[str, str]) -> tuple[int, int]:
        return tuple(size * (self.mesh_size if axis == self.mesh_axis else 1) for size, axis in zip(shape, sharding, strict=True))

    @property
    def global_lhs_shape(self) -> tuple[int, int]:
        return self._global_shape(self.lhs_local_shape, self.lhs_sharding)

    @property
    def global_rhs_shape(self) -> tuple[int, int]:
        return self._global_shape(self.rhs_local_shape, self.rhs_sharding)

    @property
    def global_output_shape(self) -> tuple[int, int]:
        return self._global_shape(self.output_local_shape, self.output_sharding)

    @property
    def transport_dtype(self) -> str:
        if self.collective_implementation is MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT:
            return "bf16"
        return "f32"

    @property
    def collective_resources(self) -> P2pCollectiveResources:
        if self.mesh_size == 1 or self.collective_implementation is MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER:
            return P2pCollectiveResources(0, 0, 0, 0)
        size = 2 if self.transport_dtype == "bf16" else 4
        local = self.output_local_shape[0] * self.output_local_shape[1] * size
        quarters = -(-self.output_local_shape[0] // 128) * -(-self.output_local_shape[1] // self.tile_n) * 4
        return P2pCollectiveResources(
            receive_slot_bytes=2 * self.mesh_size * (-(-local // 128) * 128),
            arrival_flag_bytes=-(-self.mesh_size * quarters * 4 // 128) * 128,
            remote_payload_bytes=(self.mesh_size - 1) * local,
            reduce_read_bytes=self.mesh_size * local,
        )

    # ------------------------------------------------------------------ identity
    def render_executable_source(self) -> str:
        """A deterministic description of what ``build()`` runs; its hash is the plan's code
        identity (role of ``lowered_pallas.py`` in the reference's run bundle)."""
        lines = [
            "# cake-b200 lowered matmul + reduce-scatter",
            f"kernel = 'cake_matmul_rs_sm100<BN={self.tile_n}, rhs=[K,N]>'",
            f"name = {self.name!r}",
            f"schedule_sha256 = {self.schedule_sha256!r}",
            f"mesh = ({self.mesh_axis!r}, {self.mesh_size})",
            f"lhs_local = {self.lhs_local_shape}  # bf16, sharding {self.lhs_sharding}",
            f"rhs_local = {self.rhs_local_shape}  # bf16, sharding {self.rhs_sharding}",
            f"partial_local = {self.partial_local_shape}  # f32 accumulators in TMEM",
            f"output_local = {self.output_local_shape}  # {self.output_dtype}, sharding {self.output_sharding}",
            f"scatter_dimension = {self.scatter_dimension}",
            f"tile = ({self.tile_m}, {self.tile_k}, {self.tile_n})",
            f"collective = {None if self.collective_implementation is None else self.collective_implementation.value!r}",
            f"transport_dtype = {self.transport_dtype!r}",
            f"abi_version = 1",
        ]
        return "\n".join(lines) + "\n"

    def source_sha256(self) -> str:
        return text_sha256(self.render_executable_source())

    # ------------------------------------------------------------------ execution
    def build(self, *, mesh: ProcessMesh | None = None) -> tuple["MatmulRsExecutable", ProcessMesh]:
        """Creates the native plan on the current GPU. ``mesh`` defaults to a single-position mesh,
        which is only valid for ``mesh_size == 1``."""
        selected = mesh or ProcessMesh.single(self.mesh_axis)
        if selected.world != self.mesh_size:
            raise ValueError(f"CUDA plan needs {self.mesh_size} mesh positions, found {selected.world}")
        return MatmulRsExecutable(self, selected), selected


def plan_distributed_matmul(
    *,
    mesh_size: int,
    m: int,
    k: int,
    n: int,
    scatter_dimension: int = 1,
    output_dtype: str = "f32",
    tile_m: int = 128,
    tile_n: int = 256,
    collective_implementation: MatmulCollectiveStrategy | None = None,
    schedule_sha256: str = "0" * 64,
    mesh_axis: str = "t",
    name: str = "distributed_matmul_physical",
) -> CudaMatmulRsPlan:
    """Plan for lhs[M, K@t] x rhs[K@t, N] -> reduce-scatter along ``scatter_dimension``
    (the program of src/tpu_cake/workloads/distributed_matmul.py:22-46 after
    lower_distributed_matmul, src/tpu_cake/lowering.py:77-269)."""
    if k % mesh_size:
        raise UnsupportedLoweringError(f"K={k} is not divisible by the mesh size {mesh_size}")
    scattered = (m, n)[scatter_dimension]
    if scattered % mesh_size:
        raise UnsupportedLoweringError("scatter dimension is not divisible by the mesh size")
    k_local = k // mesh_size
    out = [m, n]
    out[scatter_dimension] //= mesh_size
    sharding = ["", ""]
    sharding[scatter_dimension] = mesh_axis
    return CudaMatmulRsPlan(
        name=name,
        schedule_sha256=schedule_sha256,
        mesh_axis=mesh_axis,
        mesh_size=mesh_size,
        lhs_local_shape=(m, k_local),
        rhs_local_shape=(k_local, n),
        partial_local_shape=(m, n),
        output_local_shape=(out[0], out[1]),
        lhs_sharding=("", mesh_axis),
        rhs_sharding=(mesh_axis, ""),
        output_sharding=(sharding[0], sharding[1]),
        scatter_dimension=scatter_dimension,
        tile_m=tile_m,
        tile_k=k_local,
        tile_n=tile_n,
        collective_implementation=collective_implementation,
        output_dtype=output_dtype,
    )


class MatmulRsExecutable:
    """``executable(lhs_local, rhs_local) -> out_local`` on this process's GPU.

    Inputs are this rank's shards: lhs bf16 [M, K/W], rhs bf16 [K/W, N] (the reference's
    ``P(None,'t')`` / ``P('t',None)`` placement). The call is asynchronous on the current torch
    stream. Fails loudly if libcake_b200.so is not built or the GPU is not sm_100.
    """

    def __init__(self, plan: CudaMatmulRsPlan, mesh: ProcessMesh, *, contraction_only: bool = False, wait_budget_ms: int = 0):
        """``contraction_only`` builds the same contraction with the same tiles and transport dtype
        but leaves the partial in local memory (owner-major) and runs no collective: the
        "pushes disabled" twin used to measure how much communication time is exposed.
        ``wait_budget_ms`` bounds how long the slot reduction waits for a peer (0 = 20 s)."""
        self.plan = plan
        self.mesh = mesh
        self._lib = _native.load()
        strategy = plan.collective_implementation
        self._contraction_only = contraction_only
        self._p2p = mesh.world > 1 and strategy is not MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER and not contraction_only
        desc = _native.MatmulRsDesc(
            m=plan.partial_local_shape[0],
            n=plan.partial_local_shape[1],
            k_local=plan.lhs_local_shape[1],
            world=mesh.world,
            rank=mesh.rank,
            scatter_dim=plan.scatter_dimension,
            out_dtype=_CAKE_DTYPE[plan.output_dtype],
            transport_dtype=_CAKE_DTYPE[plan.transport_dtype],
            strategy=_native.CAKE_RS_P2P_OWNER_PUSH if self._p2p else _native.CAKE_RS_LOCAL_PARTIAL,
            tile_m=plan.tile_m,
            tile_n=plan.tile_n,
            rhs_layout=0,
            wait_budget_ms=wait_budget_ms,
        )
        handle = ctypes.c_void_p()
        with torch.cuda.device(mesh.device):
            _native.check(self._lib.cake_matmul_rs_create(ctypes.byref(desc), ctypes.byref(handle)))
        self._handle = handle
        self._slots: SymmetricBuffer | None = None
        self._flags: SymmetricBuffer | None = None
        self._partial: torch.Tensor | None = None
        if self._p2p:
            with torch.cuda.device(mesh.device):
                self._slots = SymmetricBuffer(mesh, self._lib.cake_matmul_rs_slot_bytes(handle))
                self._flags = SymmetricBuffer(mesh, self._lib.cake_matmul_rs_flag_bytes(handle))
            pointer_array = ctypes.c_void_p * mesh.world
            _native.check(
                self._lib.cake_matmul_rs_bind_peers(
                    handle, pointer_array(*self._slots.pointers), pointer_array(*self._flags.pointers)
                )
            )
        elif mesh.world > 1:
            self._partial = torch.empty(
                (mesh.world,) + plan.output_local_shape, dtype=_TORCH_DTYPE[plan.transport_dtype], device=mesh.device
            )

    # -- device call
    def __call__(self, lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        plan = self.plan
        self._check_operand(lhs, plan.lhs_local_shape, "lhs")
        self._check_operand(rhs, plan.rhs_local_shape, "rhs")
        if out is None:
            out = torch.empty(plan.output_local_shape, dtype=_TORCH_DTYPE[plan.output_dtype], device=self.mesh.device)
        elif tuple(out.shape) != plan.output_local_shape or out.dtype != _TORCH_DTYPE[plan.output_dtype] or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor of the plan's local output shape and dtype")
        stream = torch.cuda.current_stream(self.mesh.device).cuda_stream
        if self._partial is not None:
            import torch.distributed as dist

            _native.check(self._lib.cake_matmul_rs_enqueue(self._handle, lhs.data_ptr(), rhs.data_ptr(), self._partial.data_ptr(), stream))
            if self._contraction_only:
                return self._partial
            if plan.output_dtype == "f32":
                dist.reduce_scatter_tensor(out, self._partial, group=self.mesh.group)
            else:
                reduced = torch.empty(plan.output_local_shape, dtype=torch.float32, device=self.mesh.device)
                dist.reduce_scatter_tensor(reduced, self._partial, group=self.mesh.group)
                out.copy_(reduced)
            return out
        _native.check(self._lib.cake_matmul_rs_enqueue(self._handle, lhs.data_ptr(), rhs.data_ptr(), out.data_ptr(), stream))
        return out

    # -- the two halves of a peer-to-peer call, for phase timing
    def push(self, lhs: torch.Tensor, rhs: torch.Tensor) -> None:
        if not self._p2p:
            raise ValueError("push / reduce exist only for the peer-to-peer strategies")
        stream = torch.cuda.current_stream(self.mesh.device).cuda_stream
        _native.check(self._lib.cake_matmul_rs_enqueue_push(self._handle, lhs.data_ptr(), rhs.data_ptr(), stream))

    def reduce(self, out: torch.Tensor) -> torch.Tensor:
        if not self._p2p:
            raise ValueError("push / reduce exist only for the peer-to-peer strategies")
        stream = torch.cuda.current_stream(self.mesh.device).cuda_stream
        _native.check(self._lib.cake_matmul_rs_enqueue_reduce(self._handle, out.data_ptr(), stream))
        return out

    # -- host call (the end-to-end path: host buffers in, host buffer out)
    def run_host(self, lhs: np.ndarray, rhs: np.ndarray, out: np.ndarray) -> np.ndarray:
        """lhs / rhs: uint16 arrays holding bf16 bits (or pinned torch-backed arrays), out: float32
        or uint16 array of the local output shape. Copies in, runs, copies out, synchronises."""
        if self._partial is not None:
            raise ValueError("run_host supports mesh_size 1 or the peer-to-peer strategies")
        stream = torch.cuda.current_stream(self.mesh.device).cuda_stream
        _native.check(self._lib.cake_matmul_rs_run_host(self._handle, lhs.ctypes.data, rhs.ctypes.data, out.ctypes.data, stream))
        return out

    def status(self) -> tuple[int, int, int, int]:
        """Synchronises the stream and returns (and clears) the device status word; raises
        CakeError(CAKE_ERR_TIMEOUT) if a bounded device-side wait ran out."""
        word = _native.CakeStatus()
        stream = torch.cuda.current_stream(self.mesh.device).cuda_stream
        _native.check(self._lib.cake_matmul_rs_status(self._handle, stream, ctypes.byref(word)))
        return (word.code, word.detail0, word.detail1, word.detail2)

    @property
    def launches_per_call(self) -> int:
        return int(self._lib.cake_matmul_rs_launches_per_enqueue(self._handle))

    def close(self) -> None:
        if self._handle:
            torch.cuda.synchronize(self.mesh.device)
            self._lib.cake_matmul_rs_destroy(self._handle)
            self._handle = None
        for buffer in (self._slots, self._flags):
            if buffer is not None:
                buffer.close()
        self._slots = self._flags = None

    def _check_operand(self, tensor: torch.Tensor, shape: tuple[int, int], role: str) -> None:
        if tensor.dtype != torch.bfloat16 or tuple(tensor.shape) != shape or not tensor.is_contiguous() or tensor.device != self.mesh.device:
            raise ValueError(
                f"{role} must be a contiguous bf16 tensor of shape {shape} on {self.mesh.device}, "
                f"got {tensor.dtype} {tuple(tensor.shape)} on {tensor.device}"
            )


_IMPLEMENTATION_TO_STRATEGY = {
    None: MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER,
    "nccl": MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER,
    "p2p_owner_push": MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE,
    "p2p_owner_push_bf16": MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT,
}
_PHYSICAL_MATMUL_OPS = (
    "tpu_schedule.alloc", "tpu_schedule.alloc", "tpu_schedule.alloc", "tpu_schedule.alloc",
    "tpu_schedule.semaphore_alloc", "tpu_schedule.semaphore_alloc", "tpu_schedule.semaphore_alloc",
    "tpu_schedule.dma_start", "tpu_schedule.dma_start", "tpu_schedule.dma_wait", "tpu_schedule.dma_wait",
    "tpu_schedule.mxu_matmul", "tpu_schedule.collective", "tpu_schedule.dma_start", "tpu_schedule.dma_wait",
    "tpu_schedule.yield",
)


def _hardware_tile(schedule_tile: int, supported: tuple[int, ...], op, reject, extent: int) -> int:
    """The schedule's tile is the block of the output one step produces; the reference's default is
    the whole local operand (src/tpu_cake/dialects/tpu_schedule.py:982-984). A schedule tile that is
    a hardware tile is used as is; a larger one is covered by the largest hardware tile (the CTA
    walks it in sub-tiles); the whole of an operand smaller than every hardware tile is one partial
    hardware tile; any other smaller tile cannot be expressed."""
    if schedule_tile in supported:
        return schedule_tile
    if schedule_tile > max(supported):
        return max(supported)
    if schedule_tile == extent:
        return min(supported)
    raise reject(f"sm_100a matmul tiles are {supported}, the schedule asks for {schedule_tile}", op)


def lower_physical_matmul_to_cuda(module, *, output_dtype: str = "f32") -> CudaMatmulRsPlan:
    """Physical matmul kernel -> CUDA plan; the counterpart of ``lower_physical_matmul_to_pallas``
    (src/tpu_cake/pallas_lowering.py:689-847). Accepts exactly the 16-operation kernel that
    ``lower_distributed_matmul`` emits, checks its dataflow (loads feed the matmul operands, the
    matmul accumulator feeds the collective, the collective result is stored to the output), bf16
    inputs with an f32 accumulator, a one-axis mesh, and reads shapes, shardings, tiles, scatter
    dimension and collective implementation off the operations. ``output_dtype`` selects the dtype
    the reduced output is stored in (the schedule's result is f32; "bf16" adds the final cast)."""
    from .ir import schedule_sha256

    module.verify()

    def reject(message: str, op=None) -> UnsupportedLoweringError:
        where = f": {op.name} at {op.location}" if op is not None else ""
        return UnsupportedLoweringError(f"{message}{where}")

    if len(module.ops) != 1 or module.ops[0].name != "tpu_schedule.kernel":
        raise reject("expected one physical kernel")
    kernel = module.ops[0]
    ops = kernel.body.ops
    if tuple(op.name for op in ops) != _PHYSICAL_MATMUL_OPS:
        unexpected = next((op for op, name in zip(ops, _PHYSICAL_MATMUL_OPS) if op.name != name), kernel)
        raise reject("kernel is not the physical matmul + reduce-scatter sequence", unexpected)
    lhs_alloc, rhs_alloc, partial_alloc, reduced_alloc = ops[0:4]
    load_lhs, load_rhs, wait_lhs, wait_rhs, matmul, collective, store, wait_store = ops[7:15]
    lhs_arg, rhs_arg, out_arg = kernel.body.args
    if load_lhs.operands[0] is not lhs_arg or load_lhs.operands[1] is not lhs_alloc.result:
        raise reject("the first DMA must load the lhs argument into the lhs tile", load_lhs)
    if load_rhs.operands[0] is not rhs_arg or load_rhs.operands[1] is not rhs_alloc.result:
        raise reject("the second DMA must load the rhs argument into the rhs tile", load_rhs)
    if wait_lhs.operands[0] is not load_lhs.result or wait_rhs.operands[0] is not load_rhs.result:
        raise reject("loads must be waited on in order", wait_lhs)
    if list(matmul.operands) != [lhs_alloc.result, rhs_alloc.result, partial_alloc.result]:
        raise reject("the matmul must contract the loaded tiles into the partial accumulator", matmul)
    if list(collective.operands) != [partial_alloc.result, reduced_alloc.result]:
        raise reject("the collective must reduce the partial accumulator into the reduced output", collective)
    if store.operands[0] is not reduced_alloc.result or store.operands[1] is not out_arg or wait_store.operands[0] is not store.result:
        raise reject("the reduced output must be stored to the output argument", store)
    lhs_type, rhs_type, partial_type, out_type = lhs_arg.type, rhs_arg.type, partial_alloc.result.type, out_arg.type
    if lhs_type.element_type != "bf16" or rhs_type.element_type != "bf16" or partial_type.element_type != "f32" or out_type.element_type != "f32":
        raise reject("the CUDA backend lowers bf16 inputs with f32 accumulation and an f32 schedule result", matmul)
    axes = kernel.properties["mesh_axis_names"]
    if len(axes) != 1:
        raise reject("the CUDA backend lowers a one-axis mesh", kernel)
    if collective.properties["kind"] != "reduce_scatter" or collective.properties["reducer"] != "sum":
        raise reject("the collective must be a sum reduce-scatter", collective)
    implementation = collective.properties.get("implementation")
    if implementation not in _IMPLEMENTATION_TO_STRATEGY:
        raise reject(f"unknown collective implementation {implementation}", collective)
    mesh_size = kernel.properties["mesh_axis_sizes"][0]
    return CudaMatmulRsPlan(
        name=kernel.properties["sym_name"],
        schedule_sha256=schedule_sha256(module),
        mesh_axis=axes[0],
        mesh_size=mesh_size,
        lhs_local_shape=tuple(lhs_type.shape),
        rhs_local_shape=tuple(rhs_type.shape),
        partial_local_shape=tuple(partial_type.shape),
        output_local_shape=tuple(out_type.shape),
        lhs_sharding=tuple(lhs_type.sharding),
        rhs_sharding=tuple(rhs_type.sharding),
        output_sharding=tuple(out_type.sharding),
        scatter_dimension=collective.properties["split_dimension"],
        tile_m=_hardware_tile(matmul.properties["tile_m"], SUPPORTED_TILE_M, matmul, reject, lhs_type.shape[0]),
        tile_k=matmul.properties["tile_k"],
        tile_n=_hardware_tile(matmul.properties["tile_n"], SUPPORTED_TILE_N, matmul, reject, rhs_type.shape[1]),
        collective_link_bandwidths=tuple((t.split(":")[0], int(t.split(":")[1])) for t in kernel.properties["topology"]),
        collective_implementation=_IMPLEMENTATION_TO_STRATEGY[implementation] if mesh_size > 1 else None,
        output_dtype=output_dtype,
    )


def _saved_source_constants(source_path: Path) -> dict[str, object]:
    try:
        tree = ast.parse(source_path.read_text(), filename=str(source_path))
    except SyntaxError as error:
        raise ValueError("SAVED_CUDA_SOURCE_INVALID") from error
    constants: dict[str, object] = {}
    for statement in tree.body:
        if isinstance(statement, ast.Assign) and len(statement.targets) == 1 and isinstance(statement.targets[0], ast.Name):
            try:
                constants[statement.targets[0].id] = ast.literal_eval(statement.value)
            except (ValueError, TypeError):
                continue
    return constants


def validate_saved_cuda_plan(physical_path: Path, source_path: Path, *, schedule_sha256: str, source_sha256: str) -> CudaMatmulRsPlan:
    """Replays a saved run's lowering: the counterpart of ``validate_saved_pallas_plan``
    (src/tpu_cake/pallas_lowering.py:850-947), with its error names and its order of checks.

    Both files must have the recorded hashes. The saved physical IR is parsed (it is the reference's
    canonical text; only text that prints back to the same bytes parses), verified and lowered to a
    plan again; that plan must agree with every constant of the saved source and render that source
    again exactly. The output dtype is the one thing the IR does not carry (the dialect's matmul
    accumulates and stores f32): it is read from the saved source. Returns the replayed plan."""
    from . import xdsl_text

    physical_text = physical_path.read_text()
    if text_sha256(physical_text) != schedule_sha256:
        raise ValueError("SAVED_PHYSICAL_IR_HASH_MISMATCH")
    source_text = source_path.read_text()
    if text_sha256(source_text) != source_sha256:
        raise ValueError("SAVED_CUDA_SOURCE_HASH_MISMATCH")
    constants = _saved_source_constants(source_path)
    output_line = next((line for line in source_text.splitlines() if line.startswith("output_local")), "")
    try:
        physical = xdsl_text.parse_reference_physical_kernel(physical_text)
        physical.verify()
        plan = lower_physical_matmul_to_cuda(physical, output_dtype="bf16" if "# bf16" in output_line else "f32")
    except Exception as error:
        raise ValueError("SAVED_PHYSICAL_IR_INVALID") from error
    try:
        mesh_axis, _ = constants["mesh"]
    except (KeyError, TypeError, ValueError) as error:
        raise ValueError("SAVED_CUDA_SOURCE_PLAN_MISMATCH") from error
    if plan.schedule_sha256 != schedule_sha256 or mesh_axis != plan.mesh_axis:
        raise ValueError("SAVED_CUDA_SOURCE_PLAN_MISMATCH")
    expected = {
        "schedule_sha256": schedule_sha256, "mesh": (plan.mesh_axis, plan.mesh_size), "lhs_local": plan.lhs_local_shape,
        "rhs_local": plan.rhs_local_shape, "partial_local": plan.partial_local_shape, "output_local": plan.output_local_shape,
        "scatter_dimension": plan.scatter_dimension, "tile": (plan.tile_m, plan.tile_k, plan.tile_n),
        "collective": None if plan.collective_implementation is None else plan.collective_implementation.value,
        "transport_dtype": plan.transport_dtype,
    }
    if any(constants.get(name) != value for name, value in expected.items()):
        raise ValueError("SAVED_CUDA_SOURCE_PLAN_MISMATCH")
    name = constants.get("name")
    if not isinstance(name, str):
        raise TypeError("SAVED_CUDA_SOURCE_PLAN_MISMATCH")
    rendering_plan = replace(plan, name=name)
    if rendering_plan.render_executable_source() != source_text:
        raise ValueError("SAVED_CUDA_RENDERING_MISMATCH")
    return rendering_plan
