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

import ctypes
from dataclasses import dataclass, field
from enum import StrEnum

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

    receive_slot_bytes: int  # 2 parities x W sources x local output, in the transport dtype
    arrival_counter_bytes: int
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
        return P2pCollectiveResources(
            receive_slot_bytes=2 * self.mesh_size * local,
            arrival_counter_bytes=8 * _native.CAKE_MAX_WORLD,
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

    def __init__(self, plan: CudaMatmulRsPlan, mesh: ProcessMesh, *, contraction_only: bool = False):
        """``contraction_only`` builds the same contraction with the same tiles and transport dtype
        but leaves the partial in local memory (owner-major) and runs no collective: the
        "pushes disabled" twin used to measure how much communication time is exposed."""
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
            reserved=0,
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
