"""One-process-per-GPU mesh: rank bookkeeping and the exchange of CUDA IPC handles.

The reference runs its 8 devices from one JAX process (``jax.shard_map`` over a ``Mesh``,
src/tpu_cake/pallas_lowering.py:417-476). Here every mesh position is its own process driving
its own GPU; ``torch.distributed`` (NCCL) is the control plane that ships 64-byte IPC handles
and runs the library collectives of the ``nccl_reduce_scatter`` strategy.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from . import _native


@dataclass
class ProcessMesh:
    """This process's position on a one-axis mesh."""

    axis: str
    rank: int
    world: int
    device: torch.device
    group: object | None = None  # torch.distributed process group (None when world == 1)

    @classmethod
    def single(cls, axis: str = "t", device: int | None = None) -> "ProcessMesh":
        index = torch.cuda.current_device() if device is None else device
        return cls(axis=axis, rank=0, world=1, device=torch.device("cuda", index))

    @classmethod
    def from_environment(cls, axis: str = "t") -> "ProcessMesh":
        """Reads RANK / LOCAL_RANK / WORLD_SIZE (torchrun) and initialises NCCL when world > 1."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        if world == 1:
            return cls(axis=axis, rank=0, world=1, device=device)
        import torch.distributed as dist

        if not dist.is_initialized():
            dist.init_process_group(backend="nccl", device_id=device)
        return cls(axis=axis, rank=rank, world=world, device=device, group=dist.group.WORLD)

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            if self.device.type == "cuda":
                dist.barrier(group=self.group, device_ids=[self.device.index])
            else:
                dist.barrier(group=self.group)

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        """Every rank contributes the same number of bytes; returns all contributions by rank."""
        if self.world == 1:
            return [payload]
        import torch.distributed as dist

        mine = torch.tensor(list(payload), dtype=torch.uint8, device=self.device)
        gathered = torch.empty(self.world * len(payload), dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(gathered, mine, group=self.group)
        flat = bytes(gathered.cpu().tolist())
        return [flat[r * len(payload) : (r + 1) * len(payload)] for r in range(self.world)]


class SymmetricBuffer:
    """A zero-filled device allocation of the same size on every rank, with every peer's copy
    mapped into this process through CUDA IPC. ``pointers[r]`` is rank r's buffer as seen here."""

    def __init__(self, mesh: ProcessMesh, nbytes: int):
        lib = _native.load()
        self._lib = lib
        self.mesh = mesh
        self.nbytes = nbytes
        own = ctypes.c_void_p()
        _native.check(lib.cake_symm_alloc(nbytes, ctypes.byref(own)))
        self.own = own.value
        self.pointers: list[int] = [0] * mesh.world
        self.pointers[mesh.rank] = self.own
        self._opened: list[int] = []
        if mesh.world > 1:
            handle = ctypes.create_string_buffer(64)
            _native.check(lib.cake_ipc_export(self.own, handle))
            handles = mesh.all_gather_bytes(handle.raw)
            for r, raw in enumerate(handles):
                if r == mesh.rank:
                    continue
                mapped = ctypes.c_void_p()
                _native.check(lib.cake_ipc_open(raw, ctypes.byref(mapped)))
                self.pointers[r] = mapped.value
                self._opened.append(mapped.value)
            mesh.barrier()

    def as_tensor(self, dtype: torch.dtype, shape: tuple[int, ...]) -> torch.Tensor:
        """A torch view of this rank's own allocation (no copy), through the CUDA array interface."""

        class _Exported:
            pass

        exported = _Exported()
        exported.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.own, False), "version": 2}
        flat = torch.as_tensor(exported, device=self.mesh.device)
        return flat.view(dtype).view(shape)

    def close(self) -> None:
        for pointer in self._opened:
            self._lib.cake_ipc_close(pointer)
        self._opened = []
        if self.own:
            self.mesh.barrier()
            self._lib.cake_symm_free(self.own)
            self.own = 0
