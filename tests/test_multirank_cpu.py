"""World-size-2 host logic on CPU ranks (gloo): K sharding, the owner-major partial layout the
kernel writes for the library collective, and the byte exchange used for IPC handles."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _owner_major(partial: np.ndarray, world: int, scatter_dimension: int) -> np.ndarray:
    """[M, N] partial -> [W, out_rows, out_cols], the layout CAKE_RS_LOCAL_PARTIAL writes."""
    pieces = np.split(partial, world, axis=scatter_dimension)
    return np.ascontiguousarray(np.stack(pieces, axis=0))


def _rank_main(rank: int, world: int, port: int, scatter_dimension: int, results) -> None:
    sys.path.insert(0, str(ROOT))
    import __graft_entry__

    __graft_entry__.load_package()
    from oracle import matmul_rs as oracle
    from tpu_cake_b200 import workloads
    from tpu_cake_b200.mesh import ProcessMesh

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    try:
        mesh = ProcessMesh(axis="t", rank=rank, world=world, device=torch.device("cpu"), group=dist.group.WORLD)
        # The 64-byte handle exchange: every rank must see every rank's bytes in rank order.
        gathered = mesh.all_gather_bytes(bytes([rank]) * 64)
        assert gathered == [bytes([r]) * 64 for r in range(world)]

        lhs, rhs = workloads.distributed_matmul_inputs(world, 32, 64, 48)
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, world, rank)
        partial = lhs_r.astype(np.float32) @ rhs_r.astype(np.float32)  # stands in for the kernel
        staged = torch.from_numpy(_owner_major(partial, world, scatter_dimension))
        # Library collective on the owner-major partial: all-reduce + take own slice is the
        # reduce-scatter (gloo has no reduce_scatter_tensor).
        dist.all_reduce(staged)
        mine = staged[rank].numpy()
        expected = oracle.matmul_reduce_scatter(
            lhs.astype(np.float32), rhs.astype(np.float32), world=world, scatter_dimension=scatter_dimension
        )[rank]
        results[rank] = bool(np.allclose(mine, expected, atol=1e-3, rtol=1e-3)) and mine.shape == expected.shape
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scatter_dimension", (0, 1))
def test_two_cpu_ranks_reduce_scatter_and_handle_exchange(scatter_dimension):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), scatter_dimension, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def _decode_rank_main(rank: int, world: int, port: int, results) -> None:
    """KV-head sharding of the decode and the layout of the gathered outputs: rank r holds KV heads
    [r*Hkv/W, (r+1)*Hkv/W) of every page and the matching query heads, computes its heads (the oracle
    stands in for the kernel) and the outputs are all-gathered as [W][S][Hq/W][D]."""
    sys.path.insert(0, str(ROOT))
    import __graft_entry__

    __graft_entry__.load_package()
    from oracle import rpa as rpa_oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    try:
        generator = np.random.default_rng(5)  # same seed on every rank: replicated metadata and inputs
        lengths = np.array([9, 40, 17], dtype=np.int32)
        count, kv_heads, group, page_size, dim = 3, 4, 2, 8, 16
        q_heads = kv_heads * group
        pages_per = -(-lengths // page_size)
        pool = int(pages_per.sum()) + 2
        query = generator.normal(size=(count, q_heads, dim)).astype(np.float32)
        keys = generator.normal(size=(pool, page_size, kv_heads, dim)).astype(np.float32)
        values = generator.normal(size=(pool, page_size, kv_heads, dim)).astype(np.float32)
        table = np.zeros((count, int(pages_per.max())), dtype=np.int32)
        order = generator.permutation(pool)
        cursor = 0
        for s in range(count):
            table[s, : pages_per[s]] = order[cursor : cursor + pages_per[s]]
            cursor += int(pages_per[s])
        local_kv, local_q = kv_heads // world, q_heads // world
        heads = slice(rank * local_kv, (rank + 1) * local_kv)
        mine = rpa_oracle.rpa_separate(query[:, rank * local_q : (rank + 1) * local_q], keys[:, :, heads], values[:, :, heads],
                                       table, lengths)
        gathered = [torch.zeros((count, local_q, dim), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(np.ascontiguousarray(mine)))
        assembled = np.concatenate([piece.numpy() for piece in gathered], axis=1)  # [W][S][Hq/W][D] -> [S][Hq][D]
        expected = rpa_oracle.rpa_separate(query, keys, values, table, lengths)
        results[rank] = bool(np.allclose(assembled, expected, atol=1e-6, rtol=1e-6)) and assembled.shape == expected.shape
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_shard_decode_by_kv_head_and_gather():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_decode_rank_main, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
