"""Seeded synthetic inputs for the hot-path configurations.

Matmul inputs follow the reference's recipe exactly (src/tpu_cake/runner.py:439-456): one
generator seeded from the workload identity draws lhs then rhs as float32 normals, which are then
rounded to bfloat16. The attention configurations have no generator in the reference (its
workloads are fixed toy shapes, src/tpu_cake/workloads/inkling_rpa.py:76-84,413-468); the ones
here are seeded the same way (``semantic_seed(config, "inputs")``) and stand in for the serving
traces such kernels are normally measured on.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import ml_dtypes
import numpy as np

from .identity import semantic_seed, semantic_sha256, workload_rng

BF16 = np.dtype(ml_dtypes.bfloat16)


def distributed_matmul_workload_identity(mesh_size: int, m: int, k: int, n: int) -> str:
    return semantic_sha256("distributed-matmul-workload", str(mesh_size), str(m), str(k), str(n))


def distributed_matmul_inputs(mesh_size: int, m: int, k: int, n: int, *, scale: float = 1.0) -> tuple[np.ndarray, np.ndarray]:
    """Global lhs [m, k] and rhs [k, n] as bfloat16 arrays. ``scale`` = 1 is the reference recipe;
    the large configuration uses K**-0.5 so that outputs stay O(1)."""
    generator = workload_rng(distributed_matmul_workload_identity(mesh_size, m, k, n), "device-run", "attempt-0", "inputs")
    lhs = generator.normal(size=(m, k)).astype(np.float32)
    rhs = generator.normal(size=(k, n)).astype(np.float32)
    if scale != 1.0:
        lhs *= np.float32(scale)
        rhs *= np.float32(scale)
    return lhs.astype(BF16), rhs.astype(BF16)


def shard_matmul_inputs(lhs: np.ndarray, rhs: np.ndarray, mesh_size: int, rank: int) -> tuple[np.ndarray, np.ndarray]:
    """This rank's K block: lhs columns / rhs rows (src/tpu_cake/pallas_lowering.py:466-472)."""
    step = lhs.shape[1] // mesh_size
    return (
        np.ascontiguousarray(lhs[:, rank * step : (rank + 1) * step]),
        np.ascontiguousarray(rhs[rank * step : (rank + 1) * step, :]),
    )


@dataclass(frozen=True)
class DecodeConfig:
    """A pure-decode attention scenario: one query token per sequence."""

    name: str
    num_seqs: int
    q_heads: int
    kv_heads: int
    head_dim: int
    page_size: int
    total_pages: int
    min_kv_len: int
    max_kv_len: int
    length_distribution: str  # "uniform" or "log-uniform"

    @property
    def softmax_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)


DECODE_64 = DecodeConfig("rpa-decode-64seq", 64, 32, 8, 128, 16, 65536, 128, 8192, "uniform")
DECODE_SHARDED_256 = DecodeConfig("rpa-decode-sharded-256seq", 256, 64, 8, 128, 32, 262144, 1024, 32768, "log-uniform")


def decode_metadata(config: DecodeConfig) -> tuple[np.ndarray, np.ndarray]:
    """(kv_lens int32 [S], page_table int32 [S, max_pages]) from the config's seed. Pages are the
    first sum(ceil(len/page_size)) entries of a seeded permutation of the pool, dealt per sequence;
    unused table entries are 0."""
    generator = np.random.default_rng(semantic_seed(config.name, "inputs"))
    if config.length_distribution == "uniform":
        lengths = generator.integers(config.min_kv_len, config.max_kv_len + 1, size=config.num_seqs)
    elif config.length_distribution == "log-uniform":
        draws = generator.uniform(math.log(config.min_kv_len), math.log(config.max_kv_len), size=config.num_seqs)
        lengths = np.minimum(np.floor(np.exp(draws)).astype(np.int64), config.max_kv_len)
    else:
        raise ValueError(f"unknown length distribution {config.length_distribution}")
    lengths = lengths.astype(np.int32)
    pages_per_seq = -(-lengths.astype(np.int64) // config.page_size)
    needed = int(pages_per_seq.sum())
    if needed > config.total_pages:
        raise ValueError(f"{config.name}: needs {needed} pages, pool has {config.total_pages}")
    permutation = generator.permutation(config.total_pages)[:needed].astype(np.int32)
    max_pages = -(-config.max_kv_len // config.page_size)
    table = np.zeros((config.num_seqs, max_pages), dtype=np.int32)
    cursor = 0
    for s, count in enumerate(pages_per_seq):
        table[s, :count] = permutation[cursor : cursor + count]
        cursor += int(count)
    return lengths, table


def decode_algorithmic_bytes(kv_lens: np.ndarray, q_heads: int, kv_heads: int, head_dim: int, page_size: int, *, elem_bytes: int = 2) -> int:
    """Bytes a decode step must move: K and V of every valid token once per KV head, the query read
    and the output write, one page-table entry per page and one length per sequence. Page padding
    beyond kv_len is not counted."""
    lens = np.asarray(kv_lens, dtype=np.int64)
    kv = int(lens.sum()) * kv_heads * head_dim * elem_bytes * 2
    q_and_o = lens.size * q_heads * head_dim * elem_bytes * 2
    table = int((-(-lens // page_size)).sum()) * 4 + 8 * lens.size
    return kv + q_and_o + table


@dataclass(frozen=True)
class MixedConfig:
    """A ragged batch: decode sequences first (one query token each), then prefill sequences whose
    query tokens are appended after a prior context, in the order the reference's `distribution`
    triple expects (src/tpu_cake/rpa_owned_kernel.py:58-67)."""

    name: str
    decode_seqs: int
    prefill_seqs: int
    q_heads: int
    kv_heads: int
    head_dim: int
    page_size: int
    decode_kv: tuple[int, int]      # inclusive range of decode KV lengths
    prefill_q: tuple[int, int]      # inclusive range of prefill query lengths
    prefill_prior: tuple[int, int]  # inclusive range of the context already cached

    @property
    def softmax_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)


MIXED_8_120 = MixedConfig("rpa-mixed-8prefill-120decode", 120, 8, 32, 8, 128, 16, (256, 32768), (512, 2048), (0, 4096))


@dataclass(frozen=True)
class MixedMetadata:
    kv_lens: np.ndarray        # int32 [S]
    cu_q_lens: np.ndarray      # int32 [S+1]
    cu_kv_lens: np.ndarray     # int32 [S+1], page-aligned cumulative lengths
    page_indices: np.ndarray   # int32 flat; sequence s starts at cu_kv_lens[s] // page_size
    distribution: np.ndarray   # int32 [3]: (decode end, prefill end, mixed end)
    total_pages: int

    @property
    def num_tokens(self) -> int:
        return int(self.cu_q_lens[-1])


def mixed_metadata(config: MixedConfig, *, spare_pages: int = 64) -> MixedMetadata:
    """Seeded ragged metadata. cu_kv_lens is the cumulative sum of page-aligned lengths, the flat
    page-index convention of the reference's preflight (src/tpu_cake/rpa_lowering.py:96-101); pages
    are a seeded permutation of a pool just large enough (plus `spare_pages`)."""
    generator = np.random.default_rng(semantic_seed(config.name, "inputs"))
    decode_kv = generator.integers(config.decode_kv[0], config.decode_kv[1] + 1, size=config.decode_seqs)
    prefill_q = generator.integers(config.prefill_q[0], config.prefill_q[1] + 1, size=config.prefill_seqs)
    prior = generator.integers(config.prefill_prior[0], config.prefill_prior[1] + 1, size=config.prefill_seqs)
    kv_lens = np.concatenate([decode_kv, prior + prefill_q]).astype(np.int32)
    q_lens = np.concatenate([np.ones(config.decode_seqs, dtype=np.int64), prefill_q.astype(np.int64)])
    return ragged_metadata(kv_lens, q_lens, config.page_size, config.decode_seqs, generator, spare_pages=spare_pages)


def ragged_metadata(kv_lens, q_lens, page_size: int, decode_seqs: int, generator, *, spare_pages: int = 8) -> MixedMetadata:
    kv_lens = np.asarray(kv_lens, dtype=np.int32)
    q_lens = np.asarray(q_lens, dtype=np.int64)
    pages_per_seq = -(-kv_lens.astype(np.int64) // page_size)
    total_pages = int(pages_per_seq.sum()) + spare_pages
    cu_q = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    cu_kv = np.concatenate([[0], np.cumsum(pages_per_seq * page_size)]).astype(np.int32)
    page_indices = generator.permutation(total_pages)[: int(pages_per_seq.sum())].astype(np.int32)
    count = len(kv_lens)
    distribution = np.array([decode_seqs, count, count], dtype=np.int32)
    return MixedMetadata(kv_lens, cu_q, cu_kv, page_indices, distribution, total_pages)


def mixed_algorithmic_work(meta: MixedMetadata, q_heads: int, kv_heads: int, head_dim: int, *, elem_bytes: int = 2) -> dict:
    """The two bounds of a mixed batch: HBM bytes (every valid cached token of every KV head read
    once per sequence, queries read, outputs written, table entries and lengths read) and attention
    FLOPs 4 * head_dim * q_heads * sum over query rows of the positions the row sees."""
    kv = meta.kv_lens.astype(np.int64)
    q_lens = np.diff(meta.cu_q_lens.astype(np.int64))
    token_bytes = int(kv.sum()) * kv_heads * head_dim * elem_bytes * 2
    query_bytes = int(q_lens.sum()) * q_heads * head_dim * elem_bytes * 2
    table_bytes = int(len(meta.page_indices)) * 4 + 8 * len(kv)
    visible = q_lens * kv - q_lens * (q_lens - 1) // 2  # row i of q rows sees kv - q + i + 1 positions
    decode = q_lens == 1
    return {
        "bytes": token_bytes + query_bytes + table_bytes,
        "flops": 4 * head_dim * q_heads * int(visible.sum()),
        "decode_bytes": int(kv[decode].sum()) * kv_heads * head_dim * elem_bytes * 2,
        "prefill_flops": 4 * head_dim * q_heads * int(visible[~decode].sum()),
        "query_tokens": int(q_lens.sum()),
    }


def paged_attention_schedule(*, batch: int = 4, q_heads: int = 4, kv_heads: int = 4, head_dim: int = 32, pages: int = 32,
                             page_size: int = 16, max_pages: int = 8, target: str = "b200"):
    """Physical kernel around the prototype decode op: stage the query and the bias on chip, run
    ``tpu_schedule.ragged_paged_attention``, copy the output back (the shape of
    src/tpu_cake/workloads/inkling_rpa.py:87-142, whose defaults these are)."""
    from .dialects import KernelBuilder, buffer

    external = {"memory": "hbm", "ownership": "external", "lifetime": (0, 4)}
    extent = max_pages * page_size
    inputs = (
        buffer((batch, q_heads, head_dim), "B H D".split(), "bf16", **external),
        buffer((pages, page_size, kv_heads, head_dim), "P S H D".split(), "bf16", **external),
        buffer((pages, page_size, kv_heads, head_dim), "P S H D".split(), "bf16", **external),
        buffer((batch, max_pages), "B MP".split(), "i32", **external),
        buffer((batch,), ("B",), "i32", **external),
        buffer((q_heads, extent), "H L".split(), "bf16", **external),
        buffer((batch, q_heads, head_dim), "B H D".split(), "bf16", **external),
    )
    builder = KernelBuilder("inkling_rpa_decode", target, inputs, vmem_capacity_bytes=160 << 30, smem_capacity_bytes=227 << 10,
                            mesh={}, interconnect_bandwidth_bytes_per_second={})
    query = builder.alloc(buffer((batch, q_heads, head_dim), "B H D".split(), "bf16", memory="vmem", lifetime=(0, 2)), "query_tile")
    bias = builder.alloc(buffer((q_heads, extent), "H L".split(), "bf16", memory="vmem", lifetime=(0, 2)), "relative_bias")
    output = builder.alloc(buffer((batch, q_heads, head_dim), "B H D".split(), "bf16", memory="vmem", lifetime=(2, 4)), "attention_output")
    semaphores = [builder.semaphore() for _ in range(3)]
    query_dma = builder.dma_start(builder.inputs[0], query, semaphores[0], stage=0)
    bias_dma = builder.dma_start(builder.inputs[5], bias, semaphores[1], stage=0)
    builder.dma_wait(query_dma, stage=1)
    builder.dma_wait(bias_dma, stage=1)
    builder.ragged_paged_attention(query, builder.inputs[1], builder.inputs[2], builder.inputs[3], builder.inputs[4], bias, output,
                                   stage=2, query_block_size=1, kv_block_size=min(8, page_size))
    output_dma = builder.dma_start(output, builder.inputs[6], semaphores[2], stage=3)
    builder.dma_wait(output_dma, stage=4)
    return builder.module()


def fused_rpa_schedule(*, tokens: int, sequences: int | None = None, q_heads: int, kv_heads: int, head_dim: int, pages: int,
                       page_size: int, page_indices: int, relative_dim: int = 16, bias_extent: int = 512, softmax_scale: str | None = None,
                       execution_authority: str | None = None, target: str = "b200", mesh: dict[str, int] | None = None):
    """Physical kernel holding one ``tpu_schedule.fused_ragged_paged_attention`` over external HBM
    buffers, output and cache aliased to the query and cache inputs (the contract of
    src/tpu_cake/dialects/tpu_schedule.py:2107-2349). ``sequences`` below ``tokens`` describes a ragged
    batch and needs this backend's execution authority."""
    from .dialects import FUSED_RPA_CUDA_AUTHORITY, FUSED_RPA_UPSTREAM_AUTHORITY, KernelBuilder, buffer

    sequences = tokens if sequences is None else sequences
    padded = -(-head_dim // 128) * 128
    external = {"memory": "hbm", "ownership": "external", "lifetime": (0, 0)}
    inputs = (
        buffer((tokens, q_heads, head_dim), "T H D".split(), "bf16", **external),
        buffer((tokens, kv_heads, head_dim), "T KH D".split(), "bf16", **external),
        buffer((tokens, kv_heads, head_dim), "T KH D".split(), "bf16", **external),
        buffer((pages, page_size, kv_heads, 2, padded), "P S KH C DP".split(), "bf16", **external),
        buffer((sequences,), ("N",), "i32", **external),
        buffer((page_indices,), ("PI",), "i32", **external),
        buffer((sequences + 1,), ("N1",), "i32", **external),
        buffer((sequences + 1,), ("N1",), "i32", **external),
        buffer((3,), ("X",), "i32", **external),
        buffer((tokens, q_heads, relative_dim), "T H R".split(), "bf16", **external),
        buffer((relative_dim, bias_extent), "R E".split(), "bf16", **external),
    )
    mesh = dict(mesh or {})
    builder = KernelBuilder("inkling_fused_rpa", target, inputs, vmem_capacity_bytes=160 << 30, smem_capacity_bytes=227 << 10,
                            mesh=mesh, interconnect_bandwidth_bytes_per_second={axis: 700_000_000_000 for axis in mesh})
    if execution_authority is None:
        execution_authority = FUSED_RPA_UPSTREAM_AUTHORITY if sequences == tokens and softmax_scale is None else FUSED_RPA_CUDA_AUTHORITY
    if softmax_scale is None:
        from decimal import Decimal

        softmax_scale = str(Decimal(1) / Decimal(head_dim))
    kv_block = max(128, page_size)
    builder.fused_ragged_paged_attention(
        (*builder.inputs, builder.inputs[0], builder.inputs[3]), stage=0, softmax_scale=softmax_scale, kv_block_size=kv_block,
        kv_cluster_size=kv_block, execution_authority=execution_authority,
    )
    return builder.module()


# The toy fused-RPA experiment of the reference (src/tpu_cake/workloads/inkling_rpa.py:413-468):
# 4 decode sequences of 1, 17, 33 and 49 tokens, 4 query heads over 2 KV heads of dimension 32
# (padded to 128 in the cache), 32 pages of 16 tokens dealt out in this fixed order.
FUSED_RPA_PAGE_ORDER = (7, 2, 19, 4, 25, 1, 16, 9, 30, 12, 0, 5, 8, 11, 14, 17, 20, 23, 26, 29, 3, 6, 10, 13, 15, 18, 21, 22, 24, 27, 28, 31)
FUSED_RPA_KV_LENGTHS = (1, 17, 33, 49)
FUSED_RPA_BENCHMARK_PROTOCOL = {"seed": 97, "warmup_iterations": 5, "measured_iterations": 50}  # rpa_runner.py:82-98


def inkling_fused_rpa_inputs(seed: int = 0) -> tuple[np.ndarray, ...]:
    """The 11 inputs of the toy fused-RPA experiment as host arrays (bfloat16 through ml_dtypes,
    int32 metadata), drawn exactly as the reference draws them: one ``default_rng(seed)`` normal
    stream in the order queries, keys, values, cache (scale 0.25), relative states and projection
    (scale 0.4), each rounded float32 -> bfloat16."""
    import ml_dtypes

    generator = np.random.default_rng(seed)

    def bf16(shape, scale=1.0):
        return generator.normal(scale=scale, size=shape).astype(np.float32).astype(ml_dtypes.bfloat16)

    queries, keys, values = bf16((4, 4, 32)), bf16((4, 2, 32)), bf16((4, 2, 32))
    cache = bf16((32, 16, 2, 2, 128), scale=0.25)
    lengths = np.asarray(FUSED_RPA_KV_LENGTHS, dtype=np.int32)
    aligned = -(-lengths.astype(np.int64) // 16) * 16
    return (
        queries, keys, values, cache, lengths, np.asarray(FUSED_RPA_PAGE_ORDER, dtype=np.int32), np.arange(5, dtype=np.int32),
        np.concatenate(([0], np.cumsum(aligned))).astype(np.int32), np.full((3,), 4, dtype=np.int32),
        bf16((4, 4, 16), scale=0.4), bf16((16, 128), scale=0.4),
    )


def inkling_fused_rpa_schedule():
    """The physical kernel of the toy fused-RPA experiment (strict form: scale 1/head_dim, one query
    token per sequence)."""
    return fused_rpa_schedule(tokens=4, q_heads=4, kv_heads=2, head_dim=32, pages=32, page_size=16, page_indices=32,
                              relative_dim=16, bias_extent=128)


def inkling_sharded_rpa_schedule(*, data: int = 2, tensor: int = 4):
    """The local kernel of the data x tensor sharded fused decode, on a mesh of ``data`` x ``tensor``
    positions: the shapes of one position's shard (src/tpu_cake/workloads/inkling_rpa.py:198-228 --
    4 sequences, 8 / 4 local heads of dimension 128, 3712 local pages of one token, 8192 page slots,
    relative dimension 16 over an extent of 512)."""
    return fused_rpa_schedule(tokens=4, q_heads=8, kv_heads=4, head_dim=128, pages=3712, page_size=1, page_indices=8192,
                              relative_dim=16, bias_extent=512, mesh={"data": data, "tensor": tensor})


INKLING_SHARDED_RPA_LOCAL_CONTEXTS = (128, 512, 1024, 2048)


def inkling_sharded_fused_rpa_inputs(seed: int) -> tuple[np.ndarray, ...]:
    """The 11 GLOBAL inputs of the 2 x 4 sharded surface as host arrays, drawn as the reference draws
    them (src/tpu_cake/workloads/inkling_rpa.py:595-637): one ``default_rng(seed)`` normal stream in
    the order queries [8, 32, 128], keys and values [8, 16, 128], cache [7424, 1, 16, 2, 128]
    (scale 0.25), relative states [8, 32, 16] and projection [16, 512] (scale 0.4), each rounded
    float32 -> bfloat16; per data block four sequences of 128 / 512 / 1024 / 2048 tokens on pages of
    one token numbered inside the block, 8192 page slots."""
    import ml_dtypes

    generator = np.random.default_rng(seed)
    data, tensor, local_tokens, local_q, local_kv = 2, 4, 4, 8, 4
    contexts = INKLING_SHARDED_RPA_LOCAL_CONTEXTS
    local_pages = sum(contexts)

    def bf16(shape, scale=1.0):
        return generator.normal(scale=scale, size=shape).astype(np.float32).astype(ml_dtypes.bfloat16)

    page_indices = np.zeros((local_tokens * max(contexts),), dtype=np.int32)
    page_indices[:local_pages] = np.arange(local_pages, dtype=np.int32)
    cumulative_kv = np.concatenate((np.zeros((1,), dtype=np.int32), np.cumsum(contexts, dtype=np.int32)))
    return (
        bf16((data * local_tokens, tensor * local_q, 128)), bf16((data * local_tokens, tensor * local_kv, 128)),
        bf16((data * local_tokens, tensor * local_kv, 128)), bf16((data * local_pages, 1, tensor * local_kv, 2, 128), scale=0.25),
        np.tile(np.asarray(contexts, dtype=np.int32), data), np.tile(page_indices, data), np.tile(np.arange(local_tokens + 1, dtype=np.int32), data),
        np.tile(cumulative_kv, data), np.tile(np.full((3,), local_tokens, dtype=np.int32), data),
        bf16((data * local_tokens, tensor * local_q, 16), scale=0.4), bf16((16, 512), scale=0.4),
    )


def distributed_matmul_schedule(*, mesh_size: int = 4, m: int = 16, k: int = 32, n: int = 16, scatter_dimension: str = "N"):
    """The logical program ``einsum_local(lhs[M, K@t], rhs[K@t, N]) -> f32[M, N]{pending t:sum}``
    followed by ``reduce_scatter(axes=t, dim=scatter_dimension)``
    (src/tpu_cake/workloads/distributed_matmul.py:22-46; the reference scatters "N")."""
    from .dialects import DistributedProgramBuilder, tensor
    from .ir import SourceLocation

    if scatter_dimension not in ("M", "N"):
        raise ValueError("scatter_dimension must be 'M' or 'N'")
    lhs = tensor("bf16", (("M", m), ("K", k)), sharding={"K": ("t",)})
    rhs = tensor("bf16", (("K", k), ("N", n)), sharding={"K": ("t",)})
    builder = DistributedProgramBuilder("distributed_matmul", {"t": mesh_size}, (lhs, rhs))
    partial = builder.einsum_local(
        builder.inputs[0], builder.inputs[1], tensor("f32", (("M", m), ("N", n)), pending_reductions={"t": "sum"}),
        contracting_dimension="K", source=SourceLocation("tpu_cake_b200/workloads.py", 1, 1),
    )
    result = builder.reduce_scatter(
        partial, tensor("f32", (("M", m), ("N", n)), sharding={scatter_dimension: ("t",)}), axes=("t",),
        scatter_dimensions=(scatter_dimension,), source=SourceLocation("tpu_cake_b200/workloads.py", 2, 1),
    )
    return builder.module(result)
