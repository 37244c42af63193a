"""GPU parity of the ragged-paged-attention decode kernels against the CPU oracle, through the
C ABI. Tolerance (the build's contract for bf16 outputs of f32-accumulated attention):
max-abs <= 2e-2 and relative-L2 <= 1e-2; page-table and length indexing must be exact, which the
edge cases below check by construction (poisoned unused pages, permuted tables, boundary lengths)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import matmul_rs as metrics
from oracle import rpa as oracle
from tests.helpers import BF16, bits_to_bf16, to_device, torch_to_bf16
from tests.test_oracle_golden import fused_inputs
from tpu_cake_b200 import rpa_cuda_lowering, workloads

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-2


def assert_close(actual: np.ndarray, expected: np.ndarray) -> None:
    assert np.isfinite(actual).all()
    assert metrics.max_abs_error(actual, expected) <= MAX_ABS
    assert metrics.relative_l2_error(actual, expected) <= REL_L2


def fused_plan(inputs, **overrides) -> rpa_cuda_lowering.CudaFusedRpaPlan:
    shapes = [None if value is None else tuple(np.asarray(value).shape) for value in inputs]
    fields = dict(
        name="inkling_fused_rpa", schedule_sha256="0" * 64, query_shape=shapes[0], key_shape=shapes[1], value_shape=shapes[2],
        fused_cache_shape=shapes[3], kv_lengths_shape=shapes[4], page_indices_shape=shapes[5],
        cumulative_query_lengths_shape=shapes[6], cumulative_kv_lengths_shape=shapes[7], distribution_shape=shapes[8],
        relative_states_shape=shapes[9], relative_projection_shape=shapes[10], output_shape=shapes[0],
        softmax_scale=1.0 / shapes[0][2],
    )
    fields.update(overrides)
    return rpa_cuda_lowering.CudaFusedRpaPlan(**fields)


def run_fused(plan, inputs, device):
    executable = plan.build(device)
    try:
        device_inputs = tuple(None if value is None else to_device(np.asarray(value), device) for value in inputs)
        output, cache = plan.run_preflighted(executable, *device_inputs)
        assert executable.status() == (0, 0, 0, 0)
        return torch_to_bf16(output), torch_to_bf16(cache)
    finally:
        executable.close()


@pytest.mark.parametrize("seed", (0, 7))
def test_reference_fused_vectors(cuda_device, golden_dir, seed):
    """The reference's own toy inputs (head_dim 32 padded to 128, page 16, flat page indices,
    relative bias, scale 1/head_dim): output within its allclose(0.02, 0.02), cache bit-exact."""
    vectors = np.load(golden_dir / "rpa_reference_vectors.npz")
    inputs = fused_inputs(vectors, seed)
    output, cache = run_fused(fused_plan(inputs), inputs, cuda_device)
    expected = bits_to_bf16(vectors[f"fused/seed{seed}/output_bf16_bits"]).astype(np.float32)
    assert np.allclose(output.astype(np.float32), expected, rtol=0.02, atol=0.02)
    assert_close(output.astype(np.float32), expected)
    np.testing.assert_array_equal(cache.view(np.uint16), vectors[f"fused/seed{seed}/updated_cache_bf16_bits"])


def test_kernel_is_told_apart_from_every_oracle_mutation(cuda_device, golden_dir):
    vectors = np.load(golden_dir / "rpa_reference_vectors.npz")
    inputs = fused_inputs(vectors, 0)
    output, cache = run_fused(fused_plan(inputs), inputs, cuda_device)
    good_cache = vectors["fused/seed0/updated_cache_bf16_bits"]
    for mutation in oracle.MUTATIONS:
        wrong = bits_to_bf16(vectors[f"fused/seed0/mutation/{mutation}/output_bf16_bits"]).astype(np.float32)
        wrong_cache_equal = bool(vectors[f"fused/seed0/mutation/{mutation}/cache_equal"])
        passes = np.allclose(output.astype(np.float32), wrong, rtol=0.02, atol=0.02) and wrong_cache_equal
        assert not passes, mutation
    np.testing.assert_array_equal(cache.view(np.uint16), good_cache)


def random_case(seed, *, num_seqs, q_heads, kv_heads, page_size, lengths, pool_pages, poison=True):
    generator = np.random.default_rng(seed)
    dim = 128
    query = generator.normal(size=(num_seqs, q_heads, dim)).astype(np.float32).astype(BF16)
    key_cache = generator.normal(size=(pool_pages, page_size, kv_heads, dim)).astype(np.float32).astype(BF16)
    value_cache = generator.normal(size=(pool_pages, page_size, kv_heads, dim)).astype(np.float32).astype(BF16)
    lengths = np.asarray(lengths, dtype=np.int32)
    pages_per_seq = -(-lengths.astype(np.int64) // page_size)
    max_pages = int(pages_per_seq.max())
    permutation = generator.permutation(pool_pages)
    table = np.zeros((num_seqs, max_pages), dtype=np.int32)
    cursor = 0
    used = np.zeros(pool_pages, dtype=bool)
    for s in range(num_seqs):
        count = int(pages_per_seq[s])
        table[s, :count] = permutation[cursor : cursor + count]
        used[permutation[cursor : cursor + count]] = True
        cursor += count
    assert cursor <= pool_pages
    if poison:
        # Pages no sequence owns, and token slots past each sequence's length, hold NaN: any read
        # of them that reaches the arithmetic shows up in the output.
        key_cache[~used] = np.nan
        value_cache[~used] = np.nan
        for s in range(num_seqs):
            tail = int(lengths[s]) % page_size
            if tail:
                last = table[s, int(pages_per_seq[s]) - 1]
                key_cache[last, tail:] = np.nan
                value_cache[last, tail:] = np.nan
    return query, key_cache, value_cache, table, lengths


def run_separate(case, device, *, fused, chunk=0, bias=None, scale=None):
    query, key_cache, value_cache, table, lengths = case
    dim = query.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(dim)
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name="paged", schedule_sha256="0" * 64, query_shape=query.shape, cache_shape=key_cache.shape,
        page_table_shape=table.shape, bias_shape=None if bias is None else bias.shape, softmax_scale=scale,
        kv_chunk_tokens=chunk, cache_layout="fused" if fused else "separate",
    )
    executable = plan.build(device)
    try:
        if fused:
            caches = (to_device(oracle.fused_cache_from_separate(key_cache, value_cache), device), None)
        else:
            caches = (to_device(key_cache, device), to_device(value_cache, device))
        out = plan.invoke(executable, to_device(query, device), caches[0], caches[1], to_device(table, device),
                          to_device(lengths, device), None if bias is None else to_device(bias, device))
        assert executable.status() == (0, 0, 0, 0)
        again = plan.invoke(executable, to_device(query, device), caches[0], caches[1], to_device(table, device),
                            to_device(lengths, device), None if bias is None else to_device(bias, device))
        torch.cuda.synchronize(device)
        assert torch.equal(out.view(torch.uint16), again.view(torch.uint16)), "repeat run must be bit-identical"
        return torch_to_bf16(out).astype(np.float32)
    finally:
        executable.close()


def expected_for(case, *, bias=None, scale=None):
    query, key_cache, value_cache, table, lengths = case
    scale = scale if scale is not None else 1.0 / math.sqrt(query.shape[2])
    # NaN poison lives only where the oracle never reads (it slices to the sequence length).
    return oracle.rpa_separate(query, key_cache, value_cache, table, lengths, bias, scale=scale)


@pytest.mark.parametrize("fused", (False, True))
@pytest.mark.parametrize(
    "q_heads, kv_heads, page_size, lengths",
    [
        (4, 4, 16, [1, 15, 16, 17]),            # one query head per KV head; page_size - 1, == , + 1
        (8, 2, 16, [31, 32, 33, 511, 512, 513]),  # stage (32) and chunk (512) boundaries
        (32, 8, 16, [128, 700, 2047, 3000]),     # the decode configuration's head layout
        (64, 8, 32, [1024, 33, 1500, 2500]),     # the sharded configuration's head layout
        (8, 1, 8, [7, 8, 9, 100]),               # 8 query heads on one KV head
        (8, 4, 1, [1, 2, 31, 33, 200]),          # one token per page (the reference surface's page size)
        (8, 4, 2, [3, 64, 65]),
        (8, 4, 4, [5, 127, 130]),
    ],
)
def test_decode_edge_cases(cuda_device, fused, q_heads, kv_heads, page_size, lengths):
    pool = sum(-(-length // page_size) for length in lengths) + 7
    case = random_case(11, num_seqs=len(lengths), q_heads=q_heads, kv_heads=kv_heads, page_size=page_size,
                       lengths=lengths, pool_pages=pool)
    actual = run_separate(case, cuda_device, fused=fused)
    assert_close(actual, expected_for(case))


@pytest.mark.parametrize("chunk", (32, 64, 256, 1024))
def test_split_kv_chunk_sizes_agree(cuda_device, chunk):
    case = random_case(5, num_seqs=3, q_heads=8, kv_heads=2, page_size=16, lengths=[1000, 31, 257], pool_pages=100)
    actual = run_separate(case, cuda_device, fused=True, chunk=chunk)
    assert_close(actual, expected_for(case))


def test_dense_bias_and_reference_scale(cuda_device):
    """The prototype op's semantics: scale 1/head_dim and a dense bias indexed by key position
    (the reference's separate-cache oracle)."""
    case = random_case(3, num_seqs=4, q_heads=8, kv_heads=2, page_size=16, lengths=[17, 33, 65, 127], pool_pages=32)
    bias = np.random.default_rng(9).normal(scale=0.5, size=(8, 128)).astype(np.float32)
    actual = run_separate(case, cuda_device, fused=False, bias=bias, scale=1.0 / 128)
    assert_close(actual, expected_for(case, bias=bias, scale=1.0 / 128))


def test_batch_permutation_invariance_and_state_isolation(cuda_device):
    """Reordering sequences reorders outputs and nothing else; changing one sequence's pages leaves
    every other sequence's output bit-identical (the reference's semantic properties)."""
    lengths = [100, 37, 513, 64, 1]
    case = random_case(21, num_seqs=5, q_heads=8, kv_heads=2, page_size=16, lengths=lengths, pool_pages=80, poison=False)
    base = run_separate(case, cuda_device, fused=True)
    order = np.array([3, 0, 4, 2, 1])
    query, key_cache, value_cache, table, lens = case
    permuted = (query[order], key_cache, value_cache, table[order], lens[order])
    np.testing.assert_array_equal(run_separate(permuted, cuda_device, fused=True), base[order])
    changed_key = key_cache.copy()
    changed_key[table[2, 0]] = changed_key[table[2, 0]] * np.asarray(-1.0, dtype=BF16)
    other = run_separate((query, changed_key, value_cache, table, lens), cuda_device, fused=True)
    for s in (0, 1, 3, 4):
        np.testing.assert_array_equal(other[s], base[s])
    assert not np.array_equal(other[2], base[2])


def test_output_may_alias_query(cuda_device):
    case = random_case(2, num_seqs=3, q_heads=8, kv_heads=2, page_size=16, lengths=[40, 600, 1100], pool_pages=120)
    query, key_cache, value_cache, table, lengths = case
    expected = expected_for(case)
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name="alias", schedule_sha256="0" * 64, query_shape=query.shape, cache_shape=key_cache.shape,
        page_table_shape=table.shape, bias_shape=None, softmax_scale=1.0 / math.sqrt(128),
    )
    executable = plan.build(cuda_device)
    buffer = to_device(query, cuda_device)
    plan.invoke(executable, buffer, to_device(key_cache, cuda_device), to_device(value_cache, cuda_device),
                to_device(table, cuda_device), to_device(lengths, cuda_device), out=buffer)
    assert executable.status() == (0, 0, 0, 0)
    assert_close(torch_to_bf16(buffer).astype(np.float32), expected)
    executable.close()


def test_out_of_range_page_is_reported_not_faulted(cuda_device):
    case = random_case(4, num_seqs=2, q_heads=8, kv_heads=2, page_size=16, lengths=[40, 50], pool_pages=16, poison=False)
    query, key_cache, value_cache, table, lengths = case
    table = table.copy()
    table[1, 1] = 10_000
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name="bad-page", schedule_sha256="0" * 64, query_shape=query.shape, cache_shape=key_cache.shape,
        page_table_shape=table.shape, bias_shape=None, softmax_scale=0.1,
    )
    executable = plan.build(cuda_device)
    plan.invoke(executable, to_device(query, cuda_device), to_device(key_cache, cuda_device), to_device(value_cache, cuda_device),
                to_device(table, cuda_device), to_device(lengths, cuda_device))
    from tpu_cake_b200 import _native

    with pytest.raises(_native.CakeError) as raised:
        executable.status()
    assert raised.value.code == _native.CAKE_ERR_DEVICE_CHECK
    assert executable.status() == (0, 0, 0, 0)  # cleared; the context is still usable
    executable.close()


def test_length_beyond_the_page_table_row_is_reported_and_skipped(cuda_device):
    """A sequence whose length needs more pages than its page-table row holds (the reference rejects
    it on the host, src/tpu_cake/rpa_lowering.py:94-104): the device reports code 4 for that
    sequence, leaves its output rows untouched and never reads the next sequence's row; the other
    sequences are computed as usual. The check skips the access, so nothing faults."""
    from tpu_cake_b200 import _native

    case = random_case(9, num_seqs=3, q_heads=8, kv_heads=2, page_size=16, lengths=[40, 50, 33], pool_pages=16, poison=False)
    query, key_cache, value_cache, table, lengths = case
    bad = lengths.copy()
    bad[1] = table.shape[1] * 16 + 1  # one token more than the row can address
    for cache_layout in ("separate", "fused"):
        plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
            name="long", schedule_sha256="0" * 64, query_shape=query.shape, cache_shape=key_cache.shape,
            page_table_shape=table.shape, bias_shape=None, softmax_scale=1.0 / math.sqrt(128), cache_layout=cache_layout,
        )
        executable = plan.build(cuda_device)
        if cache_layout == "fused":
            caches = (to_device(oracle.fused_cache_from_separate(key_cache, value_cache), cuda_device), None)
        else:
            caches = (to_device(key_cache, cuda_device), to_device(value_cache, cuda_device))
        out = torch.full(query.shape, 7.0, dtype=torch.bfloat16, device=cuda_device)
        plan.invoke(executable, to_device(query, cuda_device), caches[0], caches[1], to_device(table, cuda_device),
                    to_device(bad, cuda_device), out=out)
        with pytest.raises(_native.CakeError) as raised:
            executable.status()
        assert raised.value.code == _native.CAKE_ERR_DEVICE_CHECK
        actual = torch_to_bf16(out).astype(np.float32)
        assert np.all(actual[1] == 7.0)
        expected = expected_for(case)
        assert_close(actual[[0, 2]], expected[[0, 2]])
        executable.close()


def test_gather_barrier_gives_up_when_a_peer_never_publishes(cuda_device):
    """Two mesh positions, only position 0 runs, with a wait budget of 5 ms: its flag barrier gives
    up (CAKE_ERR_TIMEOUT, code 2, missing rank 1) and the kernel returns -- nothing hangs -- its own
    slice is in both gathered buffers, and the plan works again afterwards."""
    from tpu_cake_b200 import _native

    world, lengths = 2, [40, 700, 17]
    case = random_case(32, num_seqs=len(lengths), q_heads=8, kv_heads=2, page_size=16, lengths=lengths, pool_pages=64, poison=False)
    query, key_cache, value_cache, table, lens = case
    expected = expected_for(case)
    count, local_q = len(lengths), 4
    gathered = [torch.zeros((2, world, count, local_q, 128), dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int64, device=cuda_device) for _ in range(world)]
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name="shard0", schedule_sha256="0" * 64, query_shape=(count, local_q, 128), cache_shape=(key_cache.shape[0], 16, 1, 128),
        page_table_shape=table.shape, bias_shape=None, softmax_scale=1.0 / math.sqrt(128), cache_layout="fused", wait_budget_ms=5,
    )
    executable = plan.build(cuda_device)
    q0 = to_device(np.ascontiguousarray(query[:, :local_q]), cuda_device)
    cache0 = to_device(oracle.fused_cache_from_separate(key_cache[:, :, :1], value_cache[:, :, :1]), cuda_device)
    table_d, lens_d = to_device(table, cuda_device), to_device(lens, cuda_device)
    half = executable.enqueue_allgather(q0, cache0, None, lens_d, table_d, [g.data_ptr() for g in gathered], [f.data_ptr() for f in flags], world, 0)
    with pytest.raises(_native.CakeError) as raised:
        executable.status()
    assert raised.value.code == _native.CAKE_ERR_TIMEOUT and "never heard from rank 1" in str(raised.value)
    for buffer in gathered:
        assert_close(torch_to_bf16(buffer[half, 0]).astype(np.float32), expected[:, :local_q])
    # The peer "arrives": with its flag published the next call's barrier passes.
    flags[0][1] = 2
    half = executable.enqueue_allgather(q0, cache0, None, lens_d, table_d, [g.data_ptr() for g in gathered], [f.data_ptr() for f in flags], world, 0)
    assert executable.status() == (0, 0, 0, 0)
    assert_close(torch_to_bf16(gathered[1][half, 0]).astype(np.float32), expected[:, :local_q])
    executable.close()


def test_decode_configuration_full_size(cuda_device):
    """64 sequences, KV lengths uniform in [128, 8192], 32 / 8 heads, page 16, pool of 65536 pages:
    a sample of sequences (shortest, longest, and a few between) against the oracle."""
    config = workloads.DECODE_64
    lengths, table = workloads.decode_metadata(config)
    generator = torch.Generator(device=cuda_device).manual_seed(64)
    shape = (config.total_pages, config.page_size, config.kv_heads, 2, config.head_dim)
    cache = torch.empty(shape, dtype=torch.bfloat16, device=cuda_device)
    for start in range(0, config.total_pages, 8192):
        cache[start : start + 8192] = torch.randn((8192, *shape[1:]), generator=generator, device=cuda_device).to(torch.bfloat16)
    query = torch.randn((config.num_seqs, config.q_heads, config.head_dim), generator=generator, device=cuda_device).to(torch.bfloat16)
    plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
        name=config.name, schedule_sha256="0" * 64, query_shape=tuple(query.shape),
        cache_shape=(config.total_pages, config.page_size, config.kv_heads, config.head_dim),
        page_table_shape=table.shape, bias_shape=None, softmax_scale=config.softmax_scale, cache_layout="fused",
    )
    executable = plan.build(cuda_device)
    out = plan.invoke(executable, query, cache, None, to_device(table, cuda_device), to_device(lengths, cuda_device))
    assert executable.status() == (0, 0, 0, 0)
    actual = torch_to_bf16(out).astype(np.float32)
    order = np.argsort(lengths)
    sample = [int(order[0]), int(order[-1]), int(order[31]), 0, 17, 63]
    query_host = torch_to_bf16(query)
    for s in sample:
        count = -(-int(lengths[s]) // config.page_size)
        pages = torch.from_numpy(table[s, :count].astype(np.int64)).to(cuda_device)
        rows = torch_to_bf16(cache[pages])  # [count, ps, kv_heads, 2, dim]
        expected = oracle.rpa_separate(
            query_host[s : s + 1], rows[:, :, :, 0, :], rows[:, :, :, 1, :], np.arange(count, dtype=np.int32)[None, :],
            lengths[s : s + 1], None, scale=config.softmax_scale,
        )
        assert_close(actual[s : s + 1], expected)
    executable.close()


def test_sharded_decode_writes_every_ranks_gathered_buffer(cuda_device):
    """KV heads sharded over 4 mesh positions, all emulated on this GPU: every position decodes its
    heads and stores its slice into every position's gathered buffer (no waiting: each call is
    enqueued with wait=False); afterwards every buffer holds the full [W, S, Hq/W, D] result."""
    import ctypes

    from tpu_cake_b200 import _native

    world, lengths = 4, [40, 700, 1300, 17, 512]
    case = random_case(31, num_seqs=len(lengths), q_heads=16, kv_heads=4, page_size=16, lengths=lengths, pool_pages=200, poison=False)
    query, key_cache, value_cache, table, lens = case
    expected = expected_for(case)  # [S, 16, 128]
    count, local_q, local_kv = len(lengths), 4, 1
    lib = _native.load()
    gathered = [torch.zeros((2, world, count, local_q, 128), dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int64, device=cuda_device) for _ in range(world)]
    table_d, lens_d = to_device(table, cuda_device), to_device(lens, cuda_device)
    executables, keep = [], []
    for rank in range(world):
        plan = rpa_cuda_lowering.CudaPagedAttentionPlan(
            name=f"shard{rank}", schedule_sha256="0" * 64, query_shape=(count, local_q, 128),
            cache_shape=(key_cache.shape[0], 16, local_kv, 128), page_table_shape=table.shape, bias_shape=None,
            softmax_scale=1.0 / math.sqrt(128), cache_layout="fused",
        )
        executable = plan.build(cuda_device)
        q_r = to_device(np.ascontiguousarray(query[:, rank * local_q : (rank + 1) * local_q]), cuda_device)
        fused = oracle.fused_cache_from_separate(key_cache[:, :, rank : rank + 1], value_cache[:, :, rank : rank + 1])
        cache_r = to_device(fused, cuda_device)
        keep.append((q_r, cache_r))
        half = executable.enqueue_allgather(q_r, cache_r, None, lens_d, table_d, [g.data_ptr() for g in gathered],
                                            [f.data_ptr() for f in flags], world, rank, wait=False)
        assert half == 1  # the first call fills half 1, the second half 0
        executables.append(executable)
    torch.cuda.synchronize(cuda_device)
    first = [torch_to_bf16(buffer[1]).astype(np.float32) for buffer in gathered]
    # Second call with negated queries: it must land in the other half and leave the first alone.
    for rank, (executable, (q_r, cache_r)) in enumerate(zip(executables, keep)):
        half = executable.enqueue_allgather(-q_r, cache_r, None, lens_d, table_d, [g.data_ptr() for g in gathered],
                                            [f.data_ptr() for f in flags], world, rank, wait=False)
        assert half == 0
    torch.cuda.synchronize(cuda_device)
    for executable in executables:
        assert executable.status() == (0, 0, 0, 0)
        executable.close()
    for index, buffer in enumerate(gathered):
        full = torch_to_bf16(buffer[1]).astype(np.float32)  # [W, S, Hq/W, D]
        assembled = np.concatenate([full[r] for r in range(world)], axis=1)
        assert_close(assembled, expected)
        np.testing.assert_array_equal(full, first[index])
        np.testing.assert_array_equal(full, torch_to_bf16(gathered[0][1]).astype(np.float32))
        other = torch_to_bf16(buffer[0]).astype(np.float32)
        assert np.isfinite(other).all() and not np.array_equal(other, full)
        np.testing.assert_array_equal(other, torch_to_bf16(gathered[0][0]).astype(np.float32))
    for flag in flags:
        assert flag.cpu().tolist()[:world] == [2] * world


def test_chunk_search_on_the_decode_kernel(cuda_device, tmp_path):
    """search-rpa with device timing on a shrunken pool of the 64-sequence configuration: all runs
    agree with each other within the attention tolerance and the result carries per-candidate medians."""
    from tpu_cake_b200 import rpa_search

    contract = rpa_search.RpaSearchContract(
        workload="rpa-decode-64seq", baseline="chunk-512", warmup_iterations=1, measured_iterations=3, rounds=5, bootstrap_samples=1000,
        pool_pages=20480,
        candidates=(rpa_search.RpaSearchCandidate("chunk-512", 512), rpa_search.RpaSearchCandidate("chunk-1024", 1024)),
    )
    result = rpa_search.run_rpa_search(tmp_path / "search", contract)
    assert result.baseline == "chunk-512" and all(row.sample_count == 15 for row in result.candidates)
    assert all(50_000 < row.median_ns < 5_000_000 for row in result.candidates)


def test_data_tensor_sharded_surface_on_one_gpu(cuda_device):
    """All eight positions of the 2 x 4 surface run one after the other on one GPU (they exchange
    nothing): every shard's output and updated cache equal the oracle's for that data block,
    restricted to the shard's heads."""
    from tests.sharded_cases import build_sharded_surface

    global_inputs, block_inputs = build_sharded_surface(11)
    shapes = [tuple(np.asarray(v).shape) for v in global_inputs]
    local = rpa_cuda_lowering.CudaFusedRpaPlan(
        name="surface", schedule_sha256="0" * 64, query_shape=(4, 8, 128), key_shape=(4, 4, 128), value_shape=(4, 4, 128),
        fused_cache_shape=(shapes[3][0] // 2, 1, 4, 2, 128), kv_lengths_shape=(4,), page_indices_shape=(shapes[5][0] // 2,),
        cumulative_query_lengths_shape=(5,), cumulative_kv_lengths_shape=(5,), distribution_shape=(3,),
        relative_states_shape=(4, 8, 16), relative_projection_shape=(16, 512), output_shape=(4, 8, 128), softmax_scale=1.0 / 128,
    )
    surface = rpa_cuda_lowering.ShardedCudaFusedRpaPlan(local)
    expected = [oracle.rpa_fused(block) for block in block_inputs]  # per data block, all heads
    executable = surface.build(cuda_device)
    try:
        outputs, caches = {}, {}
        for rank in range(8):
            position = surface.mesh_position(rank)
            shard = surface.shard_inputs(global_inputs, position)
            device_inputs = tuple(to_device(np.ascontiguousarray(value), cuda_device) for value in shard)
            output, cache = surface.run_local(executable, *device_inputs)
            assert executable.status() == (0, 0, 0, 0)
            outputs[position], caches[position] = torch_to_bf16(output), torch_to_bf16(cache)
            d, t = position
            assert_close(outputs[position].astype(np.float32), expected[d][0][:, 8 * t : 8 * t + 8].astype(np.float32))
        global_cache = surface.assemble(caches, 1)
        want_cache = np.concatenate([cache for _, cache in expected], axis=0)
        np.testing.assert_array_equal(global_cache.view(np.uint16), want_cache.view(np.uint16))
        assert surface.assemble(outputs, 0).shape == (8, 32, 128)
    finally:
        executable.close()


def test_sharded_surface_chained_timing_rounds(cuda_device):
    """The surface's timing protocol on one mesh position: rounds restart from the placed inputs,
    calls inside a round feed output and cache forward; every round yields its samples."""
    from tests.sharded_cases import build_sharded_surface

    global_inputs, _ = build_sharded_surface(13)
    shapes = [tuple(np.asarray(v).shape) for v in global_inputs]
    local = rpa_cuda_lowering.CudaFusedRpaPlan(
        name="surface", schedule_sha256="0" * 64, query_shape=(4, 8, 128), key_shape=(4, 4, 128), value_shape=(4, 4, 128),
        fused_cache_shape=(shapes[3][0] // 2, 1, 4, 2, 128), kv_lengths_shape=(4,), page_indices_shape=(shapes[5][0] // 2,),
        cumulative_query_lengths_shape=(5,), cumulative_kv_lengths_shape=(5,), distribution_shape=(3,),
        relative_states_shape=(4, 8, 16), relative_projection_shape=(16, 512), output_shape=(4, 8, 128), softmax_scale=1.0 / 128,
    )
    surface = rpa_cuda_lowering.ShardedCudaFusedRpaPlan(local)
    shard = tuple(np.ascontiguousarray(v) for v in surface.shard_inputs(global_inputs, surface.mesh_position(6)))
    executable = surface.build(cuda_device)
    try:
        rounds = surface.timing_rounds(executable, shard, warmup_iterations=2, timing_rounds=3, samples_per_round=5)
        assert [r["round_index"] for r in rounds] == [0, 1, 2]
        assert all(len(r["samples_ns"]) == 5 and r["median_ns"] > 0 for r in rounds)
        # A chained call is still a valid decode: run one more from placed inputs and compare with the oracle.
        device_inputs = tuple(to_device(v, cuda_device) for v in shard)
        output, _ = surface.run_local(executable, *device_inputs)
        expected, _ = oracle.rpa_fused(shard)
        maximum, relative = rpa_cuda_lowering.surface_errors(torch_to_bf16(output).astype(np.float32), expected.astype(np.float32))
        assert maximum <= MAX_ABS and relative <= REL_L2
    finally:
        executable.close()
