"""GPU parity of the ragged (mixed prefill / decode) attention path against the CPU oracle, through
the C ABI. The reference has no oracle of its own for query runs longer than one token; the oracle
used here is tied to the pinned decode oracle row by row and to the outputs of the array program
shipped with the kernel the reference wraps (tests/test_mixed_cpu.py), and one test below compares
the kernels with those stored outputs directly. Tolerance: max-abs <= 2e-2
and relative-L2 <= 1e-2 on bf16 outputs; the updated cache must be bit-exact."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import matmul_rs as metrics
from oracle import rpa as oracle
from tests.helpers import BF16, to_device, torch_to_bf16
from tests.mixed_cases import build_mixed_case
from tpu_cake_b200 import _native, rpa_cuda_lowering, workloads

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-2


def mixed_plan(inputs, *, scale=None, update_cache=True) -> rpa_cuda_lowering.CudaMixedRpaPlan:
    q, k, _, cache, lens, pages = inputs[:6]
    return rpa_cuda_lowering.CudaMixedRpaPlan(
        name="inkling_mixed_rpa", schedule_sha256="0" * 64, query_shape=tuple(q.shape), key_shape=tuple(k.shape),
        fused_cache_shape=tuple(cache.shape), sequences=len(lens), page_indices_shape=tuple(pages.shape),
        softmax_scale=scale if scale is not None else 1.0 / q.shape[2], update_cache=update_cache,
    )


def run_mixed(plan, inputs, device, repeats=1):
    executable = plan.build(device)
    try:
        plan.preflight(*inputs)
        device_inputs = tuple(None if value is None else to_device(np.asarray(value), device) for value in inputs)
        results = []
        for _ in range(repeats):
            output, cache = plan.invoke(executable, *device_inputs)
            assert executable.status() == (0, 0, 0, 0)
            results.append((torch_to_bf16(output), torch_to_bf16(cache)))
        return results if repeats > 1 else results[0]
    finally:
        executable.close()


def assert_close(actual, expected):
    actual, expected = actual.astype(np.float32), expected.astype(np.float32)
    assert np.isfinite(actual).all()
    assert metrics.max_abs_error(actual, expected) <= MAX_ABS
    assert metrics.relative_l2_error(actual, expected) <= REL_L2


@pytest.mark.parametrize(
    "decode_kv, prefill, q_heads, kv_heads, page_size",
    [
        ([17, 300, 64], [(130, 5), (64, 0), (257, 100)], 8, 2, 16),   # GQA 4: two heads per work item
        ([], [(128, 0), (129, 63), (1, 64), (200, 1)], 4, 2, 16),      # prefill only, tile and stage boundaries
        ([90], [(70, 10), (300, 7)], 3, 3, 16),                        # GQA 1: one head per work item
        ([33, 5], [(190, 0)], 16, 2, 32),                              # GQA 8, 32-token pages
        ([12], [(150, 9)], 4, 1, 8),
        ([7], [(75, 3)], 2, 1, 1),                                     # one token per page
    ],
)
def test_mixed_batches_match_the_oracle(cuda_device, decode_kv, prefill, q_heads, kv_heads, page_size):
    inputs, _ = build_mixed_case(11, decode_kv, prefill, q_heads=q_heads, kv_heads=kv_heads, page_size=page_size)
    scale = 128**-0.5
    expected_out, expected_cache = oracle.rpa_mixed(*inputs[:8], scale=scale)
    output, cache = run_mixed(mixed_plan(inputs, scale=scale), inputs, cuda_device)
    np.testing.assert_array_equal(cache.view(np.uint16), expected_cache.view(np.uint16))
    assert_close(output, expected_out)


@pytest.mark.parametrize("name", ["mixed_a", "mixed_b"])
def test_mixed_batches_match_the_shipped_reference_program(cuda_device, golden_dir, name):
    """Against the stored outputs of ``ref_ragged_paged_attention``
    (ecosystem/source/jax/ragged_paged_attention.py:73-148) on the cache after the update."""
    vectors = np.load(golden_dir / "mixed_reference_vectors.npz")
    bits = lambda key: vectors[f"{name}/{key}_bf16_bits"].view(BF16)  # noqa: E731
    plain = lambda key: vectors[f"{name}/{key}"]  # noqa: E731
    inputs = (bits("queries"), bits("keys"), bits("values"), bits("cache"), plain("kv_lengths"), plain("page_indices"),
              plain("cu_q_lens"), plain("cu_kv_lens"), plain("distribution"), None, None)
    scale = float(plain("softmax_scale"))
    output, _ = run_mixed(mixed_plan(inputs, scale=scale), inputs, cuda_device)
    assert_close(output, vectors[f"{name}/reference_output_bf16_bits"].view(BF16))


def test_poisoned_unused_rows_are_never_read(cuda_device):
    """Every cache row outside the sequences' valid tokens is NaN: page tails beyond kv_len, pages
    no sequence owns. A finite result within tolerance shows the indexing reads none of them."""
    inputs, _ = build_mixed_case(21, [50, 3], [(100, 27), (140, 0)], poison=True)
    expected_out, expected_cache = oracle.rpa_mixed(*inputs[:8], scale=0.1)
    output, cache = run_mixed(mixed_plan(inputs, scale=0.1), inputs, cuda_device)
    assert_close(output, expected_out)
    np.testing.assert_array_equal(cache.view(np.uint16), expected_cache.view(np.uint16))


def test_without_cache_update_the_cache_is_untouched(cuda_device):
    inputs, _ = build_mixed_case(31, [40], [(96, 32)])
    expected_out, _ = oracle.rpa_mixed(*inputs[:8], scale=0.09, update_cache=False)
    output, cache = run_mixed(mixed_plan(inputs, scale=0.09, update_cache=False), inputs, cuda_device)
    assert_close(output, expected_out)
    np.testing.assert_array_equal(cache.view(np.uint16), np.asarray(inputs[3]).view(np.uint16))


def test_repeats_are_bit_identical_and_decode_rows_equal_the_decode_call(cuda_device):
    inputs, meta = build_mixed_case(41, [100, 257, 31], [(160, 40)])
    first, second = run_mixed(mixed_plan(inputs, scale=0.088), inputs, cuda_device, repeats=2)
    np.testing.assert_array_equal(first[0].view(np.uint16), second[0].view(np.uint16))
    # The three decode sequences alone, through the decode entry point, on the same updated cache.
    decode_inputs = (inputs[0][:3], inputs[1][:3], inputs[2][:3], first[1], meta.kv_lens[:3], meta.page_indices,
                     np.arange(4, dtype=np.int32), meta.cu_kv_lens[:4], np.array([3, 3, 3], np.int32), None, None)
    shapes = [None if value is None else tuple(np.asarray(value).shape) for value in decode_inputs]
    plan = rpa_cuda_lowering.CudaFusedRpaPlan(
        name="decode_rows", schedule_sha256="0" * 64, query_shape=shapes[0], key_shape=shapes[1], value_shape=shapes[2],
        fused_cache_shape=shapes[3], kv_lengths_shape=shapes[4], page_indices_shape=shapes[5],
        cumulative_query_lengths_shape=shapes[6], cumulative_kv_lengths_shape=shapes[7], distribution_shape=shapes[8],
        relative_states_shape=None, relative_projection_shape=None, output_shape=shapes[0], softmax_scale=0.088, update_cache=False,
    )
    executable = plan.build(cuda_device)
    try:
        device_inputs = tuple(None if value is None else to_device(np.asarray(value), cuda_device) for value in decode_inputs)
        output, _ = plan.invoke(executable, *device_inputs)
        assert executable.status() == (0, 0, 0, 0)
        np.testing.assert_array_equal(torch_to_bf16(output).view(np.uint16), first[0][:3].view(np.uint16))
    finally:
        executable.close()


def test_bad_metadata_is_reported_not_faulted(cuda_device):
    """A sequence whose KV length is shorter than its query run: the plan kernel records status 4
    and the sequence is skipped; nothing is read out of range."""
    inputs, meta = build_mixed_case(51, [20], [(64, 8)])
    arrays = [None if value is None else np.array(value) for value in inputs]
    arrays[4][1] = 10  # kv_len 10 < 64 query tokens
    plan = mixed_plan(inputs, scale=0.1, update_cache=False)
    executable = plan.build(cuda_device)
    try:
        device_inputs = tuple(None if value is None else to_device(value, cuda_device) for value in arrays)
        plan.invoke(executable, *device_inputs)
        with pytest.raises(_native.CakeError, match=r"sequence metadata out of range \(1, 10, 64\)") as raised:
            executable.status()
        assert raised.value.code == _native.CAKE_ERR_DEVICE_CHECK
        assert executable.status() == (0, 0, 0, 0)  # reading the status word clears it
    finally:
        executable.close()


def test_full_size_mixed_configuration_on_sampled_sequences(cuda_device):
    """8 prefill + 120 decode sequences at full size; the oracle checks two prefill sequences (the
    shortest and the one with the longest context) and three decode sequences."""
    config = workloads.MIXED_8_120
    meta = workloads.mixed_metadata(config)
    generator = torch.Generator(device=cuda_device).manual_seed(5)
    tokens = meta.num_tokens
    q = torch.randn((tokens, config.q_heads, 128), generator=generator, device=cuda_device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((tokens, config.kv_heads, 128), generator=generator, device=cuda_device, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((tokens, config.kv_heads, 128), generator=generator, device=cuda_device, dtype=torch.float32).to(torch.bfloat16)
    cache = torch.empty((meta.total_pages, config.page_size, config.kv_heads, 2, 128), device=cuda_device, dtype=torch.bfloat16)
    for start in range(0, meta.total_pages, 16384):
        block = cache[start : start + 16384]
        block.copy_(torch.randn(block.shape, generator=generator, device=cuda_device, dtype=torch.float32))
    plan = rpa_cuda_lowering.CudaMixedRpaPlan(
        name="mixed_full", schedule_sha256="0" * 64, query_shape=tuple(q.shape), key_shape=tuple(k.shape),
        fused_cache_shape=tuple(cache.shape), sequences=128, page_indices_shape=tuple(meta.page_indices.shape),
        softmax_scale=config.softmax_scale,
    )
    executable = plan.build(cuda_device)
    try:
        args = (q, k, v, cache, to_device(meta.kv_lens, cuda_device), to_device(meta.page_indices, cuda_device),
                to_device(meta.cu_q_lens, cuda_device), to_device(meta.cu_kv_lens, cuda_device), meta.distribution, None, None)
        output, _ = plan.invoke(executable, *args)
        assert executable.status() == (0, 0, 0, 0)
        q_lens = np.diff(meta.cu_q_lens)
        prefill = np.arange(120, 128)
        chosen = [int(prefill[np.argmin(q_lens[120:])]), int(prefill[np.argmax(meta.kv_lens[120:])]), 0, 57, 119]
        page_size = config.page_size
        for s in chosen:
            first = int(meta.cu_kv_lens[s]) // page_size
            pages = meta.page_indices[first : first + -(-int(meta.kv_lens[s]) // page_size)]
            rows = slice(int(meta.cu_q_lens[s]), int(meta.cu_q_lens[s + 1]))
            local_cache = torch_to_bf16(cache[torch.from_numpy(pages.astype(np.int64)).to(cuda_device)])
            single = (torch_to_bf16(q[rows]), torch_to_bf16(k[rows]), torch_to_bf16(v[rows]), local_cache,
                      meta.kv_lens[s : s + 1], np.arange(len(pages), dtype=np.int32),
                      np.array([0, rows.stop - rows.start], np.int32), np.array([0, len(pages) * page_size], np.int32))
            expected, _ = oracle.rpa_mixed(*single, scale=config.softmax_scale, update_cache=False)
            assert_close(torch_to_bf16(output[rows]), expected)
    finally:
        executable.close()
