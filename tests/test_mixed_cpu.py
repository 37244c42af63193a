"""CPU checks of the ragged (mixed prefill / decode) path: the mixed oracle is tied to the pinned
decode oracle and to the outputs of the array program shipped with the kernel the reference wraps,
the host preflight accepts and rejects what it should, and the seeded 128-sequence configuration
has the stated shape."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import rpa
from tests.mixed_cases import build_mixed_case
from tpu_cake_b200 import rpa_cuda_lowering, workloads


def test_all_decode_batch_equals_the_pinned_decode_oracle():
    inputs, _ = build_mixed_case(3, [17, 33, 64, 100], [])
    out_mixed, cache_mixed = rpa.rpa_mixed(*inputs[:8])
    out_decode, cache_decode = rpa.rpa_fused(inputs, use_relative_bias=False)
    np.testing.assert_array_equal(cache_mixed.view(np.uint16), cache_decode.view(np.uint16))
    np.testing.assert_allclose(out_mixed.astype(np.float32), out_decode.astype(np.float32), rtol=2**-7, atol=1e-6)


def test_every_prefill_token_equals_a_decode_at_its_own_length():
    """Query token i of a prefill sequence, on the updated cache, is a one-token decode of a sequence
    of length prior + i + 1: the pinned decode oracle reproduces the mixed oracle row by row."""
    inputs, meta = build_mixed_case(5, [40], [(37, 0), (20, 29)], q_heads=4, kv_heads=2, page_size=8)
    out_mixed, cache = rpa.rpa_mixed(*inputs[:8])
    q = inputs[0]
    page_size = 8
    for s in (1, 2):
        q_len = int(meta.cu_q_lens[s + 1] - meta.cu_q_lens[s])
        first = int(meta.cu_kv_lens[s]) // page_size
        pages = meta.page_indices[first : first + -(-int(meta.kv_lens[s]) // page_size)]
        for i in (0, 1, q_len // 2, q_len - 1):
            token = int(meta.cu_q_lens[s]) + i
            length = int(meta.kv_lens[s]) - q_len + i + 1
            single = (q[token : token + 1], inputs[1][token : token + 1], inputs[2][token : token + 1], cache,
                      np.array([length], np.int32), pages.astype(np.int32), np.array([0, 1], np.int32),
                      np.array([0, -(-length // page_size) * page_size], np.int32), np.array([1, 1, 1], np.int32), None, None)
            expected, _ = rpa.rpa_fused(single, update_cache=False, use_relative_bias=False)
            np.testing.assert_allclose(out_mixed[token].astype(np.float32), expected[0].astype(np.float32), rtol=2**-7, atol=1e-6)


def test_cache_update_writes_every_query_token_at_its_position():
    inputs, meta = build_mixed_case(9, [5], [(19, 3)], q_heads=2, kv_heads=1, page_size=4)
    _, cache = rpa.rpa_mixed(*inputs[:8])
    before = inputs[3]
    changed = np.any(cache.view(np.uint16) != before.view(np.uint16), axis=(2, 3, 4))
    expected = np.zeros_like(changed)
    for s, q_len in ((0, 1), (1, 19)):
        first = int(meta.cu_kv_lens[s]) // 4
        for i in range(q_len):
            position = int(meta.kv_lens[s]) - q_len + i
            expected[meta.page_indices[first + position // 4], position % 4] = True
    np.testing.assert_array_equal(changed, expected)


def load_reference_case(golden_dir, name):
    vectors = np.load(golden_dir / "mixed_reference_vectors.npz")
    bits = lambda key: vectors[f"{name}/{key}_bf16_bits"].view(rpa.BF16)  # noqa: E731
    plain = lambda key: vectors[f"{name}/{key}"]  # noqa: E731
    inputs = (bits("queries"), bits("keys"), bits("values"), bits("cache"), plain("kv_lengths"), plain("page_indices"),
              plain("cu_q_lens"), plain("cu_kv_lens"))
    return inputs, float(plain("softmax_scale")), vectors[f"{name}/reference_output_bf16_bits"]


@pytest.mark.parametrize("name", ["mixed_a", "mixed_b"])
def test_mixed_oracle_against_the_shipped_reference_program(golden_dir, name):
    """``ref_ragged_paged_attention`` (ecosystem/source/jax/ragged_paged_attention.py:73-148) rounds the
    softmax probabilities to bf16 before the product with V. With the same rounding the oracle agrees
    bit for bit on all but a few outputs (a different summation order of the scores flips the rounding
    of a rare probability by one bf16 step, which moves an output by a few 1e-4); without it, in
    float32 as the GPU tests use it, it stays within 1e-2 max-abs / 5e-3 relative L2."""
    inputs, scale, reference_bits = load_reference_case(golden_dir, name)
    reference = reference_bits.view(rpa.BF16).astype(np.float32)
    rounded, _ = rpa.rpa_mixed(*inputs, scale=scale, probabilities_in_bf16=True)
    assert (rounded.view(np.uint16) == reference_bits).mean() >= 0.999
    np.testing.assert_allclose(rounded.astype(np.float32), reference, rtol=2**-7, atol=5e-4)
    plain, _ = rpa.rpa_mixed(*inputs, scale=scale)
    difference = plain.astype(np.float32) - reference
    assert np.abs(difference).max() <= 1e-2
    assert np.linalg.norm(difference) / np.linalg.norm(reference) <= 5e-3


def shapes_of(inputs):
    return tuple(None if value is None else tuple(np.asarray(value).shape) for value in inputs)


def test_preflight_accepts_a_good_batch_and_returns_the_decode_count():
    inputs, _ = build_mixed_case(1, [10, 20], [(30, 4)])
    assert rpa_cuda_lowering.preflight_mixed_metadata(inputs, shapes_of(inputs)) == 2


@pytest.mark.parametrize(
    "mutate, message",
    [
        (lambda a: a[8].__setitem__(0, 3) or a[8].__setitem__(1, 2), "distribution"),
        (lambda a: a[8].__setitem__(0, 3), "decode sequences must come first"),
        (lambda a: a[4].__setitem__(2, 5), "include the query tokens"),
        (lambda a: a[7].__setitem__(1, 17), "page-aligned"),
        (lambda a: a[5].__setitem__(0, 10**6), "outside the fused cache"),
        (lambda a: a[5].__setitem__(0, a[5][1]), "aliases a physical page"),
    ],
)
def test_preflight_rejects(mutate, message):
    inputs, _ = build_mixed_case(1, [10, 20], [(30, 4)])
    arrays = [None if value is None else np.array(value) for value in inputs]
    mutate(arrays)
    with pytest.raises(ValueError, match=message):
        rpa_cuda_lowering.preflight_mixed_metadata(tuple(arrays), shapes_of(inputs))


def test_seeded_mixed_configuration():
    config = workloads.MIXED_8_120
    meta = workloads.mixed_metadata(config)
    q_lens = np.diff(meta.cu_q_lens)
    assert len(meta.kv_lens) == 128 and tuple(meta.distribution) == (120, 128, 128)
    assert np.all(q_lens[:120] == 1) and q_lens[120:].min() >= 512 and q_lens[120:].max() <= 2048
    assert meta.kv_lens[:120].min() >= 256 and meta.kv_lens[:120].max() <= 32768
    prior = meta.kv_lens[120:] - q_lens[120:]
    assert prior.min() >= 0 and prior.max() <= 4096
    assert np.all(meta.cu_kv_lens % config.page_size == 0)
    assert np.unique(meta.page_indices).size == meta.page_indices.size
    work = workloads.mixed_algorithmic_work(meta, config.q_heads, config.kv_heads, config.head_dim)
    assert work["bytes"] > work["decode_bytes"] > 0 and work["flops"] > work["prefill_flops"] > 0
    again = workloads.mixed_metadata(config)
    np.testing.assert_array_equal(again.page_indices, meta.page_indices)
