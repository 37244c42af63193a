"""Builders of small ragged (mixed prefill / decode) batches shared by the CPU and GPU tests."""

from __future__ import annotations

import numpy as np

from tests.helpers import BF16
from tpu_cake_b200 import workloads


def build_mixed_case(seed, decode_kv, prefill, *, q_heads=8, kv_heads=2, page_size=16, poison=False, spare_pages=7):
    """decode_kv: KV lengths of the decode sequences; prefill: (query length, prior context) pairs.
    Returns (inputs 11-tuple of numpy arrays, metadata). With ``poison`` every cache row the batch
    must not read (unused pages, page tails beyond kv_len) is NaN."""
    generator = np.random.default_rng(seed)
    kv_lens = list(decode_kv) + [q + prior for q, prior in prefill]
    q_lens = [1] * len(decode_kv) + [q for q, _ in prefill]
    meta = workloads.ragged_metadata(kv_lens, q_lens, page_size, len(decode_kv), generator, spare_pages=spare_pages)
    tokens = meta.num_tokens
    q = generator.normal(size=(tokens, q_heads, 128)).astype(np.float32).astype(BF16)
    k = generator.normal(size=(tokens, kv_heads, 128)).astype(np.float32).astype(BF16)
    v = generator.normal(size=(tokens, kv_heads, 128)).astype(np.float32).astype(BF16)
    cache = generator.normal(size=(meta.total_pages, page_size, kv_heads, 2, 128)).astype(np.float32).astype(BF16)
    if poison:
        keep = np.zeros((meta.total_pages, page_size), dtype=bool)
        for s, length in enumerate(meta.kv_lens):
            first = int(meta.cu_kv_lens[s]) // page_size
            for position in range(int(length)):
                keep[meta.page_indices[first + position // page_size], position % page_size] = True
        cache[~keep] = np.float32(np.nan)
    inputs = (q, k, v, cache, meta.kv_lens, meta.page_indices, meta.cu_q_lens, meta.cu_kv_lens, meta.distribution, None, None)
    return inputs, meta
