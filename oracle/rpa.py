"""Oracle for Inkling ragged paged attention (numpy, float32): pure decode, pinned; mixed batches, unpinned.

Restates the reference's two numpy oracles:
  - ``rpa_separate``: separate K / V caches [pages, page_size, heads, dim], a 2-D page table and a
    dense additive bias indexed by key position (src/tpu_cake/workloads/inkling_rpa.py:37-73);
  - ``rpa_fused``: the fused interleaved cache [pages, page_size, 2*kv_heads/2, 2, dim_padded] with
    flat page indices, the cache update of the new token and the relative-position bias
    (src/tpu_cake/workloads/inkling_rpa.py:471-589).
Both take the softmax scale as a parameter; the reference fixes it to 1/head_dim
(inkling_rpa.py:67-68, 538-542), which is the default here.
"""

from __future__ import annotations

import math

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)

MUTATIONS = (
    "wrong_scale",
    "omit_relative_bias",
    "wrong_page_index",
    "ignore_page_indices",
    "swap_kv_interleave",
    "skip_cache_update",
)


def _softmax_rows(scores: np.ndarray) -> np.ndarray:
    shifted = scores - scores.max(axis=-1, keepdims=True)
    weights = np.exp(shifted, dtype=np.float32)
    return weights / weights.sum(axis=-1, keepdims=True)


def _attend(query: np.ndarray, keys: np.ndarray, values: np.ndarray, scale: float, bias: np.ndarray | None) -> np.ndarray:
    """query [Hq, D]; keys [L, Hk, D]; values [L, Hv, Dv]; GQA map q_head // (Hq / H)."""
    q_heads = query.shape[0]
    key_of = np.arange(q_heads) // (q_heads // keys.shape[1])
    value_of = np.arange(q_heads) // (q_heads // values.shape[1])
    scores = np.einsum("hd,lhd->hl", query, keys[:, key_of, :], dtype=np.float32) * np.float32(scale)
    if bias is not None:
        scores = scores + bias
    weights = _softmax_rows(scores.astype(np.float32))
    return np.einsum("hl,lhd->hd", weights, values[:, value_of, :], dtype=np.float32)


def rpa_separate(
    query: np.ndarray,
    key_cache: np.ndarray,
    value_cache: np.ndarray,
    page_table: np.ndarray,
    sequence_lengths: np.ndarray,
    bias: np.ndarray | None = None,
    *,
    scale: float | None = None,
) -> np.ndarray:
    """Decode attention over separate paged K / V caches; returns float32 [B, Hq, Dv]."""
    query = np.asarray(query, dtype=np.float32)
    key_cache = np.asarray(key_cache, dtype=np.float32)
    value_cache = np.asarray(value_cache, dtype=np.float32)
    batch, q_heads, dim = query.shape
    page_size = key_cache.shape[1]
    if value_cache.shape[1] != page_size:
        raise ValueError("key and value caches must use the same page size")
    if key_cache.shape[3] != dim:
        raise ValueError("query and key head dimensions must match")
    if q_heads % key_cache.shape[2] or q_heads % value_cache.shape[2]:
        raise ValueError("query heads must divide evenly across key and value heads")
    if bias is not None and bias.shape[0] != q_heads:
        raise ValueError("relative bias must provide one row per query head")
    if scale is None:
        scale = 1.0 / dim
    out = np.empty((batch, q_heads, value_cache.shape[3]), dtype=np.float32)
    for b in range(batch):
        length = int(sequence_lengths[b])
        pages = np.asarray(page_table[b, : math.ceil(length / page_size)], dtype=np.int64)
        keys = key_cache[pages].reshape(-1, key_cache.shape[2], key_cache.shape[3])[:length]
        values = value_cache[pages].reshape(-1, value_cache.shape[2], value_cache.shape[3])[:length]
        row_bias = None if bias is None else np.asarray(bias, dtype=np.float32)[:, :length]
        out[b] = _attend(query[b], keys, values, scale, row_bias)
    return out


def rpa_fused(
    inputs: tuple[np.ndarray, ...],
    *,
    scale: float | None = None,
    mutation: str | None = None,
    update_cache: bool = True,
    use_relative_bias: bool = True,
) -> tuple[np.ndarray, np.ndarray]:
    """Fused-cache decode with cache update and relative bias.

    ``inputs`` is the reference's 11-tuple (queries [N,Hq,D], keys [N,Hkv,D], values [N,Hkv,D],
    cache [P,ps,2*Hkv/pack,pack,Dpad], kv_lengths [N], page_indices [PI], cu_q_lens [N+1],
    cu_kv_lens [N+1], distribution [3], relative_states [N,Hq,R], relative_projection [R,E]).
    Returns (output, updated cache), both bfloat16 (ml_dtypes), like the reference.
    """
    if mutation is not None and mutation not in MUTATIONS:
        raise ValueError(f"unknown oracle mutation {mutation}")
    (q_in, k_in, v_in, cache_in, lens_in, pages_in, cu_q_in, cu_kv_in, dist_in, states_in, proj_in) = inputs
    queries = np.asarray(q_in, dtype=np.float32)
    new_keys = np.asarray(k_in, dtype=np.float32)
    new_values = np.asarray(v_in, dtype=np.float32)
    cache = np.array(np.asarray(cache_in, dtype=np.float32))
    lengths = np.asarray(lens_in, dtype=np.int64)
    page_indices = np.array(np.asarray(pages_in, dtype=np.int64))
    cu_q = np.asarray(cu_q_in, dtype=np.int64)
    cu_kv = np.asarray(cu_kv_in, dtype=np.int64)
    distribution = np.asarray(dist_in, dtype=np.int64)
    count = lengths.shape[0]
    if not np.array_equal(distribution, np.full(3, count)):
        raise ValueError("fused RPA oracle requires a decode-only distribution")
    if not np.array_equal(cu_q, np.arange(count + 1)):
        raise ValueError("fused RPA oracle requires one query token per sequence")
    if mutation == "ignore_page_indices":
        page_indices = np.arange(page_indices.size, dtype=np.int64)
    elif mutation == "wrong_page_index":
        page_indices[0] = (page_indices[0] + 1) % cache.shape[0]

    page_size, pack = cache.shape[1], cache.shape[3]
    dim = queries.shape[-1]
    k_slot, v_slot = (1, 0) if mutation == "swap_kv_interleave" else (0, 1)
    if update_cache and mutation != "skip_cache_update":
        for s in range(count):
            position = int(lengths[s]) - 1
            page = page_indices[int(cu_kv[s]) // page_size + position // page_size]
            slot = position % page_size
            for head in range(new_keys.shape[1]):
                for which, source in ((k_slot, new_keys), (v_slot, new_values)):
                    index = 2 * head + which
                    row = cache[page, slot, index // pack, index % pack]
                    row[:] = 0.0
                    row[: source.shape[-1]] = source[s, head]

    flat = cache.reshape(cache.shape[0], page_size, cache.shape[2] * pack, cache.shape[4])
    if scale is None:
        scale = 1.0 / dim
    if mutation == "wrong_scale":
        scale = 1.0 / math.sqrt(dim)
    apply_bias = use_relative_bias and mutation != "omit_relative_bias" and states_in is not None
    if apply_bias:
        states = np.asarray(states_in, dtype=np.float32)
        projection = np.asarray(proj_in, dtype=np.float32)
        extent = projection.shape[1]
    out = np.empty_like(queries, dtype=np.float32)
    for s in range(count):
        length = int(lengths[s])
        first = int(cu_kv[s]) // page_size
        pages = page_indices[first : first + math.ceil(length / page_size)]
        rows = flat[pages].reshape(-1, flat.shape[2], flat.shape[3])[:length]
        keys = rows[:, k_slot::2, :dim][:, : new_keys.shape[1]]
        values = rows[:, v_slot::2, :dim][:, : new_values.shape[1]]
        bias = None
        if apply_bias:
            distance = (length - 1) - np.arange(length)
            gathered = projection[:, np.clip(distance, 0, extent - 1)]
            bias = np.einsum("hr,rl->hl", states[s], gathered, dtype=np.float32)
            bias = np.where(distance[None, :] < extent, bias, np.float32(0.0)).astype(np.float32)
        out[s] = _attend(queries[s], keys, values, scale, bias)
    return out.astype(BF16), cache.astype(BF16)


def fused_cache_from_separate(key_cache: np.ndarray, value_cache: np.ndarray) -> np.ndarray:
    """[P,ps,H,D] x 2 -> fused [P,ps,H,2,D]: head h's K at interleaved index 2h, V at 2h+1
    (pack = 2, inkling_rpa.py:524-534)."""
    return np.ascontiguousarray(np.stack([key_cache, value_cache], axis=3))


def rpa_mixed(
    queries: np.ndarray,
    new_keys: np.ndarray,
    new_values: np.ndarray,
    cache: np.ndarray,
    kv_lengths: np.ndarray,
    page_indices: np.ndarray,
    cu_q_lens: np.ndarray,
    cu_kv_lens: np.ndarray,
    *,
    scale: float | None = None,
    update_cache: bool = True,
    probabilities_in_bf16: bool = False,
) -> tuple[np.ndarray, np.ndarray]:
    """Ragged batch (decode and prefill sequences mixed) on the fused cache, causal, no bias.

    The reference's own oracle rejects query lengths above one
    (src/tpu_cake/workloads/inkling_rpa.py:505-509); this function extends ``rpa_fused`` by the
    semantics of the kernel the reference wraps (causal=1, new tokens appended at the end of each
    sequence; src/tpu_cake/rpa_lowering.py:232-273): sequence s owns query tokens
    [cu_q[s], cu_q[s+1]); query token i of a sequence with q query tokens and kv_len cached tokens
    sits at position kv_len - q + i, its K/V are written there first, and it attends to positions
    0..kv_len - q + i. PINNED two ways: tests/test_mixed_cpu.py ties it to the pinned decode oracle
    (every query token equals a one-token decode at its own length), and compares it with the
    outputs of the array program shipped with that kernel
    (ecosystem/source/jax/ragged_paged_attention.py:73-148, ``ref_ragged_paged_attention``) stored
    in tests/golden/mixed_reference_vectors.npz. That program rounds the softmax probabilities to
    the value dtype before multiplying by V; ``probabilities_in_bf16`` does the same here.
    Returns (output [T,Hq,D] bfloat16, updated cache bfloat16).
    """
    q = np.asarray(queries, dtype=np.float32)
    k_new = np.asarray(new_keys, dtype=np.float32)
    v_new = np.asarray(new_values, dtype=np.float32)
    cache = np.array(np.asarray(cache, dtype=np.float32))
    lengths = np.asarray(kv_lengths, dtype=np.int64)
    pages_flat = np.asarray(page_indices, dtype=np.int64)
    cu_q = np.asarray(cu_q_lens, dtype=np.int64)
    cu_kv = np.asarray(cu_kv_lens, dtype=np.int64)
    page_size, pack = cache.shape[1], cache.shape[3]
    dim, kv_heads = q.shape[-1], k_new.shape[1]
    if scale is None:
        scale = 1.0 / dim
    count = lengths.shape[0]
    if update_cache:
        for s in range(count):
            q_len = int(cu_q[s + 1] - cu_q[s])
            for i in range(q_len):
                position = int(lengths[s]) - q_len + i
                page = pages_flat[int(cu_kv[s]) // page_size + position // page_size]
                for head in range(kv_heads):
                    for which, source in ((0, k_new), (1, v_new)):
                        index = 2 * head + which
                        row = cache[page, position % page_size, index // pack, index % pack]
                        row[:] = 0.0
                        row[:dim] = source[cu_q[s] + i, head]
    flat = cache.reshape(cache.shape[0], page_size, cache.shape[2] * pack, cache.shape[4])
    out = np.zeros_like(q, dtype=np.float32)
    group = q.shape[1] // kv_heads
    for s in range(count):
        length, q_len = int(lengths[s]), int(cu_q[s + 1] - cu_q[s])
        if q_len == 0:
            continue
        first = int(cu_kv[s]) // page_size
        pages = pages_flat[first : first + math.ceil(length / page_size)]
        rows = flat[pages].reshape(-1, flat.shape[2], flat.shape[3])[:length]
        keys = rows[:, 0::2, :dim][:, :kv_heads]      # [L, Hkv, D]
        values = rows[:, 1::2, :dim][:, :kv_heads]
        q_seq = q[cu_q[s] : cu_q[s + 1]].reshape(q_len, kv_heads, group, dim)
        scores = np.einsum("thgd,lhd->thgl", q_seq, keys, dtype=np.float32) * np.float32(scale)
        visible = np.arange(length)[None, :] <= (length - q_len + np.arange(q_len))[:, None]
        scores = np.where(visible[:, None, None, :], scores, -np.inf).astype(np.float32)
        weights = _softmax_rows(scores)
        if probabilities_in_bf16:
            weights = weights.astype(BF16).astype(np.float32)
        out[cu_q[s] : cu_q[s + 1]] = np.einsum("thgl,lhd->thgd", weights, values, dtype=np.float32).reshape(q_len, -1, dim)
    return out.astype(BF16), cache.astype(BF16)
