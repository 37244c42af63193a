"""Generates ``mixed_reference_vectors.npz``: ragged (prefill + decode) batches and the outputs of
the reference function the reference project ships for them.

    python tests/golden/make_mixed_golden.py /path/to/tpu-cake

The reference project has no oracle of its own for query runs longer than one token; what it ships is
the kernel package it wraps, whose file ``ecosystem/source/jax/ragged_paged_attention.py`` holds
``ref_ragged_paged_attention`` (lines 73-148): a plain array program (gather pages, K at even and V
at odd combined heads, causal mask ``kv_len - q_len + i < j``, softmax cast to the value dtype, output
cast to the query dtype). jax is not installed here, so the file is loaded with ``jax.numpy`` mapped
to numpy (bfloat16 from ml_dtypes, the same round-to-nearest-even conversion) and every import it
does not need for this function replaced by an inert stand-in. The function does not update the
cache, so it is given the cache AFTER the new tokens were written (by indexing only, no arithmetic).
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path
from unittest import mock

import ml_dtypes
import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
BF16 = np.dtype(ml_dtypes.bfloat16)

CASES = {
    # name: (seed, decode KV lengths, (query length, prior context) of the prefill sequences, heads, page size)
    "mixed_a": (21, [33, 70], [(5, 0), (37, 20), (70, 60)], 4, 1, 16),
    "mixed_b": (22, [16], [(129, 0), (40, 64)], 4, 2, 8),
}


def _install_numpy_as_jax() -> None:
    jnp = types.ModuleType("jax.numpy")
    for name in ("float32", "int32", "finfo", "dtype", "repeat", "where", "logical_or", "tanh", "concatenate"):
        setattr(jnp, name, getattr(np, name))
    jnp.bfloat16 = BF16

    def einsum(spec, a, b, preferred_element_type=None):
        return np.einsum(spec, np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)).astype(preferred_element_type or a.dtype)

    jnp.einsum = einsum

    def softmax(x, axis=-1):
        x = np.asarray(x, dtype=np.float32)
        e = np.exp(x - x.max(axis=axis, keepdims=True))
        return e / e.sum(axis=axis, keepdims=True)

    def broadcasted_iota(dtype, shape, dimension):
        index = np.arange(shape[dimension], dtype=dtype)
        return np.broadcast_to(index.reshape([-1 if d == dimension else 1 for d in range(len(shape))]), shape)

    lax = types.ModuleType("jax.lax")
    lax.broadcasted_iota = broadcasted_iota
    nn = types.ModuleType("jax.nn")
    nn.softmax = softmax
    jax = types.ModuleType("jax")
    jax.numpy, jax.lax, jax.nn, jax.Array = jnp, lax, nn, np.ndarray
    jax.jit = lambda function=None, **_: function if function is not None else (lambda f: f)
    sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.nn": nn})
    for name in ("jax._src", "jax._src.dtypes", "jax.experimental", "jax.experimental.pallas", "jax.experimental.pallas.tpu",
                 "jax.experimental.pallas.ops", "jax.experimental.pallas.ops.tpu", "jax.experimental.pallas.ops.tpu.ragged_paged_attention",
                 "jax.experimental.pallas.ops.tpu.ragged_paged_attention.tuned_block_sizes"):
        sys.modules[name] = mock.MagicMock(name=name)


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_mixed_golden.py PATH_TO_TPU_CAKE_CHECKOUT")
    source = Path(sys.argv[1]).resolve() / "ecosystem" / "source" / "jax" / "ragged_paged_attention.py"
    _install_numpy_as_jax()
    spec = importlib.util.spec_from_file_location("reference_ragged_paged_attention", source)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)

    import __graft_entry__

    __graft_entry__.load_package()  # the batch builder uses the package's seeded metadata generator
    from tests.mixed_cases import build_mixed_case

    arrays: dict[str, np.ndarray] = {}
    for name, (seed, decode_kv, prefill, q_heads, kv_heads, page_size) in CASES.items():
        inputs, meta = build_mixed_case(seed, decode_kv, prefill, q_heads=q_heads, kv_heads=kv_heads, page_size=page_size, spare_pages=2)
        q, k_new, v_new, cache = inputs[:4]
        # The cache with every query token's K / V written at its position.
        updated = np.array(cache)
        sequences = len(meta.kv_lens)
        pages_per_seq = max(-(-int(length) // page_size) for length in meta.kv_lens)
        table = np.zeros((sequences, pages_per_seq), dtype=np.int32)
        for s in range(sequences):
            first = int(meta.cu_kv_lens[s]) // page_size
            count = -(-int(meta.kv_lens[s]) // page_size)
            table[s, :count] = meta.page_indices[first : first + count]
            q_len = int(meta.cu_q_lens[s + 1] - meta.cu_q_lens[s])
            for i in range(q_len):
                position = int(meta.kv_lens[s]) - q_len + i
                page = table[s, position // page_size]
                updated[page, position % page_size, :, 0] = k_new[int(meta.cu_q_lens[s]) + i]
                updated[page, position % page_size, :, 1] = v_new[int(meta.cu_q_lens[s]) + i]
        combined = updated.reshape(updated.shape[0], page_size, 2 * kv_heads, 128)  # K of head h at 2h, V at 2h + 1
        scale = 1.0 / 128
        out = module.ref_ragged_paged_attention(q, combined, meta.kv_lens.astype(np.int32), table, meta.cu_q_lens.astype(np.int32),
                                                np.array([sequences], dtype=np.int32), sm_scale=scale)
        assert out.dtype == BF16 and out.shape == q.shape
        for key, value in (("queries", q), ("keys", k_new), ("values", v_new), ("cache", cache)):
            arrays[f"{name}/{key}_bf16_bits"] = np.ascontiguousarray(value).view(np.uint16)
        for key, value in (("kv_lengths", meta.kv_lens), ("page_indices", meta.page_indices), ("cu_q_lens", meta.cu_q_lens),
                           ("cu_kv_lens", meta.cu_kv_lens), ("distribution", meta.distribution)):
            arrays[f"{name}/{key}"] = np.asarray(value)
        arrays[f"{name}/softmax_scale"] = np.float64(scale)
        arrays[f"{name}/reference_output_bf16_bits"] = np.ascontiguousarray(out).view(np.uint16)
    np.savez_compressed(HERE / "mixed_reference_vectors.npz", **arrays)
    print("wrote mixed_reference_vectors.npz", {k: v.shape for k, v in arrays.items() if k.endswith("reference_output_bf16_bits")})


if __name__ == "__main__":
    main()
