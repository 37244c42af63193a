"""Builder of a global data x tensor sharded decode problem for the surface tests."""

from __future__ import annotations

import numpy as np

from tests.helpers import BF16


def build_sharded_surface(seed, *, data=2, tensor=4, local_seqs=4, local_q_heads=8, local_kv_heads=4, page_size=1,
                          contexts=(128, 512, 1024, 700), relative_dim=16, extent=512):
    """Global inputs whose ``data`` blocks are self-contained: block d owns sequences, pages, page
    indices (numbered inside the block), cumulative arrays starting at 0 and its own distribution
    triple, as a shard_map over the data axis would hand them out."""
    generator = np.random.default_rng(seed)
    q_heads, kv_heads = local_q_heads * tensor, local_kv_heads * tensor
    blocks = []
    for _ in range(data):
        lens = np.array(contexts[:local_seqs], dtype=np.int32)
        pages_per = -(-lens.astype(np.int64) // page_size)
        local_pages = int(pages_per.sum()) + 8
        page_slots = int(pages_per.sum()) + 16
        indices = np.zeros(page_slots, dtype=np.int32)
        indices[: int(pages_per.sum())] = generator.permutation(local_pages)[: int(pages_per.sum())]
        cu_kv = np.concatenate([[0], np.cumsum(pages_per * page_size)]).astype(np.int32)
        blocks.append({
            "q": generator.normal(size=(local_seqs, q_heads, 128)).astype(np.float32).astype(BF16),
            "k": generator.normal(size=(local_seqs, kv_heads, 128)).astype(np.float32).astype(BF16),
            "v": generator.normal(size=(local_seqs, kv_heads, 128)).astype(np.float32).astype(BF16),
            "cache": generator.normal(size=(local_pages, page_size, kv_heads, 2, 128)).astype(np.float32).astype(BF16),
            "lens": lens, "pages": indices, "cu_q": np.arange(local_seqs + 1, dtype=np.int32), "cu_kv": cu_kv,
            "dist": np.full(3, local_seqs, dtype=np.int32),
            "states": generator.normal(scale=0.3, size=(local_seqs, q_heads, relative_dim)).astype(np.float32).astype(BF16),
        })
    projection = generator.normal(scale=0.3, size=(relative_dim, extent)).astype(np.float32).astype(BF16)
    names = ("q", "k", "v", "cache", "lens", "pages", "cu_q", "cu_kv", "dist", "states")
    global_inputs = tuple(np.concatenate([block[name] for block in blocks], axis=0) for name in names) + (projection,)
    block_inputs = [tuple(block[name] for name in names) + (projection,) for block in blocks]
    return global_inputs, block_inputs
