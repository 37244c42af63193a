"""The allocation-free decode entry point against the regular one.

Some hosts of this library cannot allocate device memory at all: a plugin inside a serving engine
that owns the only allocator, or a loop whose memory pool is frozen once serving starts. For them
``cake_rpa_decode_static_scratch`` keeps the split-KV scratch in an array built into the library.
This test calls it through the C ABI, twice in a row with different inputs (the second call finds
the first call's leftovers in the shared array), and requires the same bits as
``cake_rpa_decode_enqueue`` produces with a caller-provided workspace. It lives in a file that
sorts last so that a run stopping at the first failure has already run every other test, and it
does not depend on any other test having run.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import matmul_rs as metrics
from oracle import rpa as oracle
from tests.helpers import BF16, to_device, torch_to_bf16
from tpu_cake_b200 import _native

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 16 << 20


def make_case(seed: int, lengths: list[int], *, q_heads=8, kv_heads=2, page_size=16, pool=160):
    generator = np.random.default_rng(seed)
    count = len(lengths)
    query = generator.normal(size=(count, q_heads, 128)).astype(np.float32).astype(BF16)
    keys = generator.normal(size=(pool, page_size, kv_heads, 128)).astype(np.float32).astype(BF16)
    values = generator.normal(size=(pool, page_size, kv_heads, 128)).astype(np.float32).astype(BF16)
    lens = np.asarray(lengths, dtype=np.int32)
    pages = -(-lens.astype(np.int64) // page_size)
    table = np.zeros((count, int(pages.max())), dtype=np.int32)
    permutation = generator.permutation(pool)
    cursor = 0
    for s in range(count):
        table[s, : pages[s]] = permutation[cursor : cursor + pages[s]]
        cursor += int(pages[s])
    return query, keys, values, table, lens


def descriptor(case, chunk: int) -> _native.RpaDesc:
    query, keys, _values, table, _lens = case
    return _native.RpaDesc(
        num_seqs=query.shape[0], num_q_tokens=query.shape[0], q_heads=query.shape[1], kv_heads=keys.shape[2], head_dim=128,
        head_dim_padded=128, page_size=keys.shape[1], cache_layout=_native.CAKE_RPA_CACHE_SEPARATE,
        table_layout=_native.CAKE_RPA_TABLE_2D, max_pages_per_seq=table.shape[1], total_pages=keys.shape[0],
        sm_scale=1.0 / math.sqrt(128), bias_mode=0, bias_extent=0, rel_dim=0, update_cache=0, kv_chunk_tokens=chunk, wait_budget_ms=0,
    )


def test_static_scratch_decode_matches_workspace_decode_twice(cuda_device):
    lib = _native.load()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    # Two different problems back to back: split-KV with several chunks per sequence, then a
    # different batch with other lengths, so stale partials from the first call sit in the array.
    for seed, lengths, chunk in ((1, [700, 33, 1200], 256), (2, [90, 1500, 17, 512], 128)):
        case = make_case(seed, lengths)
        query, keys, values, table, lens = (to_device(a, cuda_device) for a in case)
        desc = descriptor(case, chunk)

        handle = ctypes.c_void_p()
        _native.check(lib.cake_rpa_create(ctypes.byref(desc), ctypes.byref(handle)))
        workspace = torch.empty(lib.cake_rpa_workspace_bytes(handle), dtype=torch.uint8, device=cuda_device)
        assert workspace.numel() <= STATIC_SCRATCH_BYTES
        expected = torch.full_like(query, float("nan"))
        _native.check(lib.cake_rpa_decode_enqueue(
            handle, query.data_ptr(), None, None, keys.data_ptr(), values.data_ptr(), lens.data_ptr(), table.data_ptr(),
            None, None, None, expected.data_ptr(), workspace.data_ptr(), stream))
        word = _native.CakeStatus()
        _native.check(lib.cake_rpa_status(handle, stream, ctypes.byref(word)))
        lib.cake_rpa_destroy(handle)

        actual = torch.full_like(query, float("nan"))
        _native.check(lib.cake_rpa_decode_static_scratch(
            ctypes.byref(desc), query.data_ptr(), None, None, keys.data_ptr(), values.data_ptr(), lens.data_ptr(),
            table.data_ptr(), None, None, None, actual.data_ptr(), status.data_ptr(), stream))
        torch.cuda.synchronize(cuda_device)
        assert status.cpu().tolist() == [0, 0, 0, 0]
        assert torch.equal(actual.view(torch.uint16), expected.view(torch.uint16))
        reference = oracle.rpa_separate(*case[:3], case[3], case[4], None, scale=1.0 / math.sqrt(128))
        got = torch_to_bf16(actual).astype(np.float32)
        assert metrics.max_abs_error(got, reference) <= 2e-2 and metrics.relative_l2_error(got, reference) <= 1e-2


def test_static_scratch_rejects_shapes_beyond_its_array(cuda_device):
    lib = _native.load()
    desc = _native.RpaDesc(
        num_seqs=256, num_q_tokens=256, q_heads=64, kv_heads=8, head_dim=128, head_dim_padded=128, page_size=32,
        cache_layout=_native.CAKE_RPA_CACHE_FUSED, table_layout=_native.CAKE_RPA_TABLE_2D, max_pages_per_seq=1024,
        total_pages=262144, sm_scale=0.1, bias_mode=0, bias_extent=0, rel_dim=0, update_cache=0, kv_chunk_tokens=0, wait_budget_ms=0,
    )
    code = lib.cake_rpa_decode_static_scratch(ctypes.byref(desc), *([None] * 13))
    assert code == _native.CAKE_ERR_UNSUPPORTED
    message = lib.cake_last_error().decode()
    assert "static scratch" in message and "bytes" in message
