"""The C-ABI library loads, exports what include/cake_abi.h declares, and validates arguments
without touching a GPU."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from tpu_cake_b200 import _native

ROOT = Path(__file__).resolve().parent.parent


def declared_functions() -> list[str]:
    header = (ROOT / "include" / "cake_abi.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(cake_[a-z0-9_]+)\s*\(", header)))


def test_header_declares_only_exported_symbols():
    lib = _native.load()
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/cake_abi.h but not exported"
    assert sorted(_native.EXPORTED_SYMBOLS) == names


def test_abi_version_and_error_text():
    lib = _native.load()
    assert lib.cake_abi_version() == 1
    assert isinstance(lib.cake_last_error(), bytes)


def test_struct_layouts_match_header():
    # 3 x int64 + 10 x int32 and 10 x int32 + int64 + float + 7 x int32, naturally aligned.
    assert ctypes.sizeof(_native.MatmulRsDesc) == 64
    assert ctypes.sizeof(_native.RpaDesc) == 80
    assert ctypes.sizeof(_native.CakeStatus) == 16


@pytest.mark.parametrize(
    "overrides, code, fragment",
    [
        ({"m": 0}, _native.CAKE_ERR_INVALID_ARGUMENT, "positive"),
        ({"world": 9}, _native.CAKE_ERR_INVALID_ARGUMENT, "bad mesh"),
        ({"rank": 2, "world": 2}, _native.CAKE_ERR_INVALID_ARGUMENT, "bad mesh"),
        ({"scatter_dim": 2}, _native.CAKE_ERR_INVALID_ARGUMENT, "scatter_dim"),
        ({"tile_m": 64}, _native.CAKE_ERR_UNSUPPORTED, "tile_m"),
        ({"tile_n": 96}, _native.CAKE_ERR_UNSUPPORTED, "tile_n"),
        ({"k_local": 100}, _native.CAKE_ERR_UNSUPPORTED, "multiple of 8"),
        ({"world": 8, "m": 100, "scatter_dim": 0}, _native.CAKE_ERR_INVALID_ARGUMENT, "divisible"),
        ({"out_dtype": 7}, _native.CAKE_ERR_INVALID_ARGUMENT, "dtype"),
    ],
)
def test_matmul_create_rejects_bad_descriptors(overrides, code, fragment):
    lib = _native.load()
    fields = dict(m=128, n=256, k_local=64, world=1, rank=0, scatter_dim=1, out_dtype=0, transport_dtype=0,
                  strategy=0, tile_m=128, tile_n=128, rhs_layout=0, wait_budget_ms=0)
    fields.update(overrides)
    desc = _native.MatmulRsDesc(**fields)
    handle = ctypes.c_void_p()
    assert lib.cake_matmul_rs_create(ctypes.byref(desc), ctypes.byref(handle)) == code
    assert fragment in lib.cake_last_error().decode()
    with pytest.raises(_native.CakeError) as raised:
        _native.check(code)
    assert raised.value.code == code


@pytest.mark.parametrize(
    "overrides, code, fragment",
    [
        ({"num_q_tokens": 7}, _native.CAKE_ERR_INVALID_ARGUMENT, "query tokens for"),
        ({"q_heads": 6, "kv_heads": 4}, _native.CAKE_ERR_INVALID_ARGUMENT, "multiple of kv_heads"),
        ({"q_heads": 36, "kv_heads": 2}, _native.CAKE_ERR_UNSUPPORTED, "at most 8"),
        ({"head_dim": 256, "head_dim_padded": 256}, _native.CAKE_ERR_UNSUPPORTED, "head_dim"),
        ({"page_size": 24}, _native.CAKE_ERR_UNSUPPORTED, "page_size"),
        ({"cache_layout": 0, "head_dim": 64}, _native.CAKE_ERR_UNSUPPORTED, "head_dim 128"),
        ({"kv_chunk_tokens": 48}, _native.CAKE_ERR_INVALID_ARGUMENT, "kv_chunk_tokens"),
        ({"bias_mode": 1, "bias_extent": 0}, _native.CAKE_ERR_INVALID_ARGUMENT, "bias_extent"),
    ],
)
def test_rpa_create_rejects_bad_descriptors(overrides, code, fragment):
    lib = _native.load()
    fields = dict(num_seqs=8, num_q_tokens=8, q_heads=8, kv_heads=2, head_dim=128, head_dim_padded=128, page_size=16,
                  cache_layout=1, table_layout=0, max_pages_per_seq=4, total_pages=64, sm_scale=0.1, bias_mode=0,
                  bias_extent=0, rel_dim=0, update_cache=0, kv_chunk_tokens=0, wait_budget_ms=0)
    fields.update(overrides)
    desc = _native.RpaDesc(**fields)
    handle = ctypes.c_void_p()
    assert lib.cake_rpa_create(ctypes.byref(desc), ctypes.byref(handle)) == code
    assert fragment in lib.cake_last_error().decode()


def test_null_arguments_are_errors_not_crashes():
    lib = _native.load()
    assert lib.cake_matmul_rs_create(None, None) == _native.CAKE_ERR_INVALID_ARGUMENT
    assert lib.cake_rpa_create(None, None) == _native.CAKE_ERR_INVALID_ARGUMENT
    assert lib.cake_matmul_rs_destroy(None) == _native.CAKE_OK
    assert lib.cake_rpa_destroy(None) == _native.CAKE_OK
    assert lib.cake_symm_alloc(0, None) == _native.CAKE_ERR_INVALID_ARGUMENT
