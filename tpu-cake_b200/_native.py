"""ctypes binding of libcake_b200.so (the C ABI declared in include/cake_abi.h).

There is no fallback: if the shared library has not been built, importing anything that needs
it raises. Build it with ``python -c "import __graft_entry__ as g; g.build()"`` from the
repository root (or ``python tpu-cake_b200/build_native.py``).
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_DIR / "lib" / "libcake_b200.so"

CAKE_OK = 0
CAKE_ERR_INVALID_ARGUMENT = -1
CAKE_ERR_CUDA = -2
CAKE_ERR_UNSUPPORTED = -3
CAKE_ERR_TIMEOUT = -4
CAKE_ERR_DEVICE_CHECK = -5
CAKE_ERR_STATE = -6

CAKE_DTYPE_F32 = 0
CAKE_DTYPE_BF16 = 1
CAKE_RS_LOCAL_PARTIAL = 0
CAKE_RS_P2P_OWNER_PUSH = 1
CAKE_RPA_CACHE_SEPARATE = 0
CAKE_RPA_CACHE_FUSED = 1
CAKE_RPA_TABLE_2D = 0
CAKE_RPA_TABLE_FLAT = 1
CAKE_MAX_WORLD = 8

EXPORTED_SYMBOLS = (
    "cake_abi_version",
    "cake_last_error",
    "cake_symm_alloc",
    "cake_symm_free",
    "cake_ipc_export",
    "cake_ipc_open",
    "cake_ipc_close",
    "cake_matmul_rs_create",
    "cake_matmul_rs_destroy",
    "cake_matmul_rs_partial_bytes",
    "cake_matmul_rs_slot_bytes",
    "cake_matmul_rs_flag_bytes",
    "cake_matmul_rs_bind_peers",
    "cake_matmul_rs_enqueue",
    "cake_matmul_rs_enqueue_push",
    "cake_matmul_rs_enqueue_reduce",
    "cake_matmul_rs_run_host",
    "cake_matmul_rs_status",
    "cake_matmul_rs_launches_per_enqueue",
    "cake_rpa_create",
    "cake_rpa_destroy",
    "cake_rpa_workspace_bytes",
    "cake_rpa_decode_enqueue",
    "cake_rpa_mixed_enqueue",
    "cake_rpa_decode_allgather_enqueue",
    "cake_rpa_decode_static_scratch",
    "cake_rpa_status",
    "cake_rpa_launches_per_enqueue",
)


class CakeError(RuntimeError):
    """A non-zero status from libcake_b200.so; ``code`` is the CAKE_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libcake_b200 error {code}: {message}")
        self.code = code


class CakeStatus(ctypes.Structure):
    _fields_ = [
        ("code", ctypes.c_int32),
        ("detail0", ctypes.c_int32),
        ("detail1", ctypes.c_int32),
        ("detail2", ctypes.c_int32),
    ]


class MatmulRsDesc(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int64),
        ("n", ctypes.c_int64),
        ("k_local", ctypes.c_int64),
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("scatter_dim", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("transport_dtype", ctypes.c_int32),
        ("strategy", ctypes.c_int32),
        ("tile_m", ctypes.c_int32),
        ("tile_n", ctypes.c_int32),
        ("rhs_layout", ctypes.c_int32),
        ("wait_budget_ms", ctypes.c_int32),
    ]


class RpaDesc(ctypes.Structure):
    _fields_ = [
        ("num_seqs", ctypes.c_int32),
        ("num_q_tokens", ctypes.c_int32),
        ("q_heads", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("head_dim_padded", ctypes.c_int32),
        ("page_size", ctypes.c_int32),
        ("cache_layout", ctypes.c_int32),
        ("table_layout", ctypes.c_int32),
        ("max_pages_per_seq", ctypes.c_int32),
        ("total_pages", ctypes.c_int64),
        ("sm_scale", ctypes.c_float),
        ("bias_mode", ctypes.c_int32),
        ("bias_extent", ctypes.c_int32),
        ("rel_dim", ctypes.c_int32),
        ("update_cache", ctypes.c_int32),
        ("kv_chunk_tokens", ctypes.c_int32),
        ("wait_budget_ms", ctypes.c_int32),
    ]


_lib: ctypes.CDLL | None = None


def library_path() -> Path:
    override = os.environ.get("CAKE_B200_LIBRARY")
    return Path(override) if override else LIBRARY_PATH


def load() -> ctypes.CDLL:
    """Loads the shared library once and declares every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()'). "
            "This package has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(path))
    vp, i32, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_size_t
    lib.cake_abi_version.restype = i32
    lib.cake_abi_version.argtypes = []
    lib.cake_last_error.restype = ctypes.c_char_p
    lib.cake_last_error.argtypes = []
    lib.cake_symm_alloc.restype = i32
    lib.cake_symm_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    lib.cake_symm_free.restype = i32
    lib.cake_symm_free.argtypes = [vp]
    lib.cake_ipc_export.restype = i32
    lib.cake_ipc_export.argtypes = [vp, ctypes.c_char_p]
    lib.cake_ipc_open.restype = i32
    lib.cake_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.cake_ipc_close.restype = i32
    lib.cake_ipc_close.argtypes = [vp]

    lib.cake_matmul_rs_create.restype = i32
    lib.cake_matmul_rs_create.argtypes = [ctypes.POINTER(MatmulRsDesc), ctypes.POINTER(vp)]
    lib.cake_matmul_rs_destroy.restype = i32
    lib.cake_matmul_rs_destroy.argtypes = [vp]
    for name in ("cake_matmul_rs_partial_bytes", "cake_matmul_rs_slot_bytes", "cake_matmul_rs_flag_bytes"):
        getattr(lib, name).restype = sz
        getattr(lib, name).argtypes = [vp]
    lib.cake_matmul_rs_bind_peers.restype = i32
    lib.cake_matmul_rs_bind_peers.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.cake_matmul_rs_enqueue.restype = i32
    lib.cake_matmul_rs_enqueue.argtypes = [vp, vp, vp, vp, vp]
    lib.cake_matmul_rs_enqueue_push.restype = i32
    lib.cake_matmul_rs_enqueue_push.argtypes = [vp, vp, vp, vp]
    lib.cake_matmul_rs_enqueue_reduce.restype = i32
    lib.cake_matmul_rs_enqueue_reduce.argtypes = [vp, vp, vp]
    lib.cake_matmul_rs_run_host.restype = i32
    lib.cake_matmul_rs_run_host.argtypes = [vp, vp, vp, vp, vp]
    lib.cake_matmul_rs_status.restype = i32
    lib.cake_matmul_rs_status.argtypes = [vp, vp, ctypes.POINTER(CakeStatus)]
    lib.cake_matmul_rs_launches_per_enqueue.restype = i32
    lib.cake_matmul_rs_launches_per_enqueue.argtypes = [vp]

    lib.cake_rpa_create.restype = i32
    lib.cake_rpa_create.argtypes = [ctypes.POINTER(RpaDesc), ctypes.POINTER(vp)]
    lib.cake_rpa_destroy.restype = i32
    lib.cake_rpa_destroy.argtypes = [vp]
    lib.cake_rpa_workspace_bytes.restype = sz
    lib.cake_rpa_workspace_bytes.argtypes = [vp]
    lib.cake_rpa_decode_enqueue.restype = i32
    lib.cake_rpa_decode_enqueue.argtypes = [vp] + [vp] * 12 + [vp]
    lib.cake_rpa_mixed_enqueue.restype = i32
    lib.cake_rpa_mixed_enqueue.argtypes = [vp] * 10 + [i32, vp, vp, vp]
    lib.cake_rpa_decode_allgather_enqueue.restype = i32
    lib.cake_rpa_decode_allgather_enqueue.argtypes = (
        [vp] * 11 + [ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, i32, vp, vp]
    )
    lib.cake_rpa_decode_static_scratch.restype = i32
    lib.cake_rpa_decode_static_scratch.argtypes = [ctypes.POINTER(RpaDesc)] + [vp] * 13
    lib.cake_rpa_status.restype = i32
    lib.cake_rpa_status.argtypes = [vp, vp, ctypes.POINTER(CakeStatus)]
    lib.cake_rpa_launches_per_enqueue.restype = i32
    lib.cake_rpa_launches_per_enqueue.argtypes = [vp]
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raises CakeError with the library's message for a non-zero status."""
    if code != CAKE_OK:
        message = load().cake_last_error()
        raise CakeError(code, message.decode() if message else "")
