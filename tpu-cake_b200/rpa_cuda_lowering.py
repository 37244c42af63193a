"""CUDA backend lowering of Inkling ragged paged attention (decode, and mixed prefill/decode batches).

Mirror of the reference's RPA backend (src/tpu_cake/rpa_lowering.py):
  - ``CudaFusedRpaPlan`` has the tensor-contract fields of ``FusedRpaPlan`` (:131-170) and its
    ``preflight`` / ``invoke`` / ``run_preflighted`` methods (:228-288). ``invoke`` runs the
    sm_100a kernels instead of handing the inputs to a pinned external JAX kernel.
  - ``preflight_decode_metadata`` is the integer validation of ``_preflight_decode_metadata``
    (:71-128), same checks, same messages.
  - ``CudaMixedRpaPlan`` / ``preflight_mixed_metadata`` extend the same contract to batches whose
    sequences carry more than one query token, which the reference's adapter rejects (:76-86): decode
    sequences first, then prefill sequences, as its ``distribution`` triple orders them
    (src/tpu_cake/rpa_owned_kernel.py:58-67).
  - ``CudaPagedAttentionPlan`` lowers the prototype op ``tpu_schedule.ragged_paged_attention``
    (separate K / V caches, 2-D page table, dense bias;
    src/tpu_cake/dialects/tpu_schedule.py:2003-2103), which has no lowering in the reference.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from . import _native
from .identity import text_sha256

FUSED_INPUT_NAMES = (
    "queries",
    "keys",
    "values",
    "fused_cache",
    "kv_lengths",
    "page_indices",
    "cumulative_query_lengths",
    "cumulative_kv_lengths",
    "distribution",
    "relative_states",
    "relative_projection",
)


def preflight_decode_metadata(inputs: tuple, input_shapes: tuple[tuple[int, ...], ...]) -> None:
    """Rejects decode metadata the kernel must not be run on. Integer arithmetic in int64 on the
    host; raises ValueError with the reference's messages."""
    lengths = np.asarray(_to_host(inputs[4]), dtype=np.int64)
    page_indices = np.asarray(_to_host(inputs[5]), dtype=np.int64)
    cu_q = np.asarray(_to_host(inputs[6]), dtype=np.int64)
    cu_kv = np.asarray(_to_host(inputs[7]), dtype=np.int64)
    distribution = np.asarray(_to_host(inputs[8]), dtype=np.int64)
    count = input_shapes[4][0]
    if distribution.shape != (3,) or np.any(distribution != count):
        raise ValueError(
            "Inkling fused RPA adapter accepts decode-only distribution "
            f"{(count,) * 3}, got {tuple(int(v) for v in distribution)}"
        )
    if cu_q.shape != (count + 1,) or np.any(cu_q != np.arange(count + 1)):
        raise ValueError("Inkling fused RPA adapter requires one query token per sequence")
    if np.any(lengths <= 0):
        raise ValueError("Inkling fused RPA requires positive KV lengths")
    total_pages, page_size = input_shapes[3][0], input_shapes[3][1]
    if np.any(lengths > total_pages * page_size):
        raise ValueError("fused RPA KV length exceeds total cache capacity")
    padded = -(-lengths // page_size) * page_size
    expected_cu_kv = np.zeros(count + 1, dtype=np.int64)
    np.cumsum(padded, out=expected_cu_kv[1:])
    if cu_kv.shape != expected_cu_kv.shape or np.any(cu_kv != expected_cu_kv):
        raise ValueError("fused RPA cumulative KV lengths must be page-aligned")
    needed = int(expected_cu_kv[-1]) // page_size
    if needed > page_indices.size:
        raise ValueError("fused RPA page table cannot cover all KV lengths")
    used = page_indices[:needed]
    if np.any(used < 0) or np.any(used >= total_pages):
        raise ValueError("fused RPA page index is outside the fused cache")
    per_sequence: list[np.ndarray] = []
    for s in range(count):
        pages = page_indices[int(cu_kv[s]) // page_size : int(cu_kv[s + 1]) // page_size]
        if np.unique(pages).size != pages.size:
            raise ValueError("fused RPA page table aliases logical pages within one sequence")
        per_sequence.append(pages)
    writes = []
    for s in range(count):
        last = int(lengths[s]) - 1
        page = int(page_indices[int(cu_kv[s]) // page_size + last // page_size])
        writes.append((page, last % page_size))
    if len(set(writes)) != len(writes):
        raise ValueError("fused RPA decode updates collide in the physical cache")
    for writer, (page, _slot) in enumerate(writes):
        for reader, pages in enumerate(per_sequence):
            if reader != writer and page in pages:
                raise ValueError("fused RPA active write page is shared across sequences")


def preflight_mixed_metadata(inputs: tuple, input_shapes: tuple[tuple[int, ...], ...]) -> int:
    """Integer validation of a ragged batch, in int64 on the host, in the style of
    ``preflight_decode_metadata``. Returns the number of leading decode sequences."""
    lengths = np.asarray(_to_host(inputs[4]), dtype=np.int64)
    page_indices = np.asarray(_to_host(inputs[5]), dtype=np.int64)
    cu_q = np.asarray(_to_host(inputs[6]), dtype=np.int64)
    cu_kv = np.asarray(_to_host(inputs[7]), dtype=np.int64)
    distribution = np.asarray(_to_host(inputs[8]), dtype=np.int64)
    tokens = input_shapes[0][0]
    count = input_shapes[4][0]
    if distribution.shape != (3,) or not (0 <= distribution[0] <= distribution[1] <= distribution[2] == count):
        raise ValueError(f"ragged RPA distribution must be (decode end, prefill end, {count}), got {tuple(int(v) for v in distribution)}")
    if cu_q.shape != (count + 1,) or cu_q[0] != 0 or np.any(np.diff(cu_q) < 1) or cu_q[-1] != tokens:
        raise ValueError("ragged RPA cumulative query lengths must start at 0, grow by at least one per sequence and end at the token count")
    q_lens = np.diff(cu_q)
    decode_end = int(distribution[0])
    if np.any(q_lens[:decode_end] != 1):
        raise ValueError("ragged RPA decode sequences must come first with one query token each")
    if np.any(lengths <= 0) or np.any(lengths < q_lens):
        raise ValueError("ragged RPA KV lengths must be positive and include the query tokens")
    total_pages, page_size = input_shapes[3][0], input_shapes[3][1]
    if np.any(lengths > total_pages * page_size):
        raise ValueError("fused RPA KV length exceeds total cache capacity")
    padded = -(-lengths // page_size) * page_size
    expected_cu_kv = np.zeros(count + 1, dtype=np.int64)
    np.cumsum(padded, out=expected_cu_kv[1:])
    if cu_kv.shape != expected_cu_kv.shape or np.any(cu_kv != expected_cu_kv):
        raise ValueError("fused RPA cumulative KV lengths must be page-aligned")
    needed = int(expected_cu_kv[-1]) // page_size
    if needed > page_indices.size:
        raise ValueError("fused RPA page table cannot cover all KV lengths")
    used = page_indices[:needed]
    if np.any(used < 0) or np.any(used >= total_pages):
        raise ValueError("fused RPA page index is outside the fused cache")
    # Every sequence writes its new tokens, so no physical page may be shared at all.
    if np.unique(used).size != used.size:
        raise ValueError("ragged RPA page table aliases a physical page")
    return decode_end


class UnsupportedRpaLowering(ValueError):
    """A physical RPA kernel the CUDA backend does not lower (mirrors UnsupportedRpaLoweringError,
    src/tpu_cake/rpa_lowering.py:37-38)."""


def _single_op(module, name: str):
    module.verify()
    if len(module.ops) != 1 or module.ops[0].name != "tpu_schedule.kernel":
        raise UnsupportedRpaLowering("expected one physical kernel")
    kernel = module.ops[0]
    matches = [op for op in kernel.body.ops if op.name == name]
    if len(matches) != 1:
        raise UnsupportedRpaLowering(f"expected exactly one {name} in the kernel, found {len(matches)}")
    return kernel, matches[0]


def lower_paged_attention_to_cuda(module, *, softmax_scale: float | None = None, kv_chunk_tokens: int = 0) -> "CudaPagedAttentionPlan":
    """``tpu_schedule.ragged_paged_attention`` -> CUDA decode plan. The reference only renders this
    op's contract (src/tpu_cake/cli.py:667-676); here it gets an executable lowering. The softmax
    scale is not a property of the op: the reference oracle's 1/head_dim is the default."""
    from .ir import schedule_sha256

    kernel, op = _single_op(module, "tpu_schedule.ragged_paged_attention")
    query, key_cache, value_cache, page_table, _lengths, bias, _output = (value.type for value in op.operands)
    if key_cache.shape != value_cache.shape:
        raise UnsupportedRpaLowering("key and value caches must have one shape")
    if key_cache.element_type != "bf16" or query.element_type != "bf16":
        raise UnsupportedRpaLowering("the CUDA decode kernels take bf16 queries and caches")
    if query.shape[2] != 128:
        raise UnsupportedRpaLowering("separate K / V caches are lowered for head_dim 128")
    return CudaPagedAttentionPlan(
        name=kernel.properties["sym_name"], schedule_sha256=schedule_sha256(module), query_shape=tuple(query.shape),
        cache_shape=tuple(key_cache.shape), page_table_shape=tuple(page_table.shape), bias_shape=tuple(bias.shape),
        softmax_scale=softmax_scale if softmax_scale is not None else 1.0 / query.shape[2], kv_chunk_tokens=kv_chunk_tokens,
    )


def lower_fused_rpa_to_cuda(module, *, with_relative_bias: bool = True, kv_chunk_tokens: int = 0):
    """``tpu_schedule.fused_ragged_paged_attention`` -> ``CudaFusedRpaPlan`` (one query token per
    sequence) or ``CudaMixedRpaPlan`` (ragged query runs; relative bias not lowered). Mirrors
    ``lower_fused_rpa_kernel`` (src/tpu_cake/rpa_lowering.py:291-392)."""
    from .ir import schedule_sha256

    kernel, op = _single_op(module, "tpu_schedule.fused_ragged_paged_attention")
    if op.properties["sliding_window"] != 0:
        raise UnsupportedRpaLowering("sliding-window attention is not lowered by the CUDA backend")
    types = [value.type for value in op.operands]
    q, k, _v, cache, lens, pages = types[:6]
    states, projection = types[9], types[10]
    scale = float(op.properties["softmax_scale"])
    if q.shape[0] == lens.shape[0]:
        return CudaFusedRpaPlan(
            name=kernel.properties["sym_name"], schedule_sha256=schedule_sha256(module), query_shape=tuple(q.shape),
            key_shape=tuple(k.shape), value_shape=tuple(k.shape), fused_cache_shape=tuple(cache.shape), kv_lengths_shape=tuple(lens.shape),
            page_indices_shape=tuple(pages.shape), cumulative_query_lengths_shape=(lens.shape[0] + 1,),
            cumulative_kv_lengths_shape=(lens.shape[0] + 1,), distribution_shape=(3,),
            relative_states_shape=tuple(states.shape) if with_relative_bias else None,
            relative_projection_shape=tuple(projection.shape) if with_relative_bias else None, output_shape=tuple(q.shape),
            softmax_scale=scale, kv_chunk_tokens=kv_chunk_tokens,
        )
    return CudaMixedRpaPlan(
        name=kernel.properties["sym_name"], schedule_sha256=schedule_sha256(module), query_shape=tuple(q.shape), key_shape=tuple(k.shape),
        fused_cache_shape=tuple(cache.shape), sequences=lens.shape[0], page_indices_shape=tuple(pages.shape), softmax_scale=scale,
        kv_chunk_tokens=kv_chunk_tokens,
    )


def lower_inkling_rpa_to_cuda(module, *, with_relative_bias: bool = True, kv_chunk_tokens: int = 0):
    """The name the reference's callers use (``lower_inkling_rpa_to_pallas``,
    src/tpu_cake/rpa_lowering.py:1084): fused-RPA kernel -> ``CudaFusedRpaPlan`` with ``preflight`` /
    ``invoke`` / ``run_preflighted`` (:228-288)."""
    return lower_fused_rpa_to_cuda(module, with_relative_bias=with_relative_bias, kv_chunk_tokens=kv_chunk_tokens)


def lower_inkling_sharded_rpa_to_cuda(module, *, kv_chunk_tokens: int = 0) -> "ShardedCudaFusedRpaPlan":
    """Counterpart of ``lower_inkling_sharded_rpa_to_pallas`` (src/tpu_cake/rpa_lowering.py:1139): the
    kernel describes one mesh position's shard and names a ``data`` x ``tensor`` mesh; the result
    places global inputs (``place_inputs``) and builds the local executable (``build_executable``)."""
    kernel, _ = _single_op(module, "tpu_schedule.fused_ragged_paged_attention")
    axes, sizes = tuple(kernel.properties["mesh_axis_names"]), tuple(kernel.properties["mesh_axis_sizes"])
    if axes != ("data", "tensor"):
        raise UnsupportedRpaLowering(f"sharded RPA runs on a data x tensor mesh, the kernel names {axes}")
    local = lower_fused_rpa_to_cuda(module, kv_chunk_tokens=kv_chunk_tokens)
    if not isinstance(local, CudaFusedRpaPlan):
        raise UnsupportedRpaLowering("the sharded surface lowers decode batches (one query token per sequence)")
    return ShardedCudaFusedRpaPlan(local_plan=local, mesh_axes=axes, mesh_shape=sizes)


def default_kv_chunk_tokens(kv_heads: int) -> int:
    """The library's split-KV chunk when a plan asks for none: 512 tokens, 1024 with one or two KV
    heads on the GPU (the chunk search on the KV-head-sharded decode's per-rank shapes)."""
    return 1024 if kv_heads <= 2 else 512


def decode_resource_contract(plan) -> dict:
    """Properties of a ``tpu_schedule.cuda_rpa_decode`` op for a decode plan: the static resources of
    the sm_100a decode kernel as built (6 worker warps, 2-stage rings of 32-token stages)."""
    warps, stages, stage_tokens, row_bytes = 6, 2, 32, 256
    batch, q_heads = plan.query_shape[0], plan.query_shape[1]
    kv_heads = plan.key_shape[1] if hasattr(plan, "key_shape") else plan.cache_shape[2]
    chunk = plan.kv_chunk_tokens or default_kv_chunk_tokens(kv_heads)
    shared = warps * (stages * stage_tokens * 2 * row_bytes + 8 * row_bytes) + 1024 + 256
    return {"kv_chunk_tokens": chunk, "warps_per_cta": warps, "ring_stages": stages, "stage_tokens": stage_tokens,
            "shared_memory_bytes": shared, "workspace_bytes": max(1, batch * q_heads * 130 * 4)}


def _to_device_tensor(value, device: torch.device) -> torch.Tensor:
    """numpy (bfloat16 via ml_dtypes included) or torch value -> contiguous tensor on ``device``, bits unchanged."""
    if isinstance(value, torch.Tensor):
        return value.to(device).contiguous()
    array = np.ascontiguousarray(value)
    if array.dtype.name == "bfloat16":
        return torch.from_numpy(array.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(array.copy()).to(device)


def surface_errors(actual: np.ndarray, expected: np.ndarray) -> tuple[float, float]:
    """(max-abs, relative-L2) in float64, the error metrics of the reference's surface runner
    (src/tpu_cake/rpa_surface_runner.py:394-411); shape / dtype mismatches and non-finite values are errors."""
    import math

    if actual.shape != expected.shape or actual.dtype != expected.dtype:
        raise ValueError(f"SHARDED_RPA_OUTPUT_ABI_MISMATCH actual={actual.shape}/{actual.dtype} expected={expected.shape}/{expected.dtype}")
    a, e = actual.astype(np.float64), expected.astype(np.float64)
    if not np.all(np.isfinite(a)) or not np.all(np.isfinite(e)):
        raise ValueError("SHARDED_RPA_OUTPUT_NONFINITE")
    difference = a - e
    maximum = float(np.abs(difference).max()) if difference.size else 0.0
    relative = math.sqrt(math.fsum((difference.ravel() ** 2).tolist()) / max(math.fsum((e.ravel() ** 2).tolist()), 1e-60))
    return maximum, round(relative, 15)


def _to_host(value):
    if isinstance(value, torch.Tensor):
        return value.detach().cpu().numpy()
    return value


class RpaDecodeExecutable:
    """Owns one native decode plan and its split-KV workspace on the current GPU."""

    def __init__(self, desc: _native.RpaDesc, device: torch.device):
        self._lib = _native.load()
        self.device = device
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _native.check(self._lib.cake_rpa_create(ctypes.byref(desc), ctypes.byref(handle)))
        self._handle = handle
        self.workspace = torch.empty(self._lib.cake_rpa_workspace_bytes(handle), dtype=torch.uint8, device=device)
        self.gather_calls = 0  # all-gather calls made so far: call n fills half n & 1 of the gathered buffers

    def enqueue(self, q, new_k, new_v, cache0, cache1, kv_lens, page_table, cu_kv_lens, bias0, bias1, out) -> None:
        def ptr(t):
            return None if t is None else t.data_ptr()

        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):  # the library launches on the current device
            _native.check(
                self._lib.cake_rpa_decode_enqueue(
                    self._handle, ptr(q), ptr(new_k), ptr(new_v), ptr(cache0), ptr(cache1), ptr(kv_lens),
                    ptr(page_table), ptr(cu_kv_lens), ptr(bias0), ptr(bias1), ptr(out), self.workspace.data_ptr(), stream,
                )
            )

    def enqueue_mixed(self, q, new_k, new_v, cache0, cache1, kv_lens, page_table, cu_kv_lens, cu_q_lens, num_decode_seqs: int, out) -> None:
        """Ragged batch: ``num_decode_seqs`` one-token sequences first, prefill sequences after."""
        def ptr(t):
            return None if t is None else t.data_ptr()

        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _native.check(
                self._lib.cake_rpa_mixed_enqueue(
                    self._handle, ptr(q), ptr(new_k), ptr(new_v), ptr(cache0), ptr(cache1), ptr(kv_lens), ptr(page_table),
                    ptr(cu_kv_lens), ptr(cu_q_lens), int(num_decode_seqs), ptr(out), self.workspace.data_ptr(), stream,
                )
            )

    def enqueue_allgather(self, q, cache0, cache1, kv_lens, page_table, gathered_pointers: list[int], flag_pointers: list[int],
                          world: int, rank: int, *, wait: bool = True) -> int:
        """Decode this rank's KV-head shard and write its outputs into every rank's gathered buffer
        (``gathered_pointers[r]`` / ``flag_pointers[r]``: rank r's buffers as mapped in this process).
        The buffers hold two halves of [world, num_seqs, q_heads, head_dim]; returns the half this
        call fills (calls alternate, so a consumer of one call can still read while the next runs)."""
        array = ctypes.c_void_p * world
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _native.check(
                self._lib.cake_rpa_decode_allgather_enqueue(
                    self._handle, q.data_ptr(), None, None, cache0.data_ptr(), None if cache1 is None else cache1.data_ptr(),
                    kv_lens.data_ptr(), page_table.data_ptr(), None, None, None, array(*gathered_pointers), array(*flag_pointers),
                    world, rank, 1 if wait else 0, self.workspace.data_ptr(), stream,
                )
            )
        self.gather_calls += 1
        return self.gather_calls & 1

    def status(self) -> tuple[int, int, int, int]:
        word = _native.CakeStatus()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _native.check(self._lib.cake_rpa_status(self._handle, stream, ctypes.byref(word)))
        return (word.code, word.detail0, word.detail1, word.detail2)

    @property
    def launches_per_call(self) -> int:
        return int(self._lib.cake_rpa_launches_per_enqueue(self._handle))

    def close(self) -> None:
        if self._handle:
            torch.cuda.synchronize(self.device)
            self._lib.cake_rpa_destroy(self._handle)
            self._handle = None


def _require(tensor: torch.Tensor, shape: tuple[int, ...], dtype: torch.dtype, name: str, device: torch.device) -> None:
    if not isinstance(tensor, torch.Tensor) or tuple(tensor.shape) != tuple(shape) or tensor.dtype != dtype:
        got = (tuple(tensor.shape), tensor.dtype) if isinstance(tensor, torch.Tensor) else type(tensor)
        raise ValueError(f"{name} must be a {dtype} tensor of shape {tuple(shape)}, got {got}")
    if tensor.device != device or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous on {device}")


@dataclass(frozen=True)
class CudaFusedRpaPlan:
    name: str
    schedule_sha256: str
    query_shape: tuple[int, ...]
    key_shape: tuple[int, ...]
    value_shape: tuple[int, ...]
    fused_cache_shape: tuple[int, ...]
    kv_lengths_shape: tuple[int, ...]
    page_indices_shape: tuple[int, ...]
    cumulative_query_lengths_shape: tuple[int, ...]
    cumulative_kv_lengths_shape: tuple[int, ...]
    distribution_shape: tuple[int, ...]
    relative_states_shape: tuple[int, ...] | None
    relative_projection_shape: tuple[int, ...] | None
    output_shape: tuple[int, ...]
    softmax_scale: float
    causal: int = 1
    softmax_dtype: str = "float32"
    sliding_window: int = 0
    kv_chunk_tokens: int = 0
    wait_budget_ms: int = 0  # bound on the all-gather flag barrier (0 = 20 s)
    update_cache: bool = True
    execution_scope: str = "local-shard-caller-owned-sharding"

    def __post_init__(self) -> None:
        tokens, q_heads, dim = self.query_shape
        pages, page_size, combined, pack, dim_padded = self.fused_cache_shape
        if pack != 2:
            raise ValueError("fused cache must interleave K and V with pack = 2")
        kv_heads = self.key_shape[1]
        if combined * pack != 2 * kv_heads or self.value_shape != self.key_shape:
            raise ValueError("fused cache head axis must hold K and V of every KV head")
        if self.key_shape != (tokens, kv_heads, dim) or self.output_shape != self.query_shape:
            raise ValueError("new key / value and output shapes must match the query tokens")
        if self.kv_lengths_shape != (tokens,) or self.cumulative_kv_lengths_shape != (tokens + 1,):
            raise ValueError("decode needs one KV length per query token (tokens == sequences)")
        if self.sliding_window != 0:
            raise ValueError("sliding-window attention is not lowered by the CUDA backend")
        if self.softmax_dtype != "float32":
            raise ValueError("softmax runs in float32")
        if (self.relative_states_shape is None) != (self.relative_projection_shape is None):
            raise ValueError("relative states and projection come together")

    @property
    def input_shapes(self) -> tuple[tuple[int, ...] | None, ...]:
        return (
            self.query_shape, self.key_shape, self.value_shape, self.fused_cache_shape, self.kv_lengths_shape,
            self.page_indices_shape, self.cumulative_query_lengths_shape, self.cumulative_kv_lengths_shape,
            self.distribution_shape, self.relative_states_shape, self.relative_projection_shape,
        )

    def render_executable_source(self) -> str:
        lines = ["# cake-b200 lowered fused ragged paged attention (decode)", f"name = {self.name!r}",
                 f"schedule_sha256 = {self.schedule_sha256!r}",
                 "kernels = ('cake_rpa_plan_sm100', 'cake_rpa_cache_update_sm100', 'cake_rpa_decode_sm100', 'cake_rpa_combine_sm100')"]
        for name, shape in zip(FUSED_INPUT_NAMES, self.input_shapes, strict=True):
            lines.append(f"{name}_shape = {shape}")
        lines += [f"softmax_scale = {self.softmax_scale!r}", f"causal = {self.causal}", f"sliding_window = {self.sliding_window}",
                  f"kv_chunk_tokens = {self.kv_chunk_tokens}", f"update_cache = {self.update_cache}", "abi_version = 1"]
        return "\n".join(lines) + "\n"

    def source_sha256(self) -> str:
        return text_sha256(self.render_executable_source())

    def preflight(self, *inputs) -> None:
        self._validate_signature(inputs)
        preflight_decode_metadata(inputs, self.input_shapes)

    def _validate_signature(self, inputs: tuple) -> None:
        if len(inputs) != len(FUSED_INPUT_NAMES):
            raise ValueError(f"fused RPA takes {len(FUSED_INPUT_NAMES)} inputs, got {len(inputs)}")
        for name, value, shape in zip(FUSED_INPUT_NAMES, inputs, self.input_shapes, strict=True):
            if shape is None:
                if value is not None:
                    raise ValueError(f"{name} must be None for a plan without relative bias")
                continue
            if tuple(value.shape) != tuple(shape):
                raise ValueError(f"{name} has shape {tuple(value.shape)}, plan expects {tuple(shape)}")

    def build(self, device: torch.device | None = None) -> RpaDecodeExecutable:
        device = device or torch.device("cuda", torch.cuda.current_device())
        tokens, q_heads, dim = self.query_shape
        pages, page_size, _, _, dim_padded = self.fused_cache_shape
        with_bias = self.relative_states_shape is not None
        desc = _native.RpaDesc(
            num_seqs=tokens, num_q_tokens=tokens, q_heads=q_heads, kv_heads=self.key_shape[1], head_dim=dim,
            head_dim_padded=dim_padded, page_size=page_size, cache_layout=_native.CAKE_RPA_CACHE_FUSED,
            table_layout=_native.CAKE_RPA_TABLE_FLAT, max_pages_per_seq=self.page_indices_shape[0], total_pages=pages,
            sm_scale=self.softmax_scale, bias_mode=2 if with_bias else 0,
            bias_extent=self.relative_projection_shape[1] if with_bias else 0,
            rel_dim=self.relative_states_shape[2] if with_bias else 0, update_cache=1 if self.update_cache else 0,
            kv_chunk_tokens=self.kv_chunk_tokens, wait_budget_ms=self.wait_budget_ms,
        )
        return RpaDecodeExecutable(desc, device)

    def invoke(self, executable: RpaDecodeExecutable, *inputs) -> tuple[torch.Tensor, torch.Tensor]:
        """Runs the decode on device tensors. Returns (output, updated cache); the cache tensor is
        updated in place and returned (the reference aliases it, tpu_schedule.py:2336-2339); the
        output is a new tensor."""
        self._validate_signature(inputs)
        q, k, v, cache, lens, pages, _cu_q, cu_kv, _dist, states, projection = inputs
        device = executable.device
        bf16, i32 = torch.bfloat16, torch.int32
        _require(q, self.query_shape, bf16, "queries", device)
        _require(k, self.key_shape, bf16, "keys", device)
        _require(v, self.value_shape, bf16, "values", device)
        _require(cache, self.fused_cache_shape, bf16, "fused_cache", device)
        _require(lens, self.kv_lengths_shape, i32, "kv_lengths", device)
        _require(pages, self.page_indices_shape, i32, "page_indices", device)
        _require(cu_kv, self.cumulative_kv_lengths_shape, i32, "cumulative_kv_lengths", device)
        if states is not None:
            _require(states, self.relative_states_shape, bf16, "relative_states", device)
            _require(projection, self.relative_projection_shape, bf16, "relative_projection", device)
        out = torch.empty(self.output_shape, dtype=bf16, device=device)
        executable.enqueue(q, k if self.update_cache else None, v if self.update_cache else None, cache, None,
                           lens, pages, cu_kv, states, projection, out)
        return out, cache

    def run_preflighted(self, executable: RpaDecodeExecutable, *inputs) -> tuple[torch.Tensor, torch.Tensor]:
        self.preflight(*inputs)
        return self.invoke(executable, *inputs)


@dataclass(frozen=True)
class CudaMixedRpaPlan:
    """Ragged batch on the fused cache: ``sequences`` sequences own ``tokens`` query tokens
    (decode sequences first). Same 11-input signature as ``CudaFusedRpaPlan`` without relative bias."""

    name: str
    schedule_sha256: str
    query_shape: tuple[int, ...]          # (tokens, q_heads, 128)
    key_shape: tuple[int, ...]            # (tokens, kv_heads, 128)
    fused_cache_shape: tuple[int, ...]
    sequences: int
    page_indices_shape: tuple[int, ...]
    softmax_scale: float
    causal: int = 1
    kv_chunk_tokens: int = 0
    wait_budget_ms: int = 0  # bound on the all-gather flag barrier (0 = 20 s)
    update_cache: bool = True

    def __post_init__(self) -> None:
        tokens, q_heads, dim = self.query_shape
        pages, page_size, combined, pack, dim_padded = self.fused_cache_shape
        if pack != 2 or combined * pack != 2 * self.key_shape[1]:
            raise ValueError("fused cache must interleave K and V of every KV head with pack = 2")
        if self.key_shape[0] != tokens or self.key_shape[2] != dim or dim != 128 or dim_padded != 128:
            raise UnsupportedRaggedBatch("ragged batches are lowered for head_dim 128")
        if self.causal != 1:
            raise ValueError("ragged batches are causal")
        if not 0 < self.sequences <= tokens:
            raise ValueError("every sequence owns at least one query token")

    @property
    def input_shapes(self) -> tuple[tuple[int, ...] | None, ...]:
        return (self.query_shape, self.key_shape, self.key_shape, self.fused_cache_shape, (self.sequences,),
                self.page_indices_shape, (self.sequences + 1,), (self.sequences + 1,), (3,), None, None)

    def render_executable_source(self) -> str:
        lines = ["# cake-b200 lowered fused ragged paged attention (mixed prefill / decode)", f"name = {self.name!r}",
                 f"schedule_sha256 = {self.schedule_sha256!r}",
                 "kernels = ('cake_rpa_ragged_update_sm100', 'cake_rpa_prefill_plan_sm100', 'cake_rpa_plan_sm100', "
                 "'cake_rpa_decode_sm100', 'cake_rpa_combine_sm100', 'cake_rpa_prefill_sm100')"]
        for name, shape in zip(FUSED_INPUT_NAMES, self.input_shapes, strict=True):
            lines.append(f"{name}_shape = {shape}")
        lines += [f"softmax_scale = {self.softmax_scale!r}", f"causal = {self.causal}",
                  f"kv_chunk_tokens = {self.kv_chunk_tokens}", f"update_cache = {self.update_cache}", "abi_version = 1"]
        return "\n".join(lines) + "\n"

    def source_sha256(self) -> str:
        return text_sha256(self.render_executable_source())

    def preflight(self, *inputs) -> int:
        return preflight_mixed_metadata(inputs, self.input_shapes)

    def build(self, device: torch.device | None = None) -> RpaDecodeExecutable:
        device = device or torch.device("cuda", torch.cuda.current_device())
        tokens, q_heads, dim = self.query_shape
        pages, page_size, _, _, dim_padded = self.fused_cache_shape
        desc = _native.RpaDesc(
            num_seqs=self.sequences, num_q_tokens=tokens, q_heads=q_heads, kv_heads=self.key_shape[1], head_dim=dim,
            head_dim_padded=dim_padded, page_size=page_size, cache_layout=_native.CAKE_RPA_CACHE_FUSED,
            table_layout=_native.CAKE_RPA_TABLE_FLAT, max_pages_per_seq=self.page_indices_shape[0], total_pages=pages,
            sm_scale=self.softmax_scale, bias_mode=0, bias_extent=0, rel_dim=0, update_cache=1 if self.update_cache else 0,
            kv_chunk_tokens=self.kv_chunk_tokens, wait_budget_ms=self.wait_budget_ms,
        )
        return RpaDecodeExecutable(desc, device)

    def invoke(self, executable: RpaDecodeExecutable, *inputs, out: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Runs the batch on device tensors; ``distribution`` (input 8) is read on the host. Returns
        (output, cache); the cache is updated in place."""
        if len(inputs) != len(FUSED_INPUT_NAMES):
            raise ValueError(f"fused RPA takes {len(FUSED_INPUT_NAMES)} inputs, got {len(inputs)}")
        q, k, v, cache, lens, pages, cu_q, cu_kv, distribution, states, projection = inputs
        if states is not None or projection is not None:
            raise UnsupportedRaggedBatch("relative bias is lowered for decode batches only")
        device = executable.device
        bf16, i32 = torch.bfloat16, torch.int32
        _require(q, self.query_shape, bf16, "queries", device)
        _require(cache, self.fused_cache_shape, bf16, "fused_cache", device)
        _require(lens, (self.sequences,), i32, "kv_lengths", device)
        _require(pages, self.page_indices_shape, i32, "page_indices", device)
        _require(cu_q, (self.sequences + 1,), i32, "cumulative_query_lengths", device)
        _require(cu_kv, (self.sequences + 1,), i32, "cumulative_kv_lengths", device)
        if self.update_cache:
            _require(k, self.key_shape, bf16, "keys", device)
            _require(v, self.key_shape, bf16, "values", device)
        decode_end = int(np.asarray(_to_host(distribution)).reshape(-1)[0])
        if out is None:
            out = torch.empty(self.query_shape, dtype=bf16, device=device)
        executable.enqueue_mixed(q, k if self.update_cache else None, v if self.update_cache else None, cache, None,
                                 lens, pages, cu_kv, cu_q, decode_end, out)
        return out, cache

SHARDED_INPUT_PARTITION_SPECS = (
    ("data", "tensor", ""),          # queries  [tokens, q_heads, dim]
    ("data", "tensor", ""),          # keys     [tokens, kv_heads, dim]
    ("data", "tensor", ""),          # values
    ("data", "", "tensor", "", ""),  # fused cache [pages, page, packed heads, 2, dim_padded]
    ("data",),                       # kv_lengths
    ("data",),                       # page_indices
    ("data",),                       # cumulative_query_lengths
    ("data",),                       # cumulative_kv_lengths
    ("data",),                       # distribution
    ("data", "tensor", ""),          # relative_states
    ("", ""),                        # relative_projection (replicated)
)


@dataclass(frozen=True)
class ShardedCudaFusedRpaPlan:
    """The data x tensor surface of the fused decode: the ``data`` axis splits the batch (sequences,
    their pages, their metadata), the ``tensor`` axis splits heads; every mesh position runs the
    same local plan on its shard and the outputs keep the query and cache sharding. Mirrors
    ``ShardedFusedRpaPlan`` (src/tpu_cake/rpa_lowering.py:395-571; partition specs :1124-1136).
    One process per GPU: rank r sits at (r // tensor, r % tensor). No data-path collective."""

    local_plan: "CudaFusedRpaPlan"
    mesh_axes: tuple[str, str] = ("data", "tensor")
    mesh_shape: tuple[int, int] = (2, 4)
    input_partition_specs: tuple[tuple[str, ...], ...] = SHARDED_INPUT_PARTITION_SPECS
    execution_scope: str = "one-process-per-gpu-data-tensor-shards"

    def __post_init__(self) -> None:
        if self.mesh_axes != ("data", "tensor") or min(self.mesh_shape) < 1:
            raise ValueError("sharded RPA runs on a data x tensor mesh")
        shapes = self.local_plan.input_shapes
        if len(self.input_partition_specs) != len(shapes):
            raise ValueError("sharded RPA needs one partition spec per input")
        for shape, spec in zip(shapes, self.input_partition_specs, strict=True):
            if shape is not None and len(shape) != len(spec):
                raise ValueError("sharded RPA partition specs must match input ranks")
            if any(axis and axis not in self.mesh_axes for axis in spec):
                raise ValueError("sharded RPA partition specs use an unknown mesh axis")

    @property
    def output_partition_specs(self) -> tuple[tuple[str, ...], tuple[str, ...]]:
        return (self.input_partition_specs[0], self.input_partition_specs[3])

    @property
    def schedule_sha256(self) -> str:
        return self.local_plan.schedule_sha256

    @property
    def global_input_shapes(self) -> tuple[tuple[int, ...] | None, ...]:
        sizes = dict(zip(self.mesh_axes, self.mesh_shape, strict=True))
        return tuple(
            None if shape is None else tuple(extent * sizes.get(axis, 1) for extent, axis in zip(shape, spec, strict=True))
            for shape, spec in zip(self.local_plan.input_shapes, self.input_partition_specs, strict=True)
        )

    def mesh_position(self, rank: int) -> tuple[int, int]:
        data, tensor = self.mesh_shape
        if not 0 <= rank < data * tensor:
            raise ValueError(f"rank {rank} outside the {data}x{tensor} mesh")
        return rank // tensor, rank % tensor

    def shard_inputs(self, global_inputs: tuple, position: tuple[int, int]) -> tuple:
        """This mesh position's block of every global input (numpy arrays or torch tensors): along
        each partitioned dimension, the block at the position's index on that axis."""
        index = dict(zip(self.mesh_axes, position, strict=True))
        sizes = dict(zip(self.mesh_axes, self.mesh_shape, strict=True))
        shards = []
        for value, spec, global_shape in zip(global_inputs, self.input_partition_specs, self.global_input_shapes, strict=True):
            if value is None:
                shards.append(None)
                continue
            if tuple(value.shape) != tuple(global_shape):
                raise ValueError(f"global input has shape {tuple(value.shape)}, the surface expects {tuple(global_shape)}")
            selection = []
            for extent, axis in zip(value.shape, spec, strict=True):
                if axis:
                    step = extent // sizes[axis]
                    selection.append(slice(index[axis] * step, (index[axis] + 1) * step))
                else:
                    selection.append(slice(None))
            shards.append(value[tuple(selection)])
        return tuple(shards)

    def assemble(self, per_position: dict[tuple[int, int], object], which: int):
        """Global output (which = 0) or global cache (which = 1) from the per-position numpy results."""
        spec = self.output_partition_specs[which]
        data, tensor = self.mesh_shape
        tensor_dim = spec.index("tensor")
        rows = [np.concatenate([per_position[(d, t)] for t in range(tensor)], axis=tensor_dim) for d in range(data)]
        return np.concatenate(rows, axis=spec.index("data"))

    def build(self, device: torch.device | None = None) -> "RpaDecodeExecutable":
        return self.local_plan.build(device)

    # The reference's names for the two steps (src/tpu_cake/rpa_lowering.py:395-571).
    def place_inputs(self, global_inputs: tuple, rank: int, device: torch.device | None = None) -> tuple:
        """This rank's shard of every global input as device tensors (the shard_map placement)."""
        device = device or torch.device("cuda", torch.cuda.current_device())
        shards = self.shard_inputs(global_inputs, self.mesh_position(rank))
        return tuple(None if value is None else _to_device_tensor(np.ascontiguousarray(_to_host(value)), device) for value in shards)

    def build_executable(self, device: torch.device | None = None) -> "RpaDecodeExecutable":
        return self.build(device)

    def run_local(self, executable: "RpaDecodeExecutable", *local_inputs):
        """Preflight (host integers) and decode of one mesh position's shard."""
        return self.local_plan.run_preflighted(executable, *local_inputs)

    def timing_rounds(self, executable: "RpaDecodeExecutable", host_inputs: tuple, *, warmup_iterations: int, timing_rounds: int,
                      samples_per_round: int) -> tuple[dict, ...]:
        """The chained-state timing protocol of the reference surface runner
        (src/tpu_cake/rpa_surface_runner.py:490-517): every round starts from freshly placed inputs;
        inside a round each call's output becomes the next call's queries and its updated cache the
        next call's cache; one synchronized wall-clock sample per call."""
        import statistics
        import time

        device = executable.device

        def place():
            return tuple(None if value is None else _to_device_tensor(value, device) for value in host_inputs)

        def chain(inputs, outputs):
            output, cache = outputs
            return (output, *inputs[1:3], cache, *inputs[4:])

        def execute(inputs):
            outputs = self.local_plan.invoke(executable, *inputs)
            torch.cuda.synchronize(device)
            return outputs

        inputs = place()
        self.local_plan.preflight(*host_inputs)
        for _ in range(warmup_iterations):
            inputs = chain(inputs, execute(inputs))
        rounds = []
        for round_index in range(timing_rounds):
            inputs = place()
            torch.cuda.synchronize(device)
            samples = []
            for _ in range(samples_per_round):
                started = time.perf_counter_ns()
                outputs = execute(inputs)
                samples.append(time.perf_counter_ns() - started)
                inputs = chain(inputs, outputs)
            rounds.append({"round_index": round_index, "samples_ns": tuple(samples), "median_ns": float(statistics.median(samples))})
        executable.status()
        return tuple(rounds)



class UnsupportedRaggedBatch(ValueError):
    """A ragged batch the CUDA backend does not lower."""


@dataclass(frozen=True)
class CudaPagedAttentionPlan:
    """Decode over separate K / V caches with a [B, max_pages] page table and an optional dense
    bias [q_heads, extent] indexed by key position."""

    name: str
    schedule_sha256: str
    query_shape: tuple[int, int, int]
    cache_shape: tuple[int, int, int, int]  # [pages, page_size, kv_heads, head_dim], same for K and V
    page_table_shape: tuple[int, int]
    bias_shape: tuple[int, int] | None
    softmax_scale: float
    kv_chunk_tokens: int = 0
    wait_budget_ms: int = 0  # bound on the all-gather flag barrier (0 = 20 s)
    cache_layout: str = "separate"  # or "fused": one [pages, page_size, kv_heads, 2, head_dim] tensor

    def __post_init__(self) -> None:
        batch, q_heads, dim = self.query_shape
        if self.cache_shape[3] != dim or q_heads % self.cache_shape[2]:
            raise ValueError("cache head_dim must equal the query's and q_heads must be a multiple of kv_heads")
        if self.page_table_shape[0] != batch:
            raise ValueError("page table needs one row per sequence")
        if self.bias_shape is not None and (self.bias_shape[0] != q_heads or self.bias_shape[1] < self.page_table_shape[1] * self.cache_shape[1]):
            raise ValueError("bias must cover q_heads x (max_pages * page_size) key positions (tpu_schedule.py:2098-2101)")
        if self.cache_layout not in ("separate", "fused"):
            raise ValueError("cache_layout must be 'separate' or 'fused'")

    def render_executable_source(self) -> str:
        return (
            "# cake-b200 lowered ragged paged attention (decode, 2-D page table)\n"
            f"name = {self.name!r}\nschedule_sha256 = {self.schedule_sha256!r}\nquery_shape = {self.query_shape}\n"
            f"cache_shape = {self.cache_shape}\ncache_layout = {self.cache_layout!r}\npage_table_shape = {self.page_table_shape}\n"
            f"bias_shape = {self.bias_shape}\nsoftmax_scale = {self.softmax_scale!r}\nkv_chunk_tokens = {self.kv_chunk_tokens}\nabi_version = 1\n"
        )

    def source_sha256(self) -> str:
        return text_sha256(self.render_executable_source())

    def build(self, device: torch.device | None = None) -> RpaDecodeExecutable:
        device = device or torch.device("cuda", torch.cuda.current_device())
        batch, q_heads, dim = self.query_shape
        pages, page_size, kv_heads, _ = self.cache_shape
        desc = _native.RpaDesc(
            num_seqs=batch, num_q_tokens=batch, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim, head_dim_padded=dim,
            page_size=page_size,
            cache_layout=_native.CAKE_RPA_CACHE_FUSED if self.cache_layout == "fused" else _native.CAKE_RPA_CACHE_SEPARATE,
            table_layout=_native.CAKE_RPA_TABLE_2D, max_pages_per_seq=self.page_table_shape[1], total_pages=pages,
            sm_scale=self.softmax_scale, bias_mode=1 if self.bias_shape is not None else 0,
            bias_extent=self.bias_shape[1] if self.bias_shape is not None else 0, rel_dim=0, update_cache=0,
            kv_chunk_tokens=self.kv_chunk_tokens, wait_budget_ms=self.wait_budget_ms,
        )
        return RpaDecodeExecutable(desc, device)

    def invoke(self, executable: RpaDecodeExecutable, query, key_cache, value_cache, page_table, sequence_lengths, bias=None, out=None):
        device = executable.device
        _require(query, self.query_shape, torch.bfloat16, "query", device)
        if self.cache_layout == "fused":
            pages, page_size, kv_heads, dim = self.cache_shape
            _require(key_cache, (pages, page_size, kv_heads, 2, dim), torch.bfloat16, "fused cache", device)
            if value_cache is not None:
                raise ValueError("value_cache must be None for the fused cache layout")
        else:
            _require(key_cache, self.cache_shape, torch.bfloat16, "key_cache", device)
            _require(value_cache, self.cache_shape, torch.bfloat16, "value_cache", device)
        _require(page_table, self.page_table_shape, torch.int32, "page_table", device)
        _require(sequence_lengths, (self.query_shape[0],), torch.int32, "sequence_lengths", device)
        if self.bias_shape is not None:
            _require(bias, self.bias_shape, torch.float32, "bias", device)
        elif bias is not None:
            raise ValueError("plan was lowered without a bias")
        if out is None:
            out = torch.empty(self.query_shape, dtype=torch.bfloat16, device=device)
        executable.enqueue(query, None, None, key_cache, value_cache, sequence_lengths, page_table, None, bias, None, out)
        return out
