"""Oracle for the K-sharded BF16 matmul followed by a reduce-scatter (numpy, float32).

Follows the reference:
  - inputs are float32 normals rounded to bfloat16 (src/tpu_cake/runner.py:447-456);
  - the correctness oracle is ``bf16(lhs).astype(f32) @ bf16(rhs).astype(f32)`` compared with
    ``allclose(atol=1e-3, rtol=1e-3)`` (src/tpu_cake/runner.py:490-498);
  - on the device each mesh position contracts its K slice into a float32 partial [M, N] and the
    partials are summed and scattered along ``scatter_dimension``
    (src/tpu_cake/pallas_lowering.py:446-476).
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)


def quantize_bf16(values: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 (round to nearest even) -> float32, as runner.py:447-456 does."""
    return np.asarray(values, dtype=np.float32).astype(BF16).astype(np.float32)


def matmul_reference(lhs_q: np.ndarray, rhs_q: np.ndarray) -> np.ndarray:
    """The single-product oracle of runner.py:490-493 (inputs already bf16-valued float32)."""
    return np.asarray(lhs_q, dtype=np.float32) @ np.asarray(rhs_q, dtype=np.float32)


def local_partials(lhs_q: np.ndarray, rhs_q: np.ndarray, world: int) -> list[np.ndarray]:
    """Per-mesh-position float32 partial products; K is split into ``world`` contiguous blocks
    (lhs columns / rhs rows), pallas_lowering.py:466-472."""
    k = lhs_q.shape[1]
    if k % world:
        raise ValueError(f"K={k} is not divisible by the mesh size {world}")
    step = k // world
    return [
        np.asarray(lhs_q[:, r * step : (r + 1) * step], dtype=np.float32)
        @ np.asarray(rhs_q[r * step : (r + 1) * step, :], dtype=np.float32)
        for r in range(world)
    ]


def reduced_rows(
    lhs_rows_q: np.ndarray,
    rhs_q: np.ndarray,
    *,
    world: int,
    transport_dtype: str = "f32",
    out_dtype: str = "f32",
) -> np.ndarray:
    """Full-width rows of the reduced product for a subset of lhs rows: the ``world`` split-K
    partials of those rows (pallas_lowering.py:446-472), rounded to the transport dtype if it is
    bf16, summed in rank order in float32 and rounded to ``out_dtype``. What a rank's local output
    must hold in the rows it owns; used to check large products on sampled rows."""
    if transport_dtype not in ("f32", "bf16"):
        raise ValueError(f"unknown transport dtype {transport_dtype}")
    partials = local_partials(lhs_rows_q, rhs_q, world)
    if transport_dtype == "bf16" and world > 1:
        partials = [quantize_bf16(p) for p in partials]
    total = np.zeros_like(partials[0])
    for partial in partials:
        total = total + partial
    return quantize_bf16(total) if out_dtype == "bf16" else total


def matmul_reduce_scatter(
    lhs_q: np.ndarray,
    rhs_q: np.ndarray,
    *,
    world: int,
    scatter_dimension: int,
    transport_dtype: str = "f32",
    out_dtype: str = "f32",
) -> list[np.ndarray]:
    """Local outputs of every mesh position, as float32 arrays holding ``out_dtype`` values.

    Partials are optionally rounded to the transport dtype (what crosses the link), summed in rank
    order in float32 -- the order the device reduction uses, so results are reproducible -- and
    sliced along ``scatter_dimension`` (psum_scatter(tiled=True), pallas_lowering.py:459-464).
    """
    if scatter_dimension not in (0, 1):
        raise ValueError("scatter_dimension must be 0 (M) or 1 (N)")
    partials = local_partials(lhs_q, rhs_q, world)
    if transport_dtype == "bf16" and world > 1:
        partials = [quantize_bf16(p) for p in partials]
    elif transport_dtype != "f32" and transport_dtype != "bf16":
        raise ValueError(f"unknown transport dtype {transport_dtype}")
    total = np.zeros_like(partials[0])
    for partial in partials:
        total = total + partial
    extent = total.shape[scatter_dimension]
    if extent % world:
        raise ValueError("scatter dimension is not divisible by the mesh size")
    step = extent // world
    outputs = []
    for r in range(world):
        piece = total[r * step : (r + 1) * step, :] if scatter_dimension == 0 else total[:, r * step : (r + 1) * step]
        piece = np.ascontiguousarray(piece)
        outputs.append(quantize_bf16(piece) if out_dtype == "bf16" else piece)
    return outputs


def max_abs_error(actual: np.ndarray, expected: np.ndarray) -> float:
    return float(np.max(np.abs(np.asarray(actual, dtype=np.float64) - np.asarray(expected, dtype=np.float64))))


def relative_l2_error(actual: np.ndarray, expected: np.ndarray) -> float:
    """sqrt(sum d^2 / sum e^2) in float64 (src/tpu_cake/rpa_surface_runner.py:394-411)."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    denominator = float(np.sum(e * e))
    numerator = float(np.sum((a - e) ** 2))
    if denominator == 0.0:
        return 0.0 if numerator == 0.0 else float("inf")
    return float(np.sqrt(numerator / denominator))
