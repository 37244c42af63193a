"""Shared helpers of the parity tests."""

from __future__ import annotations

import ml_dtypes
import numpy as np
import torch

BF16 = np.dtype(ml_dtypes.bfloat16)


def bf16_to_torch(array: np.ndarray, device) -> torch.Tensor:
    """numpy bfloat16 (ml_dtypes) -> torch.bfloat16 on ``device`` without changing a bit."""
    bits = np.ascontiguousarray(array.astype(BF16)).view(np.uint16)
    return torch.from_numpy(bits.copy()).view(torch.bfloat16).to(device)


def bits_to_bf16(bits: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(bits.astype(np.uint16)).view(BF16)


def torch_to_bf16(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().contiguous().cpu().view(torch.uint16).numpy().view(BF16)


def to_device(array: np.ndarray, device) -> torch.Tensor:
    if array.dtype == BF16:
        return bf16_to_torch(array, device)
    return torch.from_numpy(np.ascontiguousarray(array)).to(device)
