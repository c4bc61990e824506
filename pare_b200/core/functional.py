"""Affine quantize / dequantize on float tensors (host side).

``dequantize_tensor`` is the formula every W4A16 result in this package is checked
against: ``(q - zero) * scale`` evaluated in fp32 with the per-group reshape of the
reference's ``pare/core/functional.py:78-91,193-214``.  Granularity is inferred from
the rank of ``scale``: 0-d per_tensor, ``[out, 1]`` per_channel, ``[out, K/G, 1]``
per_group.  NF4 / FP8 helpers of the reference are outside the INT4 path and are
not provided.
"""

from __future__ import annotations

import torch
from torch import Tensor

from pare_b200.core.dtype import QuantDtype


def _grouped_view(x: Tensor, scale: Tensor) -> Tensor:
    """View ``x [out, K]`` as ``[out, K/G, G]`` when ``scale`` is per-group (rank 3)."""
    if scale.dim() == 3:
        rows, groups, _ = scale.shape
        return x.reshape(rows, groups, x.shape[-1] // groups)
    return x


def quantize_tensor(x: Tensor, scale: Tensor, zero: Tensor, dtype: QuantDtype) -> Tensor:
    """``clamp(round(x / scale + zero), qmin, qmax)`` as int32 (grouped shape for per_group)."""
    if dtype.is_float:
        raise ValueError(f"quantize_tensor is for integer dtypes; got {dtype}.")
    xg = _grouped_view(x, scale)
    return torch.round(xg / scale + zero).clamp(dtype.qmin, dtype.qmax).to(torch.int32)


def dequantize_tensor(q: Tensor, scale: Tensor, zero: Tensor) -> Tensor:
    """``(q - zero) * scale`` in fp32 (grouped shape for per_group)."""
    return (_grouped_view(q.float(), scale) - zero) * scale


def quantization_error(x: Tensor, x_hat: Tensor) -> dict[str, Tensor]:
    """MAE / RMSE / max error / SNR between a tensor and its reconstruction."""
    e = x - x_hat
    mse = e.pow(2).mean()
    return {
        "mae": e.abs().mean(),
        "rmse": mse.sqrt(),
        "max_err": e.abs().max(),
        "snr_db": 10 * torch.log10(x.pow(2).mean() / mse.clamp(1e-12)),
    }
