"""Scale / zero-point selection for uniform integer grids (host side, offline).

Same contract as the reference's ``pare/core/scale.py:24-137``: asymmetric grids
stretch over ``[min(x, 0), max(x, 0)]`` with an integer-valued float zero-point,
symmetric grids use ``absmax / max(|qmin|, |qmax|)`` and zero 0.  Result shapes:
0-d (per_tensor), ``[out, 1]`` (per_channel), ``[out, K/G, 1]`` (per_group).
Used here only to build test and benchmark layers (round-to-nearest).
"""

from __future__ import annotations

import torch
from torch import Tensor

from pare_b200.core.dtype import QuantDtype

_EPS = 1e-8


def _grid_from_range(lo: Tensor, hi: Tensor, qmin: float, qmax: float, sym: bool) -> tuple[Tensor, Tensor]:
    if sym:
        span = torch.maximum(lo.abs(), hi.abs()).clamp(min=_EPS)
        scale = span / max(abs(qmin), abs(qmax))
        return scale, torch.zeros_like(scale)
    lo = lo.clamp(max=0.0)
    hi = hi.clamp(min=0.0)
    scale = ((hi - lo) / (qmax - qmin)).clamp(min=_EPS)
    zero = torch.round(-lo / scale + qmin).clamp(qmin, qmax)
    return scale, zero


def compute_scale(
    x: Tensor,
    dtype: QuantDtype,
    *,
    granularity: str = "per_group",
    group_size: int = 128,
    sym: bool = False,
) -> tuple[Tensor, Tensor]:
    """Return ``(scale, zero)`` broadcastable against ``x`` for the given granularity."""
    if dtype.is_float:
        raise ValueError(f"compute_scale is for integer dtypes; got {dtype}")
    qmin, qmax = float(dtype.qmin), float(dtype.qmax)

    if granularity == "per_tensor":
        s, z = _grid_from_range(x.min().reshape(1), x.max().reshape(1), qmin, qmax, sym)
        return s.squeeze(), z.squeeze()
    if granularity == "per_channel":
        dims = list(range(1, x.dim()))
        return _grid_from_range(x.amin(dim=dims, keepdim=True), x.amax(dim=dims, keepdim=True), qmin, qmax, sym)
    if granularity == "per_group":
        if x.dim() != 2:
            raise ValueError(f"per_group expects a 2-D weight matrix, got shape {tuple(x.shape)}")
        rows, cols = x.shape
        if cols % group_size:
            raise ValueError(f"in_features={cols} is not divisible by group_size={group_size}")
        xg = x.reshape(rows, cols // group_size, group_size)
        return _grid_from_range(xg.amin(dim=-1, keepdim=True), xg.amax(dim=-1, keepdim=True), qmin, qmax, sym)
    raise ValueError(f"Unknown granularity: {granularity!r}")
