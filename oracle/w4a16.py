"""numpy restatement of the reference's dequantize-then-matmul path (test infrastructure).

Restates, in fp32:
  * ``unpack_int4``            pare/core/pack.py:51-67   (low nibble = even column)
  * ``dequantize_tensor``      pare/core/functional.py:78-91, 193-214   ``(q - zero) * scale``
  * ``QuantizedLinear.forward`` default branch, pare/layers/linear.py:101-118, 129, 138
Extensions with no reference code (stated in the docstrings): per-column group index
(``g_idx``) and a run-time input scale.
"""

from __future__ import annotations

import numpy as np


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """uint8 ``[..., K/2]`` → int32 ``[..., K]``; byte j gives columns 2j (bits 0-3), 2j+1 (bits 4-7)."""
    p = packed.astype(np.int32)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.int32)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = (p >> 4) & 0xF
    return out


def pack_int4(q: np.ndarray) -> np.ndarray:
    """Inverse of :func:`unpack_int4` (pare/core/pack.py:29-48)."""
    q = q.astype(np.int32) & 0xF
    return (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)


def dequantize(packed: np.ndarray, scale: np.ndarray, zero: np.ndarray, g_idx: np.ndarray | None = None) -> np.ndarray:
    """fp32 weight ``[N, K]``.

    ``scale`` / ``zero`` are fp32 ``[N, n_groups]`` (the reference's ``[N, n_groups, 1]`` with
    the last axis dropped; ``n_groups == 1`` is per_channel).  Without ``g_idx`` column k
    uses group ``k // (K / n_groups)`` exactly as the reference reshape does.  With
    ``g_idx`` (no reference counterpart) column k uses group ``g_idx[k]``.
    """
    q = unpack_int4(packed).astype(np.float32)
    n, k = q.shape
    scale = np.asarray(scale, dtype=np.float32).reshape(n, -1)
    zero = np.asarray(zero, dtype=np.float32).reshape(n, -1)
    if g_idx is None:
        groups = scale.shape[1]
        qg = q.reshape(n, groups, k // groups)
        return ((qg - zero[:, :, None]) * scale[:, :, None]).reshape(n, k)
    idx = np.asarray(g_idx, dtype=np.int64)
    return (q - zero[:, idx]) * scale[:, idx]


def linear(
    x: np.ndarray,
    packed: np.ndarray,
    scale: np.ndarray,
    zero: np.ndarray,
    bias: np.ndarray | None = None,
    g_idx: np.ndarray | None = None,
    input_scale: np.ndarray | None = None,
    round_input=None,
) -> np.ndarray:
    """``x @ dequantize(...).T (+ bias)`` in fp32 (float64 accumulation is NOT used on purpose:
    the reference's CPU path is an fp32 GEMM).

    ``input_scale`` (no reference counterpart at run time; AWQ folds it offline,
    pare/schemes/awq.py:388-424): x is divided by it in fp32 and, when ``round_input`` is
    given, rounded to the activation dtype by that callable before the product.
    """
    x = np.asarray(x, dtype=np.float32)
    if input_scale is not None:
        x = x / np.asarray(input_scale, dtype=np.float32)
        if round_input is not None:
            x = round_input(x)
    w = dequantize(packed, scale, zero, g_idx)
    y = x @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return y.astype(np.float32)


def rel_err(y: np.ndarray, ref: np.ndarray, floor: float = 1e-2) -> tuple[float, float]:
    """(max, mean) of ``|y - ref| / max(|ref|, floor * max|ref|)`` — the tolerance metric of the tests."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.maximum(np.abs(ref), floor * np.abs(ref).max() + 1e-30)
    e = np.abs(y - ref) / denom
    return float(e.max()), float(e.mean())
