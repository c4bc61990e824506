"""Nibble packing of INT4 codes — the storage layout every kernel here reads.

Layout contract (same as the reference, ``pare/core/pack.py:29-67``): packing is
along the last axis, byte ``j`` holds element ``2j`` in bits 0..3 and element
``2j+1`` in bits 4..7.  Read as little-endian 32-bit words, word ``w`` therefore
holds columns ``8w .. 8w+7`` with column ``8w+i`` at bits ``4i .. 4i+3``; the
CUDA kernels rely on exactly this.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor


def pack_int4(q: Tensor) -> Tensor:
    """Pack unsigned 4-bit codes ``(..., K)`` into uint8 ``(..., K // 2)``."""
    k = q.shape[-1]
    if k % 2:
        raise ValueError(f"Last dimension must be even for INT4 packing, got {k}")
    pairs = (q.to(torch.int32) & 0xF).reshape(*q.shape[:-1], k // 2, 2)
    return (pairs[..., 0] | (pairs[..., 1] << 4)).to(torch.uint8)


def unpack_int4(packed: Tensor) -> Tensor:
    """Inverse of :func:`pack_int4`: uint8 ``(..., K // 2)`` → int32 ``(..., K)``."""
    b = packed.to(torch.int32)
    out = torch.empty(*b.shape[:-1], b.shape[-1] * 2, dtype=torch.int32, device=b.device)
    out[..., 0::2] = b & 0xF
    out[..., 1::2] = (b >> 4) & 0xF
    return out


def pack_int4_signed(q: Tensor) -> Tensor:
    """Pack signed 4-bit values (-8..7) by biasing them into 0..15 first."""
    return pack_int4(q + 8)


def unpack_int4_signed(packed: Tensor) -> Tensor:
    """Inverse of :func:`pack_int4_signed`."""
    return unpack_int4(packed) - 8


def repack_int4_for_kernel(packed: Tensor, group_size: int = 128) -> Tensor:
    """Re-layout used by the reference's Triton kernel (``pare/core/pack.py:88-132``).

    Inside every ``group_size``-wide column tile, byte ``j`` of the result pairs
    column ``j`` (low nibble) with column ``j + group_size/2`` (high nibble).  The
    CUDA kernels in this package read the storage layout directly and never need
    this; it is kept because callers of ``matmul_w4a16`` written for the reference
    pass weights in this layout.  Vectorised (no per-tile Python loop).
    """
    n, k_half = packed.shape
    k = 2 * k_half
    assert k % group_size == 0, f"K={k} must be divisible by group_size={group_size}"
    half = group_size // 2
    q = unpack_int4(packed).reshape(n, k // group_size, 2, half)
    return (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).to(torch.uint8).reshape(n, k_half)


def unrepack_int4_from_kernel(kernel_layout: Tensor, group_size: int = 128) -> Tensor:
    """Inverse of :func:`repack_int4_for_kernel` (kernel layout → storage layout)."""
    n, k_half = kernel_layout.shape
    k = 2 * k_half
    assert k % group_size == 0
    half = group_size // 2
    b = kernel_layout.to(torch.int32).reshape(n, k // group_size, half)
    q = torch.stack([b & 0xF, (b >> 4) & 0xF], dim=2).reshape(n, k)
    return pack_int4(q)


def packed_size_bytes(shape: tuple[int, ...], bits: int) -> int:
    """Bytes needed to store ``prod(shape)`` codes of ``bits`` bits each."""
    return (math.prod(shape) * bits + 7) // 8
