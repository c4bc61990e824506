"""AutoAWQ "GEMM" tensor layout <-> the packed layout of :class:`QuantizedLinear`.

The AutoAWQ GEMM format stores a 4-bit layer transposed and packed along the *output* dimension:
``qweight`` int32 ``[K, N/8]``, ``qzeros`` int32 ``[K/G, N/8]``, ``scales`` fp16 ``[K/G, N]``; nibble ``i`` of an
int32 holds output column ``8 w + ORDER[i]`` with ``ORDER = (0, 2, 4, 6, 1, 3, 5, 7)``.  The affine convention is
the same as here (``w = (q - z) * s`` with an integer zero point), so the conversion is a lossless re-layout
(scales go through fp16 on export, as the format demands).  Counterpart of the reference's exporter
(``pare/model/export_awq.py:39-94``); the import direction lets checkpoints quantized by other tools run on
the kernels of this package.
"""

from __future__ import annotations

import torch
from torch import Tensor

from pare_b200.config import QuantConfig
from pare_b200.core.pack import pack_int4, unpack_int4
from pare_b200.layers.linear import QuantizedLinear

ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _pack_columns(codes: Tensor) -> Tensor:
    """``[..., N]`` integer codes 0..15 -> ``[..., N/8]`` int32 in the interleaved nibble order."""
    if codes.shape[-1] % 8:
        raise ValueError("the packed dimension must be a multiple of 8")
    lanes = codes.to(torch.int64).unflatten(-1, (-1, 8))[..., list(ORDER)]          # nibble i <- column ORDER[i]
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    word = (lanes << shifts).sum(-1)
    return (word - ((word >> 31) << 32)).to(torch.int32)                             # two's complement wrap


def _unpack_columns(words: Tensor) -> Tensor:
    """Inverse of :func:`_pack_columns`: int32 ``[..., N/8]`` -> uint8 codes ``[..., N]``."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    lanes = (w.unsqueeze(-1) >> shifts) & 0xF                                        # nibble i
    cols = torch.empty_like(lanes)
    cols[..., list(ORDER)] = lanes                                                   # column ORDER[i] <- nibble i
    return cols.flatten(-2).to(torch.uint8)


def to_awq_gemm(layer: QuantizedLinear) -> dict[str, Tensor]:
    """The AutoAWQ GEMM tensors of a 4-bit per-group layer (CPU tensors)."""
    cfg = layer.config
    if layer.packed_weight is None or cfg.granularity != "per_group":
        raise ValueError("only INT4 per-group layers have an AWQ GEMM form")
    if layer.g_idx is not None or layer.input_scale is not None:
        raise ValueError("act-order / run-time input scales have no place in the AWQ GEMM format")
    n, k, g = layer.out_features, layer.in_features, cfg.group_size
    if k % g or n % 8:
        raise ValueError(f"needs in_features ({k}) divisible by the group size ({g}) and out_features ({n}) by 8")
    q = unpack_int4(layer.packed_weight.cpu()).reshape(n, k)
    zero = layer.zero.detach().cpu().reshape(n, k // g)
    if not torch.equal(zero, zero.round()):
        raise ValueError("zero points must be integers")
    out = {
        "qweight": _pack_columns(q.t().contiguous()),
        "qzeros": _pack_columns(zero.t().contiguous()),
        "scales": layer.scale.detach().cpu().reshape(n, k // g).t().contiguous().to(torch.float16),
    }
    if layer.bias is not None:
        out["bias"] = layer.bias.detach().cpu().to(torch.float16)
    return out


def from_awq_gemm(qweight: Tensor, qzeros: Tensor, scales: Tensor, bias: Tensor | None = None, *,
                  group_size: int = 128) -> QuantizedLinear:
    """A :class:`QuantizedLinear` (``use_kernel=False`` until set) from AutoAWQ GEMM tensors."""
    k, n8 = qweight.shape
    n = n8 * 8
    if scales.shape != (k // group_size, n) or qzeros.shape != (k // group_size, n8):
        raise ValueError("qzeros / scales do not match qweight and the group size")
    q = _unpack_columns(qweight.cpu()).t().contiguous()                              # [N, K]
    zero = _unpack_columns(qzeros.cpu()).t().contiguous().float().unsqueeze(-1)       # [N, K/G, 1]
    scale = scales.cpu().float().t().contiguous().unsqueeze(-1)
    cfg = QuantConfig(bits=4, scheme="awq", granularity="per_group", group_size=group_size)
    return QuantizedLinear.from_tensors(pack_int4(q), None, scale, zero, cfg, None if bias is None else bias.cpu(), k, n)
