"""torch-CPU restatement of the reference's run-time path, op for op, for TIMING the CPU baseline
(test infrastructure; the benchmark's ``cpu_baseline`` / ``--impl reference`` legs are its only users).

The reference executes these ATen op sequences on the host (no native code of its own):
  * linear:  unpack nibbles to int32 -> float -> ``(q - zero) * scale`` -> ``F.linear``
             (pare/layers/linear.py:112-118, 129, 138; pare/core/pack.py:51-67;
             pare/core/functional.py:78-91)
  * cache:   concatenate the residual, quantize overflowing groups, concatenate the six
             compressed tensors, dequantize the WHOLE cache, concatenate, cast
             (pare/kv_cache.py:205-252, 294-325), then fp32 scaled-dot-product attention on
             the result (pare/kv_cache.py:183-186)
Numerically they agree with ``oracle/w4a16.py`` / ``oracle/kivi.py``; this file exists because
timing numpy would not represent the multi-threaded ATen kernels the reference really runs.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def linear_forward(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """``x [M,K]`` fp32, ``packed [N,K/2]`` uint8, ``scale/zero [N,K/G,1]`` fp32 → ``[M,N]`` fp32."""
    p = packed.to(torch.int32)
    q = torch.stack([p & 0xF, (p >> 4) & 0xF], dim=-1).reshape(packed.shape[0], -1)
    n, groups, _ = scale.shape
    w = ((q.float().reshape(n, groups, -1) - zero) * scale).reshape(n, -1)
    return F.linear(x, w.to(x.dtype))


class TorchCache:
    """One layer of the reference cache in torch ops (fp32 working precision)."""

    def __init__(self, bits: int = 4, group_size: int = 32, residual_length: int = 128) -> None:
        self.bits, self.G, self.R = bits, group_size, residual_length
        self.comp = None
        self.rk = self.rv = None

    def _quant(self, x: torch.Tensor, dim: int):
        qmax = float((1 << self.bits) - 1)
        lo, hi = x.amin(dim=dim, keepdim=True), x.amax(dim=dim, keepdim=True)
        scale = ((hi - lo) / qmax).clamp(min=1e-8)
        return ((x - lo) / scale).clamp(0, qmax).round().to(torch.uint8), scale, lo

    def update(self, new_k: torch.Tensor, new_v: torch.Tensor):
        dtype = new_k.dtype
        nk, nv = new_k.float(), new_v.float()
        rk = nk if self.rk is None else torch.cat([self.rk, nk], dim=2)
        rv = nv if self.rv is None else torch.cat([self.rv, nv], dim=2)
        groups = max(0, rk.shape[2] - self.R) // self.G
        if groups:
            n = groups * self.G
            b, h, _, d = rk.shape
            kq, ks, kz = self._quant(rk[:, :, :n].reshape(b, h, groups, self.G, d), 3)
            vq, vs, vz = self._quant(rv[:, :, :n], 3)
            new = (kq.reshape(b, h, n, d), ks.squeeze(3), kz.squeeze(3), vq, vs, vz)
            self.comp = new if self.comp is None else tuple(torch.cat([a, c], dim=2) for a, c in zip(self.comp, new))
            rk, rv = rk[:, :, n:], rv[:, :, n:]
        self.rk, self.rv = rk, rv
        if self.comp is None:
            return rk.to(dtype), rv.to(dtype)
        kq, ks, kz, vq, vs, vz = self.comp
        b, h, n, d = kq.shape
        dk = (kq.float().reshape(b, h, n // self.G, self.G, d) * ks.unsqueeze(3) + kz.unsqueeze(3)).reshape(b, h, n, d)
        dv = vq.float() * vs + vz
        return torch.cat([dk, rk], dim=2).to(dtype), torch.cat([dv, rv], dim=2).to(dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """fp32 SDPA with grouped-query head sharing (``q [B,Hq,1,D]``, ``k/v [B,Hkv,T,D]``)."""
    rep = q.shape[1] // k.shape[1]
    return F.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(rep, dim=1),
                                          v.float().repeat_interleave(rep, dim=1))
