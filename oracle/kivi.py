"""numpy restatement of the reference's KIVI cache (test infrastructure).

Restates pare/kv_cache.py in IEEE fp32:
  * ``quantize_keys``    :75-104   per (batch, head, G-token group, channel) min/max
  * ``quantize_values``  :122-151  per (batch, head, token) min/max over the whole head_dim
  * ``dequantize_*``     :107-119, 154-156   ``code * scale + zero``
  * ``Cache.update``     :205-252, 294-325   residual window + whole-group compression
Order of operations matters for bit-exact codes: ``(max - min) / qmax`` (true division),
``max(., 1e-8)``, ``(x - min) / scale`` (true division), clamp to ``[0, qmax]``, then
round-half-to-even.
"""

from __future__ import annotations

import numpy as np

_F = np.float32


def _affine_codes(x: np.ndarray, lo: np.ndarray, hi: np.ndarray, bits: int):
    qmax = _F((1 << bits) - 1)
    scale = np.maximum((hi - lo) / qmax, _F(1e-8)).astype(_F)
    q = np.rint(np.clip((x - lo) / scale, _F(0), qmax)).astype(np.uint8)
    return q, scale


def quantize_keys(k: np.ndarray, bits: int, group_size: int):
    """``k [B,H,n,D]`` fp32, n % G == 0 → codes uint8 ``[B,H,n,D]``, scale/zero fp32 ``[B,H,n/G,D]``."""
    k = np.asarray(k, dtype=_F)
    b, h, n, d = k.shape
    kg = k.reshape(b, h, n // group_size, group_size, d)
    lo = kg.min(axis=3, keepdims=True)
    hi = kg.max(axis=3, keepdims=True)
    q, scale = _affine_codes(kg, lo, hi, bits)
    return q.reshape(b, h, n, d), scale[:, :, :, 0, :], lo[:, :, :, 0, :]


def quantize_values(v: np.ndarray, bits: int, group_size: int, v_group: int | None = None):
    """``v [B,H,n,D]`` fp32 → codes ``[B,H,n,D]``, scale/zero ``[B,H,n,1]`` (one pair per token).

    ``v_group`` (not in the reference; the finer grouping of the KIVI paper): the same function with the channel
    axis viewed as ``[D/v_group, v_group]`` -- one pair per token and group of ``v_group`` channels, scale/zero
    ``[B,H,n,D/v_group]``."""
    v = np.asarray(v, dtype=_F)
    if v_group is not None and v_group != v.shape[3]:
        b, h, n, d = v.shape
        vg = v.reshape(b, h, n, d // v_group, v_group)
        lo = vg.min(axis=4, keepdims=True)
        hi = vg.max(axis=4, keepdims=True)
        q, scale = _affine_codes(vg, lo, hi, bits)
        return q.reshape(b, h, n, d), scale[..., 0], lo[..., 0]
    lo = v.min(axis=3, keepdims=True)
    hi = v.max(axis=3, keepdims=True)
    q, scale = _affine_codes(v, lo, hi, bits)
    return q, scale, lo


def dequantize_keys(q: np.ndarray, scale: np.ndarray, zero: np.ndarray, group_size: int) -> np.ndarray:
    b, h, n, d = q.shape
    qg = q.astype(_F).reshape(b, h, n // group_size, group_size, d)
    return (qg * scale[:, :, :, None, :] + zero[:, :, :, None, :]).reshape(b, h, n, d).astype(_F)


def dequantize_values(q: np.ndarray, scale: np.ndarray, zero: np.ndarray) -> np.ndarray:
    if scale.shape[3] > 1:   # [B,H,n,D/v_group]: one pair per group of channels
        b, h, n, d = q.shape
        qg = q.astype(_F).reshape(b, h, n, scale.shape[3], -1)
        return (qg * scale[..., None] + zero[..., None]).reshape(b, h, n, d).astype(_F)
    return (q.astype(_F) * scale + zero).astype(_F)


class Cache:
    """One layer of the reference cache state machine, fp32 in / fp32 out.

    ``update`` appends tokens, compresses the oldest whole groups that overflow the residual
    window and returns the dense ``(K, V)`` the reference would hand to attention (before its
    final cast to the input dtype).
    """

    def __init__(self, bits: int = 4, group_size: int = 32, residual_length: int = 128, v_group: int | None = None):
        self.bits, self.G, self.R, self.v_group = bits, group_size, residual_length, v_group
        self.comp = None   # (kq, ks, kz, vq, vs, vz)
        self.rk = None
        self.rv = None

    def update(self, new_k: np.ndarray, new_v: np.ndarray):
        nk, nv = np.asarray(new_k, dtype=_F), np.asarray(new_v, dtype=_F)
        rk = nk if self.rk is None else np.concatenate([self.rk, nk], axis=2)
        rv = nv if self.rv is None else np.concatenate([self.rv, nv], axis=2)
        groups = max(0, rk.shape[2] - self.R) // self.G
        if groups > 0:
            n = groups * self.G
            new = quantize_keys(rk[:, :, :n], self.bits, self.G) + quantize_values(rv[:, :, :n], self.bits, self.G, self.v_group)
            self.comp = new if self.comp is None else tuple(
                np.concatenate([a, b], axis=2) for a, b in zip(self.comp, new))
            rk, rv = rk[:, :, n:], rv[:, :, n:]
        self.rk, self.rv = rk, rv
        if self.comp is None:
            return rk, rv
        kq, ks, kz, vq, vs, vz = self.comp
        full_k = np.concatenate([dequantize_keys(kq, ks, kz, self.G), rk], axis=2)
        full_v = np.concatenate([dequantize_values(vq, vs, vz), rv], axis=2)
        return full_k, full_v

    @property
    def n_comp(self) -> int:
        return 0 if self.comp is None else self.comp[0].shape[2]

    @property
    def n_res(self) -> int:
        return 0 if self.rk is None else self.rk.shape[2]


def decode_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float | None = None) -> np.ndarray:
    """``softmax(q k^T * scale) v`` in fp64-free fp32 with grouped-query head sharing.

    ``q [B,Hq,Tq,D]``, ``k/v [B,Hkv,T,D]``; q head h reads kv head ``h // (Hq/Hkv)`` — the
    ``repeat_interleave`` a caller of the reference applies before
    ``scaled_dot_product_attention`` (pare/kv_cache.py:183-186).
    """
    q = np.asarray(q, dtype=_F)
    k = np.asarray(k, dtype=_F)
    v = np.asarray(v, dtype=_F)
    b, hq, tq, d = q.shape
    rep = hq // k.shape[1]
    k = np.repeat(k, rep, axis=1)
    v = np.repeat(v, rep, axis=1)
    scale = _F(1.0 / np.sqrt(d)) if scale is None else _F(scale)
    s = np.einsum("bhqd,bhtd->bhqt", q, k) * scale
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("bhqt,bhtd->bhqd", p, v).astype(_F)


def rope_rows(positions, head_dim: int, theta: float = 10000.0) -> np.ndarray:
    """``[len(positions), head_dim]`` fp32: ``cos(p f_i)`` for ``i < head_dim/2`` then ``sin(p f_i)``,
    ``f_i = theta^(-2i/head_dim)``; angles in float64, table in float32.  Rotary position embedding as published
    (Su et al., RoFormer) in the half-split pairing Llama-family models use; not part of the reference, whose
    callers hand ``update()`` keys that are already rotated (pare/kv_cache.py:205-231)."""
    half = head_dim // 2
    freq = np.float64(theta) ** (-np.arange(half, dtype=np.float64) / half)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(_F)


def apply_rope(x: np.ndarray, rows: np.ndarray) -> np.ndarray:
    """``x [..., T, D]`` rotated by ``rows [T, D]`` (or ``[D]``): ``x'[i] = x[i] cos_i - x[i+D/2] sin_i``,
    ``x'[i+D/2] = x[i+D/2] cos_i + x[i] sin_i`` in fp32, products and sums rounded separately.  The kernel rounds
    this to the activation dtype before it uses or stores the value; so does the caller of this function."""
    x = np.asarray(x, dtype=_F)
    half = x.shape[-1] // 2
    cos, sin = rows[..., :half].astype(_F), rows[..., half:].astype(_F)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1).astype(_F)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float | None = None, causal: bool = True) -> np.ndarray:
    """``softmax(q k^T * scale) v`` in fp32 for ``q [B,Hq,Tq,D]`` over ``k/v [B,Hkv,Tk,D]``, ``Tk >= Tq``: the queries are
    the last ``Tq`` tokens, query i sees keys ``j <= i + (Tk - Tq)`` -- what ``scaled_dot_product_attention(...,
    is_causal=True)`` gives a caller of the reference for a prompt (pare/kv_cache.py:183-186), with the grouped-query
    ``repeat_interleave`` folded in."""
    q = np.asarray(q, dtype=_F)
    k = np.asarray(k, dtype=_F)
    v = np.asarray(v, dtype=_F)
    b, hq, tq, d = q.shape
    tk = k.shape[2]
    rep = hq // k.shape[1]
    scale = _F(1.0 / np.sqrt(d)) if scale is None else _F(scale)
    out = np.empty_like(q)
    visible = (np.arange(tk)[None, :] <= np.arange(tq)[:, None] + (tk - tq)) if causal else np.ones((tq, tk), dtype=bool)
    for h in range(hq):
        s = np.einsum("bqd,btd->bqt", q[:, h], k[:, h // rep]) * scale
        s = np.where(visible[None], s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h] = np.einsum("bqt,btd->bqd", p, v[:, h // rep])
    return out.astype(_F)
