"""KIVI quantized KV cache on CUDA — same class API as the reference's ``pare/kv_cache.py``.

Keys are quantized per channel over groups of ``group_size`` tokens, values per token over the
whole head dimension, both unsigned asymmetric min-max; the newest ``residual_length`` tokens
stay in full precision (KIVI, Liu et al., ICML 2024).  What is kept from the reference
(``pare/kv_cache.py:41-55, 163-288``): ``KVCacheConfig``, ``QuantizedKVCache(num_layers, config)``,
``update / reset / seq_len / memory_bytes``, the private ``_compressed`` / ``_residual_k`` /
``_residual_v`` lists callers peek into, and the exact compression schedule: after every
``update`` the oldest whole groups that overflow the residual window are compressed, so group
boundaries sit at absolute token positions and chunked feeding equals one-shot feeding.

What is different underneath:

* storage is preallocated and packed (2/4/8-bit codes, layouts in ``include/pare_b200.h``)
  instead of six ``torch.cat``-grown tensors of one byte per code; appends write in place;
* quantization and reconstruction are CUDA kernels (``pare_kivi_append`` / ``pare_kivi_dequant``)
  whose codes, scales and zeros are bit-identical to the reference's fp32 arithmetic;
* the residual window is kept in the input dtype (lossless for fp16/bf16 inputs) rather than
  upcast to fp32;
* :meth:`QuantizedKVCache.attend` is additive: append + fused dequantize/decode-attention that
  reads the packed cache directly, instead of ``update`` followed by dense attention.

The cache runs on CUDA tensors only; there is no eager implementation behind it.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor

from pare_b200.kernels import _lib

_V_BLOCK = 128  # tokens per block of the value-code layout


@dataclass
class KVCacheConfig:
    """``bits`` per code (2, 4 or 8), tokens per key group, tokens kept in full precision; ``v_group_size``: channels
    that share a value scale / zero -- ``None`` = the whole head_dim (the reference), 32 = the KIVI paper's groups."""

    bits: int = 4
    group_size: int = 32
    residual_length: int = 128
    v_group_size: int | None = None


def rope_table(max_positions: int, head_dim: int, theta: float = 10000.0, device=None) -> Tensor:
    """``[max_positions, head_dim]`` fp32: row p = ``cos(p f_i)`` for ``i < head_dim/2`` followed by ``sin(p f_i)``,
    ``f_i = theta^(-2i/head_dim)`` -- the rotary table in the form :meth:`QuantizedKVCache.attend` and
    :func:`apply_rope` take (angles computed in float64, stored in float32)."""
    half = head_dim // 2
    freq = theta ** (-torch.arange(half, dtype=torch.float64) / half)
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(device)


def apply_rope(x: Tensor, rows: Tensor) -> Tensor:
    """Rotary embedding of ``x [..., T, D]`` with ``rows [T, D]`` (or ``[D]``) of a :func:`rope_table`: pairs
    ``(i, i + D/2)``, products and sum in float32, each rounded separately, result rounded to ``x.dtype`` -- what the
    attention kernel does to ``q`` and the newest key."""
    if (x.is_cuda and x.dim() == 4 and x.dtype in (torch.float16, torch.bfloat16) and x.stride(3) == 1 and rows.dim() == 2
            and rows.shape[0] == x.shape[2] and rows.dtype == torch.float32 and rows.is_contiguous() and rows.device == x.device):
        out = torch.empty(x.shape, device=x.device, dtype=x.dtype)     # one pass instead of a dozen element-wise launches
        B, H, T, D = x.shape
        _lib.check(_lib.lib().pare_rope(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), out.data_ptr(), rows.data_ptr(),
                                        B, H, T, D, _lib.dtype_code(x.dtype), _lib.current_stream(x.device)), "pare_rope")
        return out
    half = x.shape[-1] // 2
    cos, sin = rows[..., :half].float(), rows[..., half:].float()
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


def prefill_attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, causal: bool = True) -> Tensor:
    """``softmax(q k^T * scale) v`` for ``q [B, Hq, Tq, D]`` over full-precision ``k, v [B, H, Tk, D]`` (``Tk >= Tq``; the
    queries are the last ``Tq`` tokens; grouped-query sharing; causal by default), float16 / bfloat16, ``D = 128``:
    the attention of a prompt before the cache compresses it.  Returns a tensor shaped like ``q``."""
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("prefill_attention needs q, k, v in the same 16-bit float dtype")
    if not q.is_cuda:
        raise RuntimeError("prefill_attention runs on CUDA tensors only")
    if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[3] != q.shape[3]:
        raise ValueError("q [B, Hq, Tq, D], k / v [B, H, Tk, D]")

    def usable(t: Tensor) -> Tensor:
        ok = t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()

    q, k, v = usable(q), usable(k), usable(v)
    B, Hq, Tq, D = q.shape
    H, Tk = k.shape[1], k.shape[2]
    # token-major storage [B, Tq, Hq, D] behind the [B, Hq, Tq, D] result: the o projection that follows reads the
    # heads of a token side by side, so its ``transpose(1, 2).reshape(B * Tq, Hq * D)`` is a view, not a copy
    out = torch.empty(B, Tq, Hq, D, device=q.device, dtype=q.dtype).transpose(1, 2)
    status = _lib.lib().pare_prefill_attn(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _lib.dtype_code(q.dtype),
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2),
        out.stride(0), out.stride(1), out.stride(2), B, Hq, H, Tq, Tk, D,
        float(scale if scale is not None else 1.0 / math.sqrt(D)), 1 if causal else 0, _lib.current_stream(q.device))
    _lib.check(status, "pare_prefill_attn")
    return out


def plan_update(r_len: int, n_new: int, residual_length: int, group_size: int) -> tuple[int, int]:
    """Compression schedule of one ``update`` (reference: ``pare/kv_cache.py:231-244``).

    Returns ``(tokens_to_compress, new_residual_length)``: whole groups, oldest first, of
    whatever exceeds the residual budget after appending ``n_new`` tokens.
    """
    total = r_len + n_new
    n_c = (max(0, total - residual_length) // group_size) * group_size
    return n_c, total - n_c


def _roundup(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _unpack_along_last(packed: Tensor, bits: int, n: int) -> Tensor:
    """uint8 ``[..., n*bits/8]`` → uint8 ``[..., n]`` (element e at bit e*bits, little endian)."""
    per = 8 // bits
    p = packed.to(torch.int32).unsqueeze(-1)
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    return ((p >> shifts) & ((1 << bits) - 1)).reshape(*packed.shape[:-1], -1)[..., :n].to(torch.uint8)


class _LayerStore:
    """Preallocated packed storage of one layer."""

    def __init__(self, B: int, H: int, D: int, cfg: KVCacheConfig, cap: int, device, dtype) -> None:
        self.B, self.H, self.D, self.cfg, self.device, self.dtype = B, H, D, cfg, device, dtype
        self.v_group = cfg.v_group_size or D          # channels per value scale / zero
        if self.v_group % 32 or D % self.v_group:
            raise ValueError("v_group_size must be a multiple of 32 that divides the head dimension")
        self.n_comp = 0
        self.r_len = 0
        self.r_cap = _roundup(cfg.residual_length + 2 * cfg.group_size, 8)
        self.res_k = torch.empty(B, H, self.r_cap, D, device=device, dtype=dtype)
        self.res_v = torch.empty(B, H, self.r_cap, D, device=device, dtype=dtype)
        self.cap = 0
        self._alloc(cap)

    def _alloc(self, cap: int) -> None:
        cap = _roundup(max(cap, _V_BLOCK), math.lcm(_V_BLOCK, self.cfg.group_size))
        B, H, D, bits, G = self.B, self.H, self.D, self.cfg.bits, self.cfg.group_size
        vg = D // self.v_group
        dev = self.device
        new = dict(
            k_codes=torch.empty(B, H, cap, D * bits // 8, dtype=torch.uint8, device=dev),
            k_scale=torch.empty(B, H, cap // G, D, dtype=torch.float32, device=dev),
            k_zero=torch.empty(B, H, cap // G, D, dtype=torch.float32, device=dev),
            v_codes=torch.empty(B, H, cap // _V_BLOCK, D, _V_BLOCK * bits // 8, dtype=torch.uint8, device=dev),
            v_scale=torch.empty(B, H, cap, vg, dtype=torch.float32, device=dev),
            v_zero=torch.empty(B, H, cap, vg, dtype=torch.float32, device=dev),
        )
        if self.cap:  # growing: carry the compressed tokens over
            n, nb = self.n_comp, _roundup(self.n_comp, _V_BLOCK) // _V_BLOCK
            new["k_codes"][:, :, :n] = self.k_codes[:, :, :n]
            new["k_scale"][:, :, : n // G] = self.k_scale[:, :, : n // G]
            new["k_zero"][:, :, : n // G] = self.k_zero[:, :, : n // G]
            new["v_codes"][:, :, :nb] = self.v_codes[:, :, :nb]
            new["v_scale"][:, :, :n] = self.v_scale[:, :, :n]
            new["v_zero"][:, :, :n] = self.v_zero[:, :, :n]
        for k, v in new.items():
            setattr(self, k, v)
        self.cap = cap

    def reserve(self, n_tokens: int) -> None:
        if n_tokens > self.cap:
            self._alloc(max(n_tokens, 2 * self.cap))

    def cache_args(self) -> tuple:
        return (self.k_codes.data_ptr(), self.k_scale.data_ptr(), self.k_zero.data_ptr(),
                self.v_codes.data_ptr(), self.v_scale.data_ptr(), self.v_zero.data_ptr())

    def geometry(self) -> tuple:
        return (self.B, self.H, self.D, self.cfg.bits, self.cfg.group_size, self.v_group, self.cap)


class _CompressedKV:
    """Read-only logical view of a layer's compressed tokens (shapes as in the reference's
    ``_CompressedKV`` NamedTuple, ``pare/kv_cache.py:62-68``); codes are unpacked on access."""

    def __init__(self, store: _LayerStore) -> None:
        self._s = store

    @property
    def k_quant(self) -> Tensor:
        s = self._s
        return _unpack_along_last(s.k_codes[:, :, : s.n_comp], s.cfg.bits, s.D)

    @property
    def v_quant(self) -> Tensor:
        s = self._s
        nb = _roundup(s.n_comp, _V_BLOCK) // _V_BLOCK
        blocks = _unpack_along_last(s.v_codes[:, :, :nb], s.cfg.bits, _V_BLOCK)        # [B,H,nb,D,128]
        return blocks.permute(0, 1, 2, 4, 3).reshape(s.B, s.H, nb * _V_BLOCK, s.D)[:, :, : s.n_comp].contiguous()

    def _key_meta(self, stored: Tensor) -> Tensor:
        """Stored key scale / zero rows -> channel order.  Inside every 128 channels the kernels keep the row as
        [word (c>>3)&3][lane quad (c>>5)&3][c&7] (what the decode-attention kernel reads conflict-free)."""
        s = self._s
        rows = stored[:, :, : s.n_comp // s.cfg.group_size]
        if s.D % 128:
            return rows
        return rows.unflatten(-1, (s.D // 128, 4, 4, 8)).transpose(-3, -2).flatten(-4)

    @property
    def k_scale(self) -> Tensor:
        return self._key_meta(self._s.k_scale)

    @property
    def k_zero(self) -> Tensor:
        return self._key_meta(self._s.k_zero)

    @property
    def v_scale(self) -> Tensor:
        return self._s.v_scale[:, :, : self._s.n_comp]   # [B, H, n, D / v_group]: [.., 1] in the reference's form

    @property
    def v_zero(self) -> Tensor:
        return self._s.v_zero[:, :, : self._s.n_comp]

    def __iter__(self):
        return iter((self.k_quant, self.k_scale, self.k_zero, self.v_quant, self.v_scale, self.v_zero))


class QuantizedKVCache:
    """Per-layer KIVI cache.

    Args:
        num_layers:  number of transformer layers.
        config:      :class:`KVCacheConfig`; defaults to 4-bit, groups of 32, residual 128.
        max_seq_len: optional token capacity to preallocate per layer; without it the packed
                     buffers start at 1024 tokens and double when full.
    """

    def __init__(self, num_layers: int, config: KVCacheConfig | None = None, max_seq_len: int | None = None) -> None:
        self.num_layers = num_layers
        self.config = config or KVCacheConfig()
        if self.config.bits not in (2, 4, 8):
            raise ValueError(f"Unsupported bits for the CUDA cache: {self.config.bits}")
        self.max_seq_len = max_seq_len
        self._stores: list[_LayerStore | None] = [None] * num_layers
        self._compressed: list[_CompressedKV | None] = [None] * num_layers
        self._residual_k: list[Tensor | None] = [None] * num_layers
        self._residual_v: list[Tensor | None] = [None] * num_layers

    # ------------------------------------------------------------------ internals
    def _store(self, layer_idx: int, like: Tensor) -> _LayerStore:
        st = self._stores[layer_idx]
        if st is None:
            if not like.is_cuda:
                raise RuntimeError("QuantizedKVCache runs on CUDA tensors only (no CPU implementation).")
            B, H, _, D = like.shape
            cap = self.max_seq_len if self.max_seq_len else 1024
            st = _LayerStore(B, H, D, self.config, cap, like.device, like.dtype)
            self._stores[layer_idx] = st
        return st

    def _append(self, layer_idx: int, new_k: Tensor, new_v: Tensor, defer_single: bool = False, rope: Tensor | None = None):
        """Append tokens to the residual window and compress what overflows it.

        With ``defer_single`` returns ``(store, deferred)``: when one token arrives and nothing has
        to be compressed, the copy into the window is left to the attention kernel (``deferred``).  ``rope``: rows of
        a :func:`rope_table` for the new tokens; applied to the keys here unless the append is deferred (then the
        attention kernel does it)."""
        if new_k.shape != new_v.shape or new_k.dim() != 4:
            raise ValueError("new_k / new_v must both be [B, H, new_tokens, D]")
        st = self._store(layer_idx, new_k)
        if new_k.dtype != st.dtype or new_k.shape[0] != st.B or new_k.shape[1] != st.H or new_k.shape[3] != st.D:
            raise ValueError("update() called with a different batch / heads / head_dim / dtype than before")
        cfg = self.config
        n_new = new_k.shape[2]
        n_c, r_after = plan_update(st.r_len, n_new, cfg.residual_length, cfg.group_size)
        total = st.r_len + n_new

        deferred = (defer_single and n_new == 1 and n_c == 0 and total <= st.r_cap
                    and new_k.data_ptr() % 16 == 0 and new_v.data_ptr() % 16 == 0
                    and all(t.stride(3) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 for t in (new_k, new_v))
                    and new_k.stride() == new_v.stride())
        if rope is not None and not deferred:   # the kernel rotates only a key it appends itself
            new_k = apply_rope(new_k, rope)
        if deferred:
            pass
        elif total <= st.r_cap:
            st.res_k[:, :, st.r_len:total] = new_k
            st.res_v[:, :, st.r_len:total] = new_v
            src_k, src_v = st.res_k, st.res_v
        else:  # bulk prefill: larger than the window buffer, go through a temporary
            src_k = torch.cat([st.res_k[:, :, : st.r_len], new_k], dim=2)
            src_v = torch.cat([st.res_v[:, :, : st.r_len], new_v], dim=2)

        if n_c > 0:
            st.reserve(st.n_comp + n_c)
            L = _lib.lib()
            status = L.pare_kivi_append(
                src_k.data_ptr(), src_v.data_ptr(), _lib.dtype_code(st.dtype),
                src_k.stride(0), src_k.stride(1), src_k.stride(2),
                n_c, st.n_comp, *st.cache_args(), *st.geometry(),
                _lib.current_stream(st.device),
            )
            _lib.check(status, "pare_kivi_append")
            st.n_comp += n_c
            keep_k = src_k[:, :, n_c:total]
            keep_v = src_v[:, :, n_c:total]
            if src_k is st.res_k:  # shifting inside the same buffer: go through a copy
                keep_k, keep_v = keep_k.clone(), keep_v.clone()
            st.res_k[:, :, :r_after] = keep_k
            st.res_v[:, :, :r_after] = keep_v
        st.r_len = r_after

        self._compressed[layer_idx] = _CompressedKV(st) if st.n_comp > 0 else None
        self._residual_k[layer_idx] = st.res_k[:, :, : st.r_len]
        self._residual_v[layer_idx] = st.res_v[:, :, : st.r_len]
        return (st, deferred) if defer_single else st

    # ------------------------------------------------------------------ public API
    def update(self, layer_idx: int, new_k: Tensor, new_v: Tensor) -> tuple[Tensor, Tensor]:
        """Append ``[B, H, new_tokens, D]`` keys / values; return the dense ``(K, V)`` of the whole
        sequence in the input dtype (reference contract, ``pare/kv_cache.py:205-252``)."""
        st = self._append(layer_idx, new_k, new_v)
        total = st.n_comp + st.r_len
        full_k = torch.empty(st.B, st.H, total, st.D, device=st.device, dtype=st.dtype)
        full_v = torch.empty_like(full_k)
        if st.n_comp > 0:
            status = _lib.lib().pare_kivi_dequant(
                *st.cache_args(), *st.geometry(), st.n_comp,
                full_k.data_ptr(), full_v.data_ptr(), _lib.dtype_code(st.dtype),
                full_k.stride(0), full_k.stride(1), full_k.stride(2),
                _lib.current_stream(st.device),
            )
            _lib.check(status, "pare_kivi_dequant")
        full_k[:, :, st.n_comp:] = st.res_k[:, :, : st.r_len]
        full_v[:, :, st.n_comp:] = st.res_v[:, :, : st.r_len]
        return full_k, full_v

    def attend(self, layer_idx: int, q: Tensor, new_k: Tensor, new_v: Tensor, scale: float | None = None,
               prepared_out=None, rope: Tensor | None = None) -> Tensor | None:
        """Append one step's keys / values, then attention of ``q`` over the whole cache.

        ``q`` is ``[B, Hq, 1, D]`` (or ``[B, Hq, D]``) with ``Hq`` a multiple of the KV heads
        (grouped-query attention, at most 8 query heads per KV head).  Equivalent to
        ``softmax(q K^T * scale) V`` on the tensors :meth:`update` would return, computed from
        the packed cache without reconstructing it.  Returns a tensor shaped like ``q``.

        A single new token that needs no compression in this step is not copied by the host
        side at all: the attention kernel reads it where it is and stores it into the residual
        window itself.  With ``prepared_out`` (a ``PreparedActivations`` of ``B`` rows and
        ``Hq * D`` columns) the result is written as prepared activations of the next linear
        instead, and ``None`` is returned.  With ``rope`` (row ``[D]`` of a :func:`rope_table` for the new token's
        position, float32) ``q`` and the new key get the rotary embedding inside the same launch, and the key is
        stored rotated; ``q`` and ``new_k`` are then what the q|k|v projection gave, one new token only.
        """
        if q.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("attend() needs q in float16 or bfloat16")
        if rope is not None:
            if new_k.shape[2] != 1 or rope.shape != (q.shape[-1],) or rope.dtype != torch.float32 or not rope.is_contiguous():
                raise ValueError("rope must be one float32 row [D] of rope_table and needs exactly one new token")
        st, fused_new = self._append(layer_idx, new_k, new_v, defer_single=True, rope=rope)
        if q.dtype != st.dtype:
            raise ValueError("attend() needs q in the cache dtype")
        q3 = q.reshape(q.shape[0], q.shape[1], q.shape[-1])
        if q3.stride(-1) != 1:
            q3 = q3.contiguous()
        B, Hq, D = q3.shape
        out = None if prepared_out is not None else torch.empty(B, Hq, D, device=q.device, dtype=q.dtype)
        if prepared_out is not None and (prepared_out.rows, prepared_out.k, prepared_out.dtype) != (B, Hq * D, q.dtype):
            raise ValueError("prepared_out does not match the attention output")
        nk = nv = None
        if fused_new:
            nk, nv = new_k[:, :, 0], new_v[:, :, 0]     # [B, H, D] views
            if nk.stride(-1) != 1 or nv.stride() != nk.stride():
                nk, nv = nk.contiguous(), nv.contiguous()
        L = _lib.lib()
        ws = _lib.workspace(st.device, L.pare_kivi_attn_workspace_bytes(B, st.H, st.n_comp, st.r_len))
        status = L.pare_kivi_decode_attn(
            q3.data_ptr(), _lib.dtype_code(q.dtype), q3.stride(0), q3.stride(1),
            *st.cache_args(), st.n_comp,
            st.res_k.data_ptr(), st.res_v.data_ptr(), st.res_k.stride(0), st.res_k.stride(1), st.res_k.stride(2), st.r_len,
            _lib.ptr(nk), _lib.ptr(nv), nk.stride(0) if fused_new else 0, nk.stride(1) if fused_new else 0,
            _lib.ptr(rope),
            _lib.ptr(out), out.stride(0) if out is not None else 0, out.stride(1) if out is not None else 0,
            prepared_out.data_ptr() if prepared_out is not None else None,
            float(scale if scale is not None else 1.0 / math.sqrt(D)),
            B, Hq, st.H, D, self.config.bits, self.config.group_size, st.v_group, st.cap,
            ws.data_ptr(), ws.numel(), _lib.current_stream(st.device),
        )
        _lib.check(status, "pare_kivi_decode_attn")
        return None if out is None else out.reshape(q.shape)

    def prefill(self, layer_idx: int, q: Tensor, new_k: Tensor, new_v: Tensor, scale: float | None = None,
                rope: Tensor | None = None) -> Tensor:
        """Causal attention of a prompt's ``q [B, Hq, T, D]`` over its own ``new_k, new_v [B, H, T, D]`` in full precision,
        then the append of those tokens (whole groups beyond the window are compressed).  On a cache that already
        holds tokens the older ones come from :meth:`update`'s dense return, as a caller of the reference would attend
        to them.  ``rope``: rows ``[T, D]`` of a :func:`rope_table` for the new tokens' positions, applied to ``q`` and
        ``new_k`` first (the keys are stored rotated)."""
        if rope is not None:
            q, new_k = apply_rope(q, rope), apply_rope(new_k, rope)
        if self.seq_len(layer_idx) == 0:
            out = prefill_attention(q, new_k, new_v, scale, causal=True)
            self._append(layer_idx, new_k, new_v)
            return out
        full_k, full_v = self.update(layer_idx, new_k, new_v)
        n_new = new_k.shape[2]
        full_k[:, :, -n_new:] = new_k          # the new tokens themselves at full precision
        full_v[:, :, -n_new:] = new_v
        return prefill_attention(q, full_k, full_v, scale, causal=True)

    def reset(self, layer_idx: int | None = None) -> None:
        """Forget one layer or all layers (buffers are released and reallocated on next use)."""
        for i in range(self.num_layers) if layer_idx is None else (layer_idx,):
            self._stores[i] = None
            self._compressed[i] = None
            self._residual_k[i] = None
            self._residual_v[i] = None

    def seq_len(self, layer_idx: int) -> int:
        st = self._stores[layer_idx]
        return 0 if st is None else st.n_comp + st.r_len

    def memory_bytes(self, layer_idx: int) -> dict[str, int]:
        """Bytes in use (not capacity) for one layer: packed codes + fp32 metadata, and the window."""
        st = self._stores[layer_idx]
        if st is None:
            return {"compressed": 0, "residual": 0, "total": 0}
        bh, n, G = st.B * st.H, st.n_comp, self.config.group_size
        comp = bh * (2 * n * st.D * self.config.bits // 8 + 2 * (n // G) * st.D * 4 + 2 * n * 4 * (st.D // st.v_group))
        res = 2 * bh * st.r_len * st.D * st.res_k.element_size()
        return {"compressed": comp, "residual": res, "total": comp + res}


# ----------------------------------------------------------------------------------------
# The four primitives of the reference module, on CUDA, returned in the reference's shapes
# (pare/kv_cache.py:75-156).  They run the same kernels as the cache.
# ----------------------------------------------------------------------------------------

def _quantize_block(k: Tensor, v: Tensor, bits: int, group_size: int, v_group_size: int | None = None) -> _CompressedKV:
    if not k.is_cuda:
        raise RuntimeError("the KIVI primitives run on CUDA tensors only")
    B, H, n, D = k.shape
    if n % group_size:
        raise ValueError(f"n={n} must be divisible by group_size={group_size}")
    st = _LayerStore(B, H, D, KVCacheConfig(bits, group_size, 0, v_group_size), n, k.device, k.dtype)
    k, v = k.contiguous(), v.contiguous()
    status = _lib.lib().pare_kivi_append(
        k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype), k.stride(0), k.stride(1), k.stride(2),
        n, 0, *st.cache_args(), *st.geometry(), _lib.current_stream(k.device))
    _lib.check(status, "pare_kivi_append")
    st.n_comp = n
    return _CompressedKV(st)


def _quantize_keys(k: Tensor, bits: int, group_size: int) -> tuple[Tensor, Tensor, Tensor]:
    c = _quantize_block(k, k, bits, group_size)
    return c.k_quant, c.k_scale, c.k_zero


def _quantize_values(v: Tensor, bits: int, group_size: int, v_group_size: int | None = None) -> tuple[Tensor, Tensor, Tensor]:
    c = _quantize_block(v, v, bits, group_size, v_group_size)
    return c.v_quant, c.v_scale, c.v_zero


def _dequantize_keys(k_quant: Tensor, k_scale: Tensor, k_zero: Tensor, group_size: int) -> Tensor:
    """fp32 ``code * scale + zero`` with one (scale, zero) per group and channel (elementwise torch;
    kept for callers of the reference's private helper, not used by the cache itself)."""
    B, H, n, D = k_quant.shape
    q = k_quant.float().reshape(B, H, n // group_size, group_size, D)
    return (q * k_scale.unsqueeze(3) + k_zero.unsqueeze(3)).reshape(B, H, n, D)


def _dequantize_values(v_quant: Tensor, v_scale: Tensor, v_zero: Tensor) -> Tensor:
    if v_scale.shape[-1] > 1:   # one pair per group of channels
        B, H, n, D = v_quant.shape
        q = v_quant.float().reshape(B, H, n, v_scale.shape[-1], -1)
        return (q * v_scale.unsqueeze(-1) + v_zero.unsqueeze(-1)).reshape(B, H, n, D)
    return v_quant.float() * v_scale + v_zero
