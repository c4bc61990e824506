"""A decode stack made only of the hot path: W4A16 linears + KIVI attention, chained per layer.

This is the measurement vehicle for "decode tok/s": every transformer block is
``rmsnorm -> fused q|k|v linear -> KIVI append + fused decode attention -> o linear ->
rmsnorm(+residual) -> fused gate|up linear -> SwiGLU -> down linear``, with random-init INT4
weights of the requested shape.  The linears are ordinary :class:`QuantizedLinear` modules
(``use_kernel=True``) and the cache an ordinary :class:`QuantizedKVCache`, i.e. the public API
a user of the reference would call; q and the new key get their rotary embedding inside the
attention launch; the token embedding and the LM head are left out (they are not part of the
path this package replaces).

Tensor parallelism (one process per GPU): ONE model is built from the seeds and every rank keeps
its slice of it -- q|k|v and gate|up split by output rows (whole heads / FFN columns per rank),
o and down by input columns in whole groups, the KV cache by KV head.  The two row-parallel
outputs of a block are summed over the ranks by the one-launch peer all-reduce over NVLink
(``pare_peer_allreduce``), NCCL for tensors too large for its exchange buffers.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch import Tensor

from pare_b200.config import QuantConfig
from pare_b200.kernels import _lib
from pare_b200.kernels.matmul_int4 import PreparedActivations
from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache, rope_table
from pare_b200.layers.linear import QuantizedLinear

SHAPES = {
    # hidden, ffn, q heads, kv heads, head_dim, layers
    "llama-3.1-8b": (4096, 14336, 32, 8, 128, 32),
    "llama-3-70b": (8192, 28672, 64, 8, 128, 80),
    "qwen2.5-7b": (3584, 18944, 28, 4, 128, 28),
}


def synthetic_linear(out_features: int, in_features: int, *, seed: int, device, group_size: int = 128,
                     awq_fold: bool = True) -> QuantizedLinear:
    """Random-init INT4 g128 layer built directly in packed form on ``device``.

    Codes are uniform in 0..15 with zero-point 8; scales are chosen so that the dequantized
    weights have standard deviation 0.02, multiplied per input-channel group by a
    LogNormal(0, 0.3) factor when ``awq_fold`` (what an AWQ-quantized layer stores: the input
    scale is folded into the weights offline, the layer at run time is a plain asymmetric one).
    """
    g = torch.Generator(device=device).manual_seed(seed)
    packed = torch.randint(0, 256, (out_features, in_features // 2), dtype=torch.uint8, device=device, generator=g)
    ng = in_features // group_size
    scale = torch.full((out_features, ng, 1), 0.02 / 4.61, device=device)
    scale = scale * (0.75 + 0.5 * torch.rand(out_features, ng, 1, device=device, generator=g))
    if awq_fold:
        scale = scale * torch.exp(0.3 * torch.randn(1, ng, 1, device=device, generator=g))
    zero = torch.randint(6, 11, (out_features, ng, 1), device=device, generator=g).float()
    cfg = QuantConfig(bits=4, scheme="awq", granularity="per_group", group_size=group_size)
    layer = QuantizedLinear.from_tensors(packed, None, scale, zero, cfg, None, in_features, out_features)
    layer.use_kernel = True
    return layer


def _take_rows(layer: QuantizedLinear, ranges: list[tuple[int, int]]) -> QuantizedLinear:
    """The output rows ``[a, b)`` of every range, concatenated (a column-parallel shard of a fused projection)."""
    idx = torch.cat([torch.arange(a, b, device=layer.packed_weight.device) for a, b in ranges])
    shard = QuantizedLinear.from_tensors(layer.packed_weight[idx].contiguous(), None, layer.scale[idx].contiguous(),
                                         layer.zero[idx].contiguous(), layer.config, None, layer.in_features, idx.numel())
    shard.use_kernel = True
    return shard


def _take_cols(layer: QuantizedLinear, a: int, b: int) -> QuantizedLinear:
    """The input columns ``[a, b)`` in whole groups (a row-parallel shard)."""
    g = layer.config.group_size
    assert a % g == 0 and b % g == 0
    shard = QuantizedLinear.from_tensors(layer.packed_weight[:, a // 2:b // 2].contiguous(), None,
                                         layer.scale[:, a // g:b // g].contiguous(), layer.zero[:, a // g:b // g].contiguous(),
                                         layer.config, None, b - a, layer.out_features)
    shard.use_kernel = True
    return shard


class DecodeBlock(nn.Module):
    """One block's four fused projections.  With ``tp_world > 1`` the FULL layers are generated from the seeds (the same
    on every rank) and this rank keeps its slice: its query / key / value heads of q|k|v, its FFN columns of gate|up,
    the matching input columns of o and down."""

    def __init__(self, hidden: int, ffn: int, hq: int, hkv: int, d: int, *, seed: int, device, dtype,
                 tp_world: int = 1, tp_rank: int = 0) -> None:
        super().__init__()
        assert hq % tp_world == 0 and hkv % tp_world == 0 and ffn % (tp_world * 128) == 0
        self.hq, self.hkv, self.d, self.ffn = hq // tp_world, hkv // tp_world, d, ffn // tp_world
        self.hidden = hidden
        qkv = synthetic_linear((hq + 2 * hkv) * d, hidden, seed=seed * 7 + 0, device=device)
        o = synthetic_linear(hidden, hq * d, seed=seed * 7 + 3, device=device)
        gate_up = synthetic_linear(2 * ffn, hidden, seed=seed * 7 + 4, device=device)
        down = synthetic_linear(hidden, ffn, seed=seed * 7 + 6, device=device)
        if tp_world > 1:
            r, nq, nkv, nf = tp_rank, self.hq * d, self.hkv * d, self.ffn
            qkv = _take_rows(qkv, [(r * nq, (r + 1) * nq), (hq * d + r * nkv, hq * d + (r + 1) * nkv),
                                   ((hq + hkv) * d + r * nkv, (hq + hkv) * d + (r + 1) * nkv)])
            o = _take_cols(o, r * nq, (r + 1) * nq)
            gate_up = _take_rows(gate_up, [(r * nf, (r + 1) * nf), (ffn + r * nf, ffn + (r + 1) * nf)])
            down = _take_cols(down, r * nf, (r + 1) * nf)
        self.qkv, self.o, self.gate_up, self.down = qkv, o, gate_up, down
        self.register_buffer("norm1", torch.ones(hidden, device=device, dtype=dtype))
        self.register_buffer("norm2", torch.ones(hidden, device=device, dtype=dtype))


class DecodeStack(nn.Module):
    """``n_layers`` decode blocks over one shared :class:`QuantizedKVCache`."""

    def __init__(self, shape: str | tuple, *, device="cuda", dtype=torch.bfloat16, n_layers: int | None = None,
                 kv_config: KVCacheConfig | None = None, max_seq_len: int = 8192, tp_world: int = 1,
                 process_group=None, seed: int = 0, peer_all_reduce: bool = True,
                 rope_theta: float | None = 500000.0, tp_rank: int | None = None) -> None:
        super().__init__()
        hidden, ffn, hq, hkv, d, layers = SHAPES[shape] if isinstance(shape, str) else shape
        self.hidden, self.d = hidden, d
        self.hkv_total = hkv
        self.n_layers = n_layers or layers
        self.dtype, self.device = dtype, torch.device(device)
        self.tp_world, self.group = tp_world, process_group
        if tp_rank is None:
            tp_rank = torch.distributed.get_rank(process_group) if tp_world > 1 else 0
        self.tp_rank = tp_rank
        self.blocks = nn.ModuleList(
            DecodeBlock(hidden, ffn, hq, hkv, d, seed=seed + i, device=self.device, dtype=dtype, tp_world=tp_world,
                        tp_rank=tp_rank)
            for i in range(self.n_layers))
        self.cache = QuantizedKVCache(self.n_layers, kv_config or KVCacheConfig(), max_seq_len=max_seq_len)
        self._code = _lib.dtype_code(dtype)
        self._prep_cache: dict[int, tuple] = {}
        # rotary table [positions, D] (None: no positional rotation); q and the new key are rotated inside the attention launch
        self.rope = rope_table(max_seq_len + 1, d, rope_theta, self.device) if rope_theta else None
        # one-launch all-reduce over NVLink peer memory for the small decode tensors; NCCL for anything larger
        self.peer_reduce = None
        if tp_world > 1 and peer_all_reduce:
            from pare_b200.parallel import PeerAllReduce
            self.peer_reduce = PeerAllReduce(process_group)

    # ---- glue kernels ------------------------------------------------------------------
    def _rmsnorm(self, x: Tensor, delta: Tensor | None, weight: Tensor, store_residual: bool, prepared=None):
        """rmsnorm(x + delta) * weight as a tensor, or into ``prepared`` (then returns None)."""
        y = None if prepared is not None else torch.empty_like(x)
        status = _lib.lib().pare_rmsnorm_residual(
            x.data_ptr(), _lib.ptr(delta), weight.data_ptr(), x.data_ptr() if store_residual else None, _lib.ptr(y),
            prepared.data_ptr() if prepared is not None else None,
            x.shape[0], x.shape[1], 1e-5, self._code, _lib.current_stream(x.device))
        _lib.check(status, "pare_rmsnorm_residual")
        return y

    def _silu_mul(self, gate_up: Tensor, n: int, prepared=None):
        out = None if prepared is not None else torch.empty(gate_up.shape[0], n, device=gate_up.device, dtype=gate_up.dtype)
        status = _lib.lib().pare_silu_mul(gate_up.data_ptr(), _lib.ptr(out),
                                          prepared.data_ptr() if prepared is not None else None,
                                          gate_up.shape[0], n, gate_up.stride(0),
                                          self._code, _lib.current_stream(gate_up.device))
        _lib.check(status, "pare_silu_mul")
        return out

    def _prepared(self, m: int):
        """Per-batch-size hand-over buffer between the attention kernel and the o projection."""
        buf = self._prep_cache.get(m)
        if buf is None:
            blk = self.blocks[0]
            buf = PreparedActivations(m, blk.hq * blk.d, self.dtype, self.device)
            self._prep_cache[m] = buf
        return buf

    def _all_reduce(self, t: Tensor) -> Tensor:
        if self.tp_world > 1:
            if self.peer_reduce is not None and t.numel() <= self.peer_reduce.max_elements() and t.shape[1] % 4 == 0:
                return self.peer_reduce(t)
            torch.distributed.all_reduce(t, group=self.group)
        return t

    # ---- cache set-up -----------------------------------------------------------------
    @torch.no_grad()
    def prefill_cache(self, batch: int, context: int, seed: int = 1) -> None:
        """Fill every layer's cache with ``context`` synthetic tokens: N(0,1) with 1 % of the channels
        (same channels for all tokens) scaled by 10, the stand-in for real K/V statistics.  Under tensor
        parallelism the tokens of ALL KV heads are generated (the same on every rank, one head at a time) and this
        rank keeps its heads."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        blk = self.blocks[0]
        mine = range(self.tp_rank * blk.hkv, (self.tp_rank + 1) * blk.hkv)
        for layer in range(self.n_layers):
            out_ch = torch.randperm(self.d, device=self.device, generator=g)[: max(1, self.d // 100)]
            ks, vs = [], []
            for head in range(self.hkv_total):
                k = torch.randn(batch, 1, context, self.d, device=self.device, generator=g)
                v = torch.randn(batch, 1, context, self.d, device=self.device, generator=g)
                if head in mine:
                    k[..., out_ch] *= 10.0
                    ks.append(k.to(self.dtype))
                    vs.append(v.to(self.dtype))
            self.cache.reset(layer)
            self.cache._append(layer, torch.cat(ks, dim=1), torch.cat(vs, dim=1))

    # ---- the prompt -----------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, x: Tensor) -> Tensor:
        """``x [B, T, hidden]``: hidden states of a prompt's tokens -> same shape, and the caches hold the prompt.

        Per block: RMSNorm, q|k|v linear (``B T`` rows: the tensor-core path for long prompts), rotary embedding, causal
        attention over the full-precision keys / values of the prompt (``QuantizedKVCache.prefill``, which then
        compresses what lies beyond the window), o linear, RMSNorm, gate|up linear, SwiGLU, down linear.  A later
        call continues the sequence (chunked prefill)."""
        B, T, hidden = x.shape
        pos0 = self.cache.seq_len(0)
        rope = self.rope[pos0:pos0 + T] if self.rope is not None else None
        resid = x.reshape(B * T, hidden).clone()
        delta = None
        for i, blk in enumerate(self.blocks):
            d, hq, hkv = blk.d, blk.hq, blk.hkv
            qkv = blk.qkv(self._rmsnorm(resid, delta, blk.norm1, store_residual=delta is not None)).view(B, T, -1)
            q = qkv[..., : hq * d].unflatten(2, (hq, d)).transpose(1, 2)                    # [B, hq, T, d] views
            k = qkv[..., hq * d:(hq + hkv) * d].unflatten(2, (hkv, d)).transpose(1, 2)
            v = qkv[..., (hq + hkv) * d:].unflatten(2, (hkv, d)).transpose(1, 2)
            attn = self.cache.prefill(i, q, k, v, scale=1.0 / math.sqrt(d), rope=rope)      # [B, hq, T, d]
            o = self._all_reduce(blk.o(attn.transpose(1, 2).reshape(B * T, hq * d)))
            h2 = self._rmsnorm(resid, o, blk.norm2, store_residual=True)
            delta = self._all_reduce(blk.down(self._silu_mul(blk.gate_up(h2), blk.ffn)))
        return (resid + delta).view(B, T, hidden)

    # ---- one decode step ---------------------------------------------------------------
    @torch.no_grad()
    def forward(self, x: Tensor) -> Tensor:
        """``x [M, hidden]``: hidden state of the newest token of each of M sequences → same shape.

        For M <= 16 a block is five launches, at any tensor-parallel degree (the sums over the ranks after the o and
        down linears are added inside those kernels): q|k|v linear (normalises the residual stream itself),
        attention (appends the new K / V token, hands its output over as prepared activations), o linear,
        gate|up linear (adds the attention branch to the residual stream and normalises it itself), down
        linear (applies the SwiGLU gate itself).  Larger M takes plain tensors and stand-alone glue kernels.
        """
        m = x.shape[0]
        resid = x.clone(memory_format=torch.contiguous_format)   # a one-row slice of a larger tensor keeps its odd row stride otherwise
        delta = None
        blk0 = self.blocks[0]
        fused = all(l.supports_prepared(m) for l in (blk0.qkv, blk0.o, blk0.gate_up, blk0.down))
        if fused:
            p_attn = self._prepared(m)
            spare = torch.empty_like(resid)   # the residual stream ping-pongs: the kernels that normalise it read one, write the other
        rope = self.rope[self.cache.seq_len(0)] if self.rope is not None else None   # the new token's position
        for i, blk in enumerate(self.blocks):
            d, hq, hkv = blk.d, blk.hq, blk.hkv
            if fused:
                qkv = blk.qkv.forward_rmsnorm(resid, delta, blk.norm1, resid_out=spare if delta is not None else None)
                if delta is not None:
                    resid, spare = spare, resid
            else:
                qkv = blk.qkv(self._rmsnorm(resid, delta, blk.norm1, store_residual=delta is not None))
            q = qkv[:, : hq * d].unflatten(1, (hq, d))
            k = qkv[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, 1, d))
            v = qkv[:, (hq + hkv) * d:].unflatten(1, (hkv, 1, d))
            if fused:
                self.cache.attend(i, q, k, v, scale=1.0 / math.sqrt(d), prepared_out=p_attn, rope=rope)
                # tensor parallel: the sums of the two row-parallel layers over the ranks are added inside their kernels
                peer = self.peer_reduce if (self.tp_world > 1 and self.peer_reduce is not None
                                            and m * self.hidden <= self.peer_reduce.max_fused_elements()) else None
                o = blk.o.forward_prepared(p_attn, peer=peer)
                if peer is None:
                    o = self._all_reduce(o)
                gate_up = blk.gate_up.forward_rmsnorm(resid, o, blk.norm2, resid_out=spare)
                resid, spare = spare, resid
                delta = blk.down.forward_silu_mul(gate_up, peer=peer)
                if peer is None:
                    delta = self._all_reduce(delta)
            else:
                attn = self.cache.attend(i, q, k, v, scale=1.0 / math.sqrt(d), rope=rope)
                o = self._all_reduce(blk.o(attn.reshape(m, hq * d)))
                h2 = self._rmsnorm(resid, o, blk.norm2, store_residual=True)
                act = self._silu_mul(blk.gate_up(h2), blk.ffn)
                delta = self._all_reduce(blk.down(act))
        return resid + delta
