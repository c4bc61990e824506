"""Tensor-parallel helpers for the hot path (one process per GPU, ``torch.distributed``).

The reference has no distributed code at all; this is the sharding its layers admit:

* **column parallel** (q, k, v, gate, up): rank r keeps output rows ``[r*N/W, (r+1)*N/W)`` — dim 0
  of ``packed_weight`` / ``scale`` / ``zero`` / ``bias``.  No communication; outputs stay sharded.
* **row parallel** (o, down): rank r keeps input columns ``[r*K/W, (r+1)*K/W)`` — dim 1 of
  ``packed_weight`` (in bytes: half of that) and whole groups of ``scale`` / ``zero``; its input is
  the matching slice of the activations (already sharded by the preceding column-parallel layer),
  the partial outputs are summed with one all-reduce, the bias is added on rank 0 only.
* **KV cache**: whole KV heads per rank together with their group of query heads; no communication
  inside attention.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from pare_b200.layers.linear import QuantizedLinear


def shard_range(total: int, rank: int, world: int, multiple: int = 1) -> tuple[int, int]:
    """``[start, stop)`` of rank's equal share of ``total``; the share must be a multiple of ``multiple``."""
    if total % world or (total // world) % multiple:
        raise ValueError(f"cannot split {total} over {world} ranks in multiples of {multiple}")
    per = total // world
    return rank * per, (rank + 1) * per


def shard_linear(layer: QuantizedLinear, mode: str, rank: int, world: int) -> QuantizedLinear:
    """Return rank's shard of an INT4 ``QuantizedLinear`` (``mode`` = ``"column"`` or ``"row"``)."""
    if layer.packed_weight is None:
        raise ValueError("only INT4 (packed) layers can be sharded")
    n, k = layer.out_features, layer.in_features
    cfg = layer.config
    scale, zero = layer.scale, layer.zero
    if mode == "column":
        a, b = shard_range(n, rank, world)
        if scale.dim() == 0:
            s, z = scale, zero
        else:
            s, z = scale[a:b], zero[a:b]
        shard = QuantizedLinear.from_tensors(
            layer.packed_weight[a:b].contiguous(), None, s.contiguous(), z.contiguous(), cfg,
            None if layer.bias is None else layer.bias.detach()[a:b], k, b - a,
            g_idx=layer.g_idx, input_scale=layer.input_scale)
    elif mode == "row":
        if layer.g_idx is not None:
            raise ValueError("row-parallel sharding of an act-order layer is not supported")
        group = cfg.group_size if cfg.granularity == "per_group" else 2
        a, b = shard_range(k, rank, world, multiple=group)
        if cfg.granularity == "per_group":
            s, z = scale[:, a // group:b // group], zero[:, a // group:b // group]
        else:
            s, z = scale, zero
        shard = QuantizedLinear.from_tensors(
            layer.packed_weight[:, a // 2:b // 2].contiguous(), None, s.contiguous(), z.contiguous(), cfg,
            layer.bias.detach() if (layer.bias is not None and rank == 0) else None, b - a, n,
            input_scale=None if layer.input_scale is None else layer.input_scale[a:b].contiguous())
    else:
        raise ValueError(f"unknown mode {mode!r}")
    shard.use_kernel = layer.use_kernel
    shard.kernel_meta_fp16 = layer.kernel_meta_fp16
    return shard


def shard_heads(n_heads: int, rank: int, world: int) -> range:
    """The KV heads (or query heads) owned by ``rank``."""
    a, b = shard_range(n_heads, rank, world)
    return range(a, b)


def row_parallel_forward(shard: QuantizedLinear, x_shard: Tensor, group=None) -> Tensor:
    """``shard(x_shard)`` summed over the ranks of ``group`` (the exchange step of o / down)."""
    y = shard(x_shard)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, group=group)
    return y


def gather_columns(y_shard: Tensor, group=None) -> Tensor:
    """All-gather the outputs of a column-parallel layer along the last dim (for logits)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return y_shard
    parts = [torch.empty_like(y_shard) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, y_shard.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


class PeerAllReduce:
    """Sum of a small ``[rows, cols]`` fp16/bf16 tensor over the ranks of ``group`` through NVLink peer memory.

    One kernel launch per call (``pare_peer_allreduce``): every rank stores its partial into every peer's
    exchange buffer (each 8 bytes with their own validity marks, so there is no fence and no separate flag) and
    adds the partials from its own buffer in rank order as they arrive (fp32, deterministic, identical on all
    ranks).  The exchange buffers are allocated once here and shared by CUDA IPC handles
    exchanged over ``torch.distributed``; every rank must construct this object and then make the same
    sequence of calls.  Capturable in a CUDA graph.  2 <= world <= 8, one process per GPU on one node.
    """

    def __init__(self, group=None, max_bytes: int = 512 << 10) -> None:
        import ctypes as C

        import torch.distributed as dist

        from pare_b200.kernels import _lib

        self._lib = _lib
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError("PeerAllReduce serves 2..8 ranks")
        # every 8 bytes of data travel with 8 bytes of validity marks; the data area is split in two halves, one for the
        # stand-alone all-reduce, one for the exchange fused into the row-parallel linears (fp32 partials: 8 bytes per
        # element, i.e. max_bytes / 2 elements of a 16-bit tensor per call)
        self.buffer_bytes = 4096 + 2 * (2 * self.world * ((2 * max_bytes + 255) // 256 * 256))
        L = _lib.lib()
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        _lib.check(L.pare_peer_buffer_create(self.buffer_bytes, C.byref(own), handle), "pare_peer_buffer_create")
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, (self.rank, bytes(handle.raw)), group=group)
        ptrs = (C.c_void_p * self.world)()
        self._opened = []
        for r, h in handles:
            if r == self.rank:
                ptrs[r] = self._own
            else:
                peer = C.c_void_p()
                _lib.check(L.pare_peer_buffer_open(h, C.byref(peer)), "pare_peer_buffer_open")
                ptrs[r] = peer.value
                self._opened.append(peer.value)
        self._ptrs = ptrs
        dist.barrier(group=group)   # nobody stores into a buffer that is not mapped everywhere yet

    def max_elements(self) -> int:
        """Elements of a tensor the stand-alone all-reduce takes."""
        return ((self.buffer_bytes - 4096) // 2 // (2 * self.world) // 256 * 256) // 4

    def max_fused_elements(self) -> int:
        """Output elements (rows x out_features) of a row-parallel linear whose sum is added inside the kernel."""
        return ((self.buffer_bytes - 4096) // 2 // (2 * self.world) // 256 * 256) // 8

    def __call__(self, x, out=None):
        assert x.is_cuda and x.dim() == 2 and x.stride(1) == 1
        y = out if out is not None else torch.empty_like(x)
        status = self._lib.lib().pare_peer_allreduce(
            x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), x.shape[0], x.shape[1], self._lib.dtype_code(x.dtype),
            self.rank, self.world, self._ptrs, self.buffer_bytes, self._lib.current_stream(x.device))
        self._lib.check(status, "pare_peer_allreduce")
        return y

    def status(self, device) -> int:
        """0, or the timeout code if a wait for a peer ran out since the buffer was created (synchronises)."""
        return self._lib.lib().pare_peer_status(self._own, self._lib.current_stream(device))

    def close(self) -> None:
        L = self._lib.lib()
        for p in self._opened:
            L.pare_peer_buffer_close(p)
        self._opened = []
        if self._own:
            L.pare_peer_buffer_destroy(self._own)
            self._own = None
