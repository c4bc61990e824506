"""Tensor-parallel sharding on CPU with the gloo backend (world size 2): the sharded eager layers must
reproduce the unsharded layer — column parallel by all-gather, row parallel by all-reduce."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

from pare_b200.config import QuantConfig
from pare_b200.layers.linear import QuantizedLinear
from pare_b200.parallel import gather_columns, row_parallel_forward, shard_heads, shard_linear, shard_range


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer(n, k, bias, seed):
    torch.manual_seed(seed)
    return QuantizedLinear.from_linear(nn.Linear(k, n, bias=bias), QuantConfig(bits=4, scheme="rtn", group_size=128))


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(123)
        x = torch.randn(3, 512)
        up = _layer(1024, 512, True, seed=1)          # column parallel
        down = _layer(512, 1024, True, seed=2)        # row parallel
        full = down(torch.relu(up(x)))
        up_r, down_r = shard_linear(up, "column", rank, world), shard_linear(down, "row", rank, world)
        h_shard = torch.relu(up_r(x))                 # stays sharded: no communication
        y = row_parallel_forward(down_r, h_shard)     # one all-reduce
        err_row = (y - full).abs().max().item()
        err_col = (gather_columns(up_r(x)) - up(x)).abs().max().item()
        if rank == 0:
            out.put((err_row, err_col, tuple(up_r.packed_weight.shape), tuple(down_r.packed_weight.shape)))
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_match_unsharded():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_row, err_col, up_shape, down_shape = out.get(timeout=10)
    assert up_shape == (512, 256) and down_shape == (512, 256)
    assert err_col == 0.0                             # same rows, same arithmetic
    assert err_row < 1e-4                             # fp32 sums in a different order


def test_shard_ranges_and_heads():
    assert shard_range(4096, 1, 4) == (1024, 2048)
    assert list(shard_heads(8, 3, 4)) == [6, 7]
    import pytest
    with pytest.raises(ValueError):
        shard_range(4096, 0, 3)
    with pytest.raises(ValueError):
        shard_range(1024, 0, 16, multiple=128)        # 64 columns per rank is not a whole group


def _stack_slices_worker(rank: int, world: int, port: int, out):
    """The slicing the decode stack uses (``_take_rows`` of a fused q|k|v / gate|up, ``_take_cols`` of o / down): every
    rank cuts the same seeded full layers, the shards' eager forwards reassemble the unsharded results."""
    from pare_b200.decode import _take_cols, _take_rows

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hkv, d, hidden, ffn = 8, 2, 128, 512, 1024
        qkv = _layer((hq + 2 * hkv) * d, hidden, False, seed=3)
        gate_up = _layer(2 * ffn, hidden, False, seed=4)
        down = _layer(hidden, ffn, False, seed=5)
        torch.manual_seed(7)
        x = torch.randn(2, hidden)
        # q|k|v: this rank's query heads, key heads and value heads, in that order
        hq_r, hkv_r = hq // world, hkv // world
        k0, v0 = hq * d, (hq + hkv) * d
        ranges = [(rank * hq_r * d, (rank + 1) * hq_r * d), (k0 + rank * hkv_r * d, k0 + (rank + 1) * hkv_r * d),
                  (v0 + rank * hkv_r * d, v0 + (rank + 1) * hkv_r * d)]
        qkv_r = _take_rows(qkv, ranges)
        qkv_r.use_kernel = False
        full = qkv(x)
        mine = torch.cat([full[:, a:b] for a, b in ranges], dim=1)
        err_qkv = (qkv_r(x) - mine).abs().max().item()
        # gate|up -> SwiGLU -> down: column slices of both halves, matching input columns of down, one all-reduce
        f_r = ffn // world
        gu_r = _take_rows(gate_up, [(rank * f_r, (rank + 1) * f_r), (ffn + rank * f_r, ffn + (rank + 1) * f_r)])
        gu_r.use_kernel = False
        down_r = _take_cols(down, rank * f_r, (rank + 1) * f_r)
        down_r.use_kernel = False
        gu = gu_r(x)
        part = down_r(torch.nn.functional.silu(gu[:, :f_r]) * gu[:, f_r:])
        dist.all_reduce(part)
        g = gate_up(x)
        want = down(torch.nn.functional.silu(g[:, :ffn]) * g[:, ffn:])
        err_mlp = (part - want).abs().max().item() / want.abs().max().item()
        if rank == 0:
            out.put((err_qkv, err_mlp, tuple(qkv_r.packed_weight.shape), tuple(down_r.packed_weight.shape)))
    finally:
        dist.destroy_process_group()


def test_decode_stack_slices_match_unsharded():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_stack_slices_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_qkv, err_mlp, qkv_shape, down_shape = out.get(timeout=10)
    assert qkv_shape == ((4 + 1 + 1) * 128, 256) and down_shape == (512, 256)
    assert err_qkv == 0.0                             # same rows, same arithmetic
    assert err_mlp < 1e-5                             # fp32 partial sums in another order
