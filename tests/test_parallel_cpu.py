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
