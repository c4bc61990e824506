"""One-shot peer all-reduce (GPU, needs two devices; skipped on a single-GPU box).

Two child processes, one per GPU, NCCL only for the handle exchange.  Checks: the sum equals the fp32
sum of the ranks' inputs rounded once to the tensor dtype (bit-exact: rank-order fp32 addition), identical
on both ranks, over many back-to-back calls (double-buffered slots), over a queue of calls of different shapes
with no host synchronisation between them while one rank launches late, eagerly and from a replayed CUDA
graph, and the status word stays clean.  Then the same sum added INSIDE the row-parallel linears (tile and
persistent streaming kernels, prepared and SwiGLU-producing forwards) against the unsharded layer, identical
bits on both ranks, and a 2-block tensor-parallel decode stack against the unsharded stack.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["PARE_ROOT"])
import torch, torch.distributed as dist
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
os.environ["NCCL_NVLS_ENABLE"] = "0"
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from pare_b200.parallel import PeerAllReduce
ar = PeerAllReduce()
ok = True
for dtype in (torch.float16, torch.bfloat16):
    for rows, cols in ((1, 4096), (4, 8192), (16, 4096), (3, 1024)):
        for it in range(5):
            g = torch.Generator(device="cuda").manual_seed(1000 * it + rows)
            parts = [torch.randn(rows, cols, device="cuda", generator=g).to(dtype) for _ in range(world)]   # same on every rank
            y = ar(parts[rank])
            ref = sum(p.float() for p in parts).to(dtype)
            ok &= bool(torch.equal(y, ref))
# calls of different shapes queued back to back with no host synchronisation in between, one rank launching late:
# a unit changes its owning CTA from call to call, every result must still be the exact sum
import time
seq = [(1, 2048), (1, 2048), (1, 2048), (1, 2400), (1, 2400), (16, 4096), (1, 2048), (3, 1024), (1, 2400)] * 3
g = torch.Generator(device="cuda").manual_seed(7)
ins = [[torch.randn(r, c, device="cuda", generator=g).half() for _ in range(world)] for r, c in seq]
torch.cuda.synchronize(); dist.barrier()
if rank == 1:
    time.sleep(0.3)
outs = [ar(parts[rank]) for parts in ins]
torch.cuda.synchronize()
for parts, y in zip(ins, outs):
    ok &= bool(torch.equal(y, sum(p.float() for p in parts).half()))
ok &= ar.status(torch.device("cuda", rank)) == 0
# replayed graph: 20 replays of two chained all-reduces
x = torch.randn(2, 4096, device="cuda").half() * (rank + 1)
s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(s):
    ar(ar(x))
torch.cuda.current_stream().wait_stream(s); torch.cuda.synchronize()
gr = torch.cuda.CUDAGraph()
with torch.cuda.graph(gr):
    out = ar(ar(x))
for _ in range(20):
    gr.replay()
torch.cuda.synchronize()
xs = [torch.empty_like(x) for _ in range(world)]
dist.all_gather(xs, x)
once = sum(t.float() for t in xs).half()
ok &= bool(torch.equal(out, (once.float() * world).half()))
ok &= ar.status(x.device) == 0
# ---- the sum over the ranks added INSIDE the row-parallel linears (no all-reduce launch) ----
from pare_b200.decode import synthetic_linear, _take_cols, DecodeStack
from pare_b200.kernels.matmul_int4 import prepare
import numpy as np
def rel(y, ref):
    ref = ref.float(); e = (y.float() - ref).abs() / torch.maximum(ref.abs(), 1e-2 * ref.abs().max())
    return float(e.max()), float(e.mean())
for (n, k), ms in (((4096, 4096), (1, 4)), ((4096, 14336), (1, 3)), ((1024, 2048), (2,))):   # tile kernel, persistent kernel (K slices), small
    full = synthetic_linear(n, k, seed=n + k, device="cuda")
    shard = _take_cols(full, rank * k // world, (rank + 1) * k // world)
    for m in ms:
        g = torch.Generator(device="cuda").manual_seed(m)
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        xs = x[:, rank * k // world:(rank + 1) * k // world].contiguous()
        ys = [shard.forward_prepared(prepare(xs), peer=ar) for _ in range(4)]        # back to back, no host sync
        gu = torch.randn(m, 2 * k, device="cuda", generator=g).to(torch.bfloat16)    # SwiGLU producer + exchange
        kk = k // world
        gus = torch.cat([gu[:, rank * kk:(rank + 1) * kk], gu[:, k + rank * kk:k + (rank + 1) * kk]], dim=1).contiguous()
        y2 = shard.forward_silu_mul(gus, peer=ar)
        torch.cuda.synchronize()
        ref = full(x)
        mx, mean = rel(ys[0], ref)
        ok &= mx <= 1e-2 and mean <= 2.5e-3
        ok &= all(bool(torch.equal(ys[0], y)) for y in ys[1:])
        act = (torch.nn.functional.silu(gu[:, :k].float()) * gu[:, k:].float()).to(torch.bfloat16)
        mx, mean = rel(y2, full(act))
        ok &= mx <= 1e-2 and mean <= 2.5e-3
        both = [torch.empty_like(ys[0]) for _ in range(world)]
        dist.all_gather(both, ys[0])
        ok &= all(bool(torch.equal(both[0], b)) for b in both)                        # identical bits on every rank
ok &= ar.status(torch.device("cuda", rank)) == 0
# a 2-block tensor-parallel decode step (5 launches per block) against the unsharded stack on the same GPU
shape = (1024, 2048, 8, 2, 128, 2)
tp = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3, tp_world=world)
tp.prefill_cache(2, 224)
xh = torch.randn(2, 1024, generator=torch.Generator().manual_seed(5)).half().cuda()
for _ in range(3):
    yt = tp(xh)
one = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3, tp_world=1, tp_rank=0)
one.prefill_cache(2, 224)
for _ in range(3):
    yo = one(xh)
mx, mean = rel(yt, yo)
print("tp stack vs unsharded", rank, mx, mean, flush=True)
ok &= mx <= 3e-2 and mean <= 3e-3
ok &= tp.peer_reduce.status(torch.device("cuda", rank)) == 0
dist.barrier(); tp.peer_reduce.close()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
ar.close()
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 1)
"""


def test_peer_allreduce_two_ranks(cuda_lib, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, PARE_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r))) for r in range(2)]
    codes = [p.wait(timeout=300) for p in procs]
    assert codes == [0, 0], codes
