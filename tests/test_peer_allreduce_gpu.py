"""One-shot peer all-reduce (GPU, needs two devices; skipped on a single-GPU box).

Two child processes, one per GPU, NCCL only for the handle exchange.  Checks: the sum equals the fp32
sum of the ranks' inputs rounded once to the tensor dtype (bit-exact: rank-order fp32 addition), identical
on both ranks, over many back-to-back calls (double-buffered slots), over a queue of calls of different shapes
with no host synchronisation between them while one rank launches late, eagerly and from a replayed CUDA
graph, and the status word stays clean.
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
