#!/usr/bin/env python
"""Benchmark of the quantized decode hot path (W4A16 linears + KIVI cache) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: Llama-3.1-8B-shaped decode stack (32 blocks; q/o 4096x4096, k/v 4096x1024, gate/up
4096x14336, down 14336x4096; random-init INT4 g128 with AWQ-style folded input scales), bf16
activations, one new token per step for ``--batch`` sequences over a 4-bit KIVI cache
(groups of 32 tokens, residual window 128) holding ``--context`` tokens.  A *step* is one pass
of that stack.  With N > 1 the same model is tensor-parallel over N GPUs (strong scaling).

One JSON line on stdout (rank 0): ``value`` = decode tok/s with everything resident in HBM
(CUDA-graph replay, CUDA events, max over ranks); ``e2e`` = the same metric through the
public Python API with the hidden state copied from pinned host memory and the result copied
back every step; ``roofline`` = the dominant kernel (fused gate|up dequant-GEMV) timed on its
own over 32 distinct layers' weights; ``layers`` = us/layer and fraction of the measured HBM
peak for every projection at M = 1/4/16 (plus the single 4096 x 4096 fp16 layer at M = 1);
``act_order`` = the same projections as GPTQ act-order layers (random column -> group map), fp16,
M = 1 .. 256; ``attention`` = the fused KIVI decode attention alone: the Llama-shaped cells and the
Qwen-shaped grid batch {1, 4, 16} x context {4k, 16k, 32k} at 4 and 2 bits; ``kivi_cache`` = the
cache-maintenance kernels (bulk append, dense dequantize, one reference-contract ``update()``);
``prefill_layers`` = the tensor-core path at M = 64 / 256 as a fraction of the measured dense bf16
peak; ``shape_70b`` = decode tok/s of the Llama-3-70B-shaped stack (80 blocks, 4-bit cache at 8192
tokens) at batch 1 / 8 / 32 on the N GPUs of the run; ``tp_check`` (N > 1) = a 2-block tensor-parallel
step against the unsharded model on rank 0; ``cpu_baseline`` = the reference's CPU op sequence
(oracle port) timed on the host cores on a bounded sample.  ``--impl reference`` prints only that
CPU arm.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "decode_tok_s_llama3.1-8b_w4a16_kivi4"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0
# kernels of this library launched per decode block: 4 linears (q|k|v and gate|up normalise their input
# themselves, down applies the SwiGLU gate itself) and attention (which appends the new K / V token itself)
LAUNCHES_PER_BLOCK = 5
# dram__bytes_read + dram__bytes_write of one gate|up GEMV launch (28672 x 4096, M = 1): a stored figure from an ncu
# capture of that launch, not measured by this script (the JSON line says so in roofline.traffic_source)
GATE_UP_DRAM_TRAFFIC = 66_143_000 + 577_000   # read + write, mean of two captured launches


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--shape", default="llama-3.1-8b")
    ap.add_argument("--skip-layer-table", action="store_true")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="for profiler captures: GPU work only")
    ap.add_argument("--table-batches", default="1,4,16", help="activation rows of the per-layer table")
    ap.add_argument("--skip-70b", action="store_true", help="leave out the 70B-shaped stack")
    ap.add_argument("--attn-filter", default="", help="run only the attention cells whose name contains this text (profiler captures)")
    ap.add_argument("--only", default="", help="comma list of tables to run (layers,act_order,attention,kivi_cache,prefill,70b)")
    return ap.parse_args()


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def w4a16_bytes(m: int, n: int, k: int, g: int = 128) -> int:
    """Algorithmic bytes of one W4A16 linear: nibbles + fp16 scale + fp16 zero + activations in/out."""
    return n * k // 2 + 2 * n * (k // g) * 2 + m * k * 2 + m * n * 2


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's op sequence (oracle/cpu_path.py) on the host cores
# ----------------------------------------------------------------------------------------------

def cpu_step_seconds(shape, batch: int, context: int, layers: int, steps: int, warmup: int, budget_s: float = 60.0):
    """Seconds per decode step on the CPU: the reference's op sequence (oracle/cpu_path.py) over ``n`` of the
    stack's blocks per step -- each with its own seven weight tensors (7 projections at M=batch in fp32 + one
    cache.update + fp32 SDPA at ``context`` tokens) -- scaled to the block count.  ``n`` is the whole stack when
    steps + warmup of that fit in ``budget_s`` seconds, else as many blocks as do (at least one)."""
    from oracle import cpu_path
    from pare_b200.decode import synthetic_linear

    hidden, ffn, hq, hkv, d, _ = shape
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)

    def block_weights(i):
        dims = [(hq * d, hidden), (hkv * d, hidden), (hkv * d, hidden), (hidden, hq * d), (ffn, hidden), (ffn, hidden), (hidden, ffn)]
        out = []
        for j, (n, k) in enumerate(dims):   # the GPU arm's generator (same distribution), on the CPU
            l = synthetic_linear(n, k, seed=i * 7 + j, device="cpu")
            out.append((l.packed_weight, l.scale, l.zero))
        return out

    cache = cpu_path.TorchCache(4, 32, 128)
    k = torch.randn(batch, hkv, context, d, generator=g).half()
    v = torch.randn(batch, hkv, context, d, generator=g).half()
    cache.update(k, v)
    q = torch.randn(batch, hq, 1, d, generator=g).half()
    k1, v1 = k[:, :, :1].clone(), v[:, :, :1].clone()

    def one_block(projs):
        for packed, scale, zero in projs:
            x = torch.randn(batch, packed.shape[1] * 2)
            cpu_path.linear_forward(x, packed, scale, zero)
        snap = (cache.comp, cache.rk, cache.rv)
        fk, fv = cache.update(k1, v1)
        cpu_path.attention(q, fk, fv)
        cache.comp, cache.rk, cache.rv = snap      # keep the context fixed from step to step

    first = block_weights(0)
    one_block(first)                               # warm the allocator and the thread pool
    second = block_weights(1)
    t0 = time.perf_counter()
    one_block(second)                              # a block whose weights are not in any cache yet
    t_block = time.perf_counter() - t0
    n = int(budget_s / max(1e-6, (steps + warmup) * t_block))
    n = max(1, min(layers, n))
    blocks = [first, second][:n] + [block_weights(i) for i in range(2, n)]

    def one_step():
        t0 = time.perf_counter()
        for projs in blocks:
            one_block(projs)
        return time.perf_counter() - t0

    for _ in range(warmup):
        one_step()
    times = sorted(one_step() for _ in range(steps))
    sec = times[len(times) // 2] * layers / n
    info = {"cores": cores, "kind": "port", "sampled_blocks": n, "blocks": layers,
            "sample": f"{n} of the stack's {layers} blocks per step, each with its own weights (7 projections at M={batch} in fp32 + "
                      f"cache.update + fp32 SDPA at {context} tokens)" + ("" if n == layers else ", scaled to the block count")}
    return sec, info


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from pare_b200.decode import SHAPES
    shape = SHAPES[args.shape]
    steps = args.steps or 3
    warmup = args.warmup if args.warmup is not None else 1
    sec, info = cpu_step_seconds(shape, args.batch, args.context, args.layers, steps, warmup)
    value = args.batch / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, **info},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU op sequence of the reference (oracle port on the host cores); the reference's GPU paths "
                "(eager dequantize + cuBLAS, Triton kernel) are not run: the reference package does not travel to the GPU box",
    }
    print(json.dumps(line), flush=True)


def workload_config(args, n_gpus: int) -> dict:
    return {
        "workload": f"{args.shape}-shaped decode stack, {args.layers} blocks, INT4 g128 AWQ-folded weights, bf16 activations, "
                    f"batch {args.batch}, KIVI 4-bit g32 r128 cache at {args.context} tokens",
        "batch": args.batch, "context": args.context, "layers": args.layers,
        "parallelism": f"tp{n_gpus}" if n_gpus > 1 else "single",
        "l2": "inputs larger than L2 (every step streams all layers' weights and cache once)",
    }


# ----------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(index)],
                stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.tmp.flush()
        rows = [r.split(",") for r in Path(self.tmp.name).read_text().strip().splitlines() if r.count(",") >= 5]
        os.unlink(self.tmp.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(r[2 + j].strip() == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows)}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------

def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL's log goes to stderr (stdout carries one JSON line only); whatever level the caller asked for is kept
        os.environ.setdefault("NCCL_DEBUG", "WARN")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world: int) -> None:
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(seconds: float, world: int) -> float:
    if world == 1:
        return seconds
    t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def capture(fn, warm: int = 2):
    """Run ``fn`` eagerly ``warm`` times on a side stream, then capture it into a CUDA graph."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    torch.cuda.synchronize()
    return g, out


def time_events(fn, steps: int, warmup: int, world: int) -> float:
    for _ in range(warmup):
        fn()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1) * 1e-3, world)


def layer_table(stack, peak: float, batches=(1, 4, 16)) -> dict:
    """us/layer and fraction of the HBM peak for each fused projection of the stack, timed alone:
    one CUDA graph of n_layers launches over the n_layers DISTINCT weight sets (hundreds of MB, so
    nothing is served from L2), average duration per launch from CUDA events.  ``us_per_layer`` is the
    public ``QuantizedLinear.forward`` (activation preparation launch + streaming kernel); ``us_kernel``
    the streaming kernel alone on prepared activations, which is what runs inside the decode stack
    (there the producer of the activation writes them prepared)."""
    from pare_b200.kernels.matmul_int4 import prepare

    table = {}
    kinds = {"qkv": lambda b: b.qkv, "o": lambda b: b.o, "gate_up": lambda b: b.gate_up, "down": lambda b: b.down}
    for name, pick in kinds.items():
        layers = [pick(b) for b in stack.blocks]
        n, k = layers[0].out_features, layers[0].in_features
        for m in batches:
            x = torch.randn(m, k, device=stack.device, dtype=stack.dtype)
            prep = prepare(x) if layers[0].supports_prepared(m) else None

            def run_public():
                for layer in layers:
                    layer(x)

            def run_kernel():
                for layer in layers:
                    layer.forward_prepared(prep)

            entry = {}
            for key, fn in (("us_per_layer", run_public), ("us_kernel", run_kernel if prep is not None else None)):
                if fn is None:
                    continue
                g, _ = capture(fn)
                reps = 20
                sec = time_events(g.replay, reps, 3, 1)
                entry[key] = round(sec / (reps * len(layers)) * 1e6, 3)
                del g
            us = entry.get("us_kernel", entry["us_per_layer"])
            gbs = w4a16_bytes(m, n, k) / us / 1e3
            entry.update({"gbs": round(gbs, 1), "frac_hbm": round(gbs / peak, 4)})
            table[f"{name}_{n}x{k}_m{m}"] = entry
    return table


def time_graph(fn, reps: int = 20) -> float:
    """Seconds per call of ``fn`` from a replayed CUDA graph (CUDA events, 3 warm-up replays)."""
    g, _ = capture(fn)
    sec = time_events(g.replay, reps, 3, 1) / reps
    del g
    return sec


def single_layer_fp16(peak: float, device) -> dict:
    """The single-layer configuration: one 4096 x 4096 RTN INT4 g128 layer (weights N(0, 0.02), built by
    ``QuantizedLinear.from_linear`` as the reference's kernel benchmark does), fp16 activations N(0, 1), M = 1; 64
    copies of the layer's tensors (0.6 GB) so that nothing is served from L2."""
    import torch.nn as nn
    from pare_b200.config import QuantConfig
    from pare_b200.layers.linear import QuantizedLinear

    torch.manual_seed(0)
    lin = nn.Linear(4096, 4096, bias=False)
    lin.weight.data.normal_(0, 0.02)
    base = QuantizedLinear.from_linear(lin, QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128))
    layers = []
    for _ in range(64):
        l = QuantizedLinear.from_tensors(base.packed_weight.clone().to(device), None, base.scale.clone().to(device),
                                         base.zero.clone().to(device), base.config, None, 4096, 4096)
        l.use_kernel = True
        layers.append(l)
    torch.manual_seed(1)
    x = torch.randn(1, 4096, device=device, dtype=torch.float16)

    def run():
        for l in layers:
            l(x)
    us = time_graph(run) / len(layers) * 1e6
    gbs = w4a16_bytes(1, 4096, 4096) / us / 1e3
    return {"us_per_layer": round(us, 3), "gbs": round(gbs, 1), "frac_hbm": round(gbs / peak, 4), "dtype": "f16",
            "note": "public forward: activation preparation launch + streaming kernel"}


def act_order_table(peak: float, tf_peak: float, device, batches=(1, 4, 16, 64, 128, 256)) -> dict:
    """GPTQ act-order layers (a seeded random permutation of the input channels mapped to groups; scales per g_idx
    group) on the 8B-shaped projections, fp16 activations N(0, 1): us per layer over 8 distinct layers, fraction of the
    HBM peak up to 16 rows and of the dense bf16 peak above (the tensor-core kernel)."""
    from pare_b200.config import QuantConfig
    from pare_b200.layers.linear import QuantizedLinear

    def make(n, k, seed):
        g = torch.Generator(device=device).manual_seed(seed)
        perm = torch.randperm(k, device=device, generator=g)
        g_idx = torch.empty(k, dtype=torch.int32, device=device)
        g_idx[perm] = (torch.arange(k, device=device) // 128).to(torch.int32)
        packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=g)
        scale = (0.02 / 4.61) * (0.75 + 0.5 * torch.rand(n, k // 128, 1, device=device, generator=g))
        zero = torch.randint(6, 11, (n, k // 128, 1), device=device, generator=g).float()
        l = QuantizedLinear.from_tensors(packed, None, scale, zero, QuantConfig(bits=4, scheme="gptq", group_size=128, act_order=True),
                                         None, k, n, g_idx=g_idx)
        l.use_kernel = True
        return l

    table = {}
    for name, (n, k) in {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}.items():
        layers = [make(n, k, 100 + i) for i in range(8)]
        for m in batches:
            x = torch.randn(m, k, device=device, dtype=torch.float16)

            def run():
                for l in layers:
                    l(x)
            us = time_graph(run, reps=10) / len(layers) * 1e6
            entry = {"us_per_layer": round(us, 2)}
            if m <= 16:
                entry["frac_hbm"] = round((w4a16_bytes(m, n, k) + 4 * k) / us / 1e3 / peak, 4)
            else:
                entry["frac_tensor"] = round(2.0 * m * n * k / us / 1e6 / tf_peak, 4)
            table[f"{name}_{n}x{k}_m{m}"] = entry
        del layers
    return table


def prefill_table(stack, batches=(64, 256)) -> dict:
    """Tensor-core path (tcgen05 tiles over dequantized operands, M > 16): us per layer, TFLOP/s and the fraction of
    the measured dense bf16 peak (burst figure: each projection is timed alone)."""
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))
    table = {}
    kinds = {"qkv": lambda b: b.qkv, "o": lambda b: b.o, "gate_up": lambda b: b.gate_up, "down": lambda b: b.down}
    for name, pick in kinds.items():
        layers = [pick(b) for b in stack.blocks][:8]
        n, k = layers[0].out_features, layers[0].in_features
        for m in batches:
            x = torch.randn(m, k, device=stack.device, dtype=stack.dtype)

            def run():
                for layer in layers:
                    layer(x)
            g, _ = capture(run)
            reps = 10
            sec = time_events(g.replay, reps, 3, 1)
            us = sec / (reps * len(layers)) * 1e6
            tf = 2.0 * m * n * k / us / 1e6
            table[f"{name}_{n}x{k}_m{m}"] = {"us_per_layer": round(us, 2), "tflops": round(tf, 1), "frac_tensor": round(tf / tf_peak, 4)}
            del g
    return table


def prefill_attention_table(dtype, device, lengths=(2048, 8192)) -> dict:
    """Causal prefill attention over full-precision K / V (32 query / 8 KV heads, D = 128, batch 1): ms per call,
    TFLOP/s by the 2 T^2 D Hq flops of the causal half, and the fraction of the measured dense bf16 peak (a
    warp-level mma.sync kernel: the tensor-core generation before tcgen05, so the fraction is modest by construction)."""
    from pare_b200.kv_cache import prefill_attention

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))
    table = {}
    for t in lengths:
        q = torch.randn(1, 32, t, 128, device=device).to(dtype)
        k = torch.randn(1, 8, t, 128, device=device).to(dtype)
        v = torch.randn(1, 8, t, 128, device=device).to(dtype)
        sec = time_events(lambda: prefill_attention(q, k, v), 10, 3, 1) / 10
        tf = 2.0 * t * t * 128 * 32 / sec / 1e12
        table[f"t{t}"] = {"ms": round(sec * 1e3, 3), "tflops": round(tf, 1), "frac_tensor": round(tf / tf_peak, 4)}
    return table


def prompt_table(args, dtype, device, lengths=(512, 2048)) -> dict:
    """The whole prompt path of the stack (``DecodeStack.prefill``: RMSNorm, tensor-core linears, rotary embedding,
    causal attention at full precision, cache append with compression, SwiGLU) on a fresh stack of 4 blocks:
    ms per block and prompt tokens/s extrapolated to the stack's block count."""
    from pare_b200.decode import SHAPES, DecodeStack

    n_blocks = 4
    total_blocks = args.layers or SHAPES[args.shape][5]
    stack = DecodeStack(args.shape, device=device, dtype=dtype, n_layers=n_blocks, max_seq_len=max(lengths) + 256)
    table = {}
    for t in lengths:
        x = torch.randn(1, t, stack.hidden, device=device).to(dtype)

        def run():
            stack.cache.reset()
            stack.prefill(x)

        sec = time_events(run, 5, 2, 1) / 5
        table[f"t{t}"] = {"ms_per_block": round(sec / n_blocks * 1e3, 3),
                          "tok_s": round(t / (sec / n_blocks * total_blocks), 1)}
    del stack
    return table


def attention_table(dtype, device, peak: float, cases, name_filter: str = "") -> dict:
    """Fused KIVI decode attention alone (D = 128, g32, residual window 128): one CUDA graph over ``layers`` distinct
    caches (at least 0.5 GB together, so nothing is served from L2), us per call and fraction of the HBM peak by the
    bytes the call must read (168 B per compressed token and KV head at 4 bits, 104 B at 2 bits, 512 B per window
    token; with values in 32-channel groups 24 B more per compressed token).  A case is
    (batch, context, query heads, KV heads, bits[, value group])."""
    from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache

    table = {}
    for case in cases:
        batch, ctx, hq, hkv, bits = case[:5]
        v_group = case[5] if len(case) > 5 else None
        key = f"b{batch}_ctx{ctx}_{hq}q{hkv}kv_{bits}bit" + (f"_vg{v_group}" if v_group else "")
        if name_filter and name_filter not in key:
            continue
        per_token = (168 if bits == 4 else 104) + (24 if v_group else 0)
        layer_bytes = batch * hkv * ctx * per_token
        layers = max(2, min(192, -(-(512 << 20) // layer_bytes)))
        cache = QuantizedKVCache(layers, KVCacheConfig(bits=bits, group_size=32, residual_length=128, v_group_size=v_group),
                                 max_seq_len=ctx + 256)
        g = torch.Generator(device=device).manual_seed(0)
        n0 = 128 + ((ctx - 128) // 32) * 32
        k = torch.randn(batch, hkv, n0, 128, device=device, generator=g)
        v = torch.randn(batch, hkv, n0, 128, device=device, generator=g)
        out_ch = torch.randperm(128, device=device, generator=g)[:1]
        k[..., out_ch] *= 10.0                                  # 1 % outlier channels
        k, v = k.to(dtype), v.to(dtype)
        for layer in range(layers):                             # distinct buffers; their contents may repeat
            cache._append(layer, k, v)
        del k, v
        q = torch.randn(batch, hq, 1, 128, device=device).to(dtype)
        k1 = torch.randn(batch, hkv, 1, 128, device=device).to(dtype)
        v1 = torch.randn(batch, hkv, 1, 128, device=device).to(dtype)

        def run():
            for layer in range(layers):
                cache.attend(layer, q, k1, v1)
                cache._stores[layer].r_len -= 1   # the same step again: the token lands in the same window slot

        us = time_graph(run, reps=10 if layer_bytes > (64 << 20) else 20) / layers * 1e6
        st = cache._stores[0]
        nbytes = batch * hkv * (st.n_comp * per_token + (st.r_len + 1) * 512) + batch * hq * 128 * 4
        table[key] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peak, 4),
                      "bytes": nbytes, "caches": layers}
        del cache
        torch.cuda.empty_cache()
    return table


def attention_cases():
    cases = [(1, 4096, 32, 8, 4), (16, 4096, 32, 8, 4), (16, 4096, 32, 8, 2), (16, 4096, 32, 8, 4, 32)]     # Llama-shaped
    for bits in (4, 2):                                                                                    # Qwen-shaped grid
        for batch in (1, 4, 16):
            for ctx in (4096, 16384, 32768):
                cases.append((batch, ctx, 28, 4, bits))
    return cases


def kivi_cache_table(dtype, device, peak: float) -> dict:
    """Cache-maintenance kernels (Qwen-shaped: 4 KV heads, D = 128, 4 bits, g32): bulk quantize-on-append of 4096 and
    32768 tokens at batch 1 and 16 (reads 2 n D 2 B of keys and values, writes 168 B per token and head), dense
    dequantize of the same (reads 168 B, writes 2 D 2 B per token and head), and one reference-contract ``update()``
    decode step at 4096 tokens (append of one token + dense reconstruction of the whole cache, the work the
    reference's ``update`` does every step, pare/kv_cache.py:205-252)."""
    from pare_b200.kernels import _lib
    from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache, _LayerStore

    table = {}
    L = _lib.lib()
    for batch, n in ((1, 4096), (16, 4096), (1, 32768), (16, 32768)):
        k = torch.randn(batch, 4, n, 128, device=device).to(dtype)
        v = torch.randn(batch, 4, n, 128, device=device).to(dtype)
        stores = [_LayerStore(batch, 4, 128, KVCacheConfig(4, 32, 0), n, device, dtype) for _ in range(2)]
        outs = [(torch.empty_like(k), torch.empty_like(v)) for _ in range(2)]
        code = _lib.dtype_code(dtype)

        def append():
            for st in stores:
                _lib.check(L.pare_kivi_append(k.data_ptr(), v.data_ptr(), code, k.stride(0), k.stride(1), k.stride(2), n, 0,
                                              *st.cache_args(), *st.geometry(), _lib.current_stream(device)), "append")

        def dequant():
            for st, (ok_, ov_) in zip(stores, outs):
                _lib.check(L.pare_kivi_dequant(*st.cache_args(), *st.geometry(), n, ok_.data_ptr(), ov_.data_ptr(), code,
                                               ok_.stride(0), ok_.stride(1), ok_.stride(2), _lib.current_stream(device)), "dequant")

        nbytes = batch * 4 * n * (2 * 128 * 2 + 168)
        for name, fn in (("append", append), ("dequant", dequant)):
            us = time_graph(fn, reps=5) / len(stores) * 1e6
            table[f"{name}_b{batch}_n{n}"] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peak, 4)}
        del stores, outs, k, v
    # reference-contract decode step: update() returns the dense K / V of the whole sequence
    cache = QuantizedKVCache(1, KVCacheConfig(4, 32, 128), max_seq_len=4096 + 256)
    k = torch.randn(1, 4, 4095, 128, device=device).to(dtype)
    cache._append(0, k, k)
    k1 = torch.randn(1, 4, 1, 128, device=device).to(dtype)

    def step():
        cache.update(0, k1, k1)
        cache._stores[0].r_len -= 1
    sec = time_events(step, 20, 3, 1) / 20
    table["update_step_b1_ctx4096"] = {"us": round(sec * 1e6, 1), "note": "append of one token + dense dequantize of 3968 tokens + window copy, eager"}
    return table


def stack_70b(args, world: int, local: int, peak: float, batches=(1, 8, 32)) -> dict:
    """Llama-3-70B-shaped stack (hidden 8192, FFN 28672, 64 query / 8 KV heads, 80 blocks, INT4 g128, 4-bit cache at
    8192 tokens), tensor-parallel over the run's GPUs: decode tok/s, ms per step and the step's fraction of the HBM
    time of the bytes each GPU must move, at batch 1 / 8 / 32."""
    from pare_b200.decode import SHAPES, DecodeStack

    shape = "llama-3-70b"
    hidden, ffn, hq, hkv, d, layers = SHAPES[shape]
    ctx = 8192
    stack = DecodeStack(shape, device=f"cuda:{local}", dtype=torch.bfloat16, max_seq_len=ctx + 256, tp_world=world)
    blk = stack.blocks[0]
    out = {}
    for batch in batches:
        stack.cache.reset()
        torch.cuda.empty_cache()
        stack.prefill_cache(batch, ctx)
        x = torch.randn(batch, hidden, device=stack.device).to(torch.bfloat16)
        barrier(world)
        graph, _ = capture(lambda: stack(x))
        steps = 10
        sec = time_events(graph.replay, steps, 3, world) / steps
        lin_bytes = sum(w4a16_bytes(batch, l.out_features, l.in_features) for l in (blk.qkv, blk.o, blk.gate_up, blk.down))
        kv_bytes = batch * blk.hkv * ((ctx - 128) * 168 + 128 * 512) + batch * blk.hq * 128 * 4
        step_bytes = layers * (lin_bytes + kv_bytes)
        out[f"b{batch}"] = {"tok_s": round(batch / sec, 1), "ms_per_step": round(sec * 1e3, 3),
                            "step_bytes_per_gpu": step_bytes, "step_frac_hbm": round(step_bytes / sec / 1e9 / peak, 4)}
        del graph
    del stack
    torch.cuda.empty_cache()
    return out


def tp_check(args, world: int, rank: int, local: int) -> dict | None:
    """A 2-block tensor-parallel decode step against the same 2 blocks unsharded on rank 0 (same seeds, hence the same
    model and cache contents): max / mean relative error of the hidden state (the shared metric of the tests)."""
    from pare_b200.decode import DecodeStack

    dev = f"cuda:{local}"
    tp = DecodeStack(args.shape, device=dev, dtype=torch.bfloat16, n_layers=2, max_seq_len=1024, tp_world=world)
    tp.prefill_cache(2, 512 + 128)
    x = torch.randn(2, tp.hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    barrier(world)
    y = tp(x)
    torch.cuda.synchronize()
    res = None
    if rank == 0:
        one = DecodeStack(args.shape, device=dev, dtype=torch.bfloat16, n_layers=2, max_seq_len=1024, tp_world=1, tp_rank=0)
        one.prefill_cache(2, 512 + 128)
        ref = one(x).float()
        e = (y.float() - ref).abs() / torch.maximum(ref.abs(), 1e-2 * ref.abs().max())
        res = {"max_rel": round(float(e.max()), 5), "mean_rel": round(float(e.mean()), 6), "blocks": 2, "batch": 2,
               "bars": "max <= 1e-1, mean <= 1.2e-2 (bf16 hand-overs; the ranks' partial sums are added in fp32 inside the row-parallel GEMV epilogues, so most elements round to the same bf16 value as the unsharded stack)"}
        del one
    status = tp.peer_reduce.status(tp.device) if tp.peer_reduce is not None else 0
    if res is not None:
        res["peer_status"] = int(status)
    if tp.peer_reduce is not None:
        barrier(world)
        tp.peer_reduce.close()
    del tp
    torch.cuda.empty_cache()
    return res


def run_ours(args) -> None:
    from pare_b200.decode import SHAPES, DecodeStack
    from pare_b200.kernels import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation of the product path)")
    _lib.lib()  # fail loudly if the CUDA library is missing
    world, rank, local = dist_setup(args.gpus)
    steps = args.steps or 200   # ~0.4 s timed: enough for several clock samples
    warmup = args.warmup if args.warmup is not None else 5
    peak, peak_kind = measured_peak()
    dtype = torch.bfloat16

    stack = DecodeStack(args.shape, device=f"cuda:{local}", dtype=dtype, n_layers=args.layers,
                        max_seq_len=args.context + 256, tp_world=world)
    # context chosen so that the residual window sits at its minimum: no compression during warm-up
    ctx = 128 + ((args.context - 128) // 32) * 32
    stack.prefill_cache(args.batch, ctx)
    hidden = stack.hidden
    x_host = torch.randn(args.batch, hidden).to(dtype).pin_memory()
    y_host = torch.empty(args.batch, hidden, dtype=dtype).pin_memory()
    x_dev = x_host.cuda(non_blocking=True)

    barrier(world)   # every rank has built its shard before the first step touches a peer
    graph, y_dev = capture(lambda: stack(x_dev))

    sampler = ClockSampler(local) if rank == 0 else None
    sec = time_events(graph.replay, steps, max(warmup, 3), world)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(y_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    sec_e2e = time_events(e2e_step, steps, max(warmup, 3), world)
    clocks = sampler.stop() if sampler else None
    check = tp_check(args, world, rank, local) if world > 1 else None

    tok_s = args.batch * steps / sec
    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": max(warmup, 3),
        "ms_per_step": sec / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
        "e2e": {"value": args.batch * steps / sec_e2e, "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        # under tensor parallelism the sums over the ranks are added inside the o and down kernels: still 5 launches a block
        "gpu_launches": (LAUNCHES_PER_BLOCK + (0 if world == 1 or (stack.peer_reduce is not None and
                         args.batch * hidden <= stack.peer_reduce.max_fused_elements()) else 2)) * args.layers * steps,
        "clocks": clocks,
    }
    # bytes one step must move: all linears (algorithmic) + the cache
    blk = stack.blocks[0]
    lin_bytes = sum(w4a16_bytes(args.batch, l.out_features, l.in_features) for l in (blk.qkv, blk.o, blk.gate_up, blk.down))
    n_comp = ctx - 128
    kv_bytes = args.batch * blk.hkv * (n_comp * 168 + 128 * 512) + args.batch * blk.hq * 128 * 4
    step_bytes = args.layers * (lin_bytes + kv_bytes)
    line["step_bytes_per_gpu"] = step_bytes
    line["step_frac_hbm"] = round(step_bytes / (sec / steps) / 1e9 / peak, 4)

    only = set(t for t in args.only.split(",") if t)
    want = lambda name: (not args.skip_layer_table) and (not only or name in only)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))
    if world == 1:
        table = layer_table(stack, peak, tuple(int(b) for b in args.table_batches.split(","))) if want("layers") else {}
        if want("layers"):
            table["single_4096x4096_f16_m1"] = single_layer_fp16(peak, stack.device)
        line["layers"] = table
        line["prefill_layers"] = prefill_table(stack) if want("prefill") else {}
        key = f"gate_up_{blk.gate_up.out_features}x{blk.gate_up.in_features}_m{args.batch}"
        if key in table:
            achieved = table[key]["gbs"]
            line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                                "frac": round(achieved / peak, 4),
                                "traffic": GATE_UP_DRAM_TRAFFIC if (args.shape, args.batch) == ("llama-3.1-8b", 1) else None,
                                "traffic_source": "ncu capture, stored", "peak_source": peak_kind,
                                "kernel": "w4a16_gemv_persist_kernel (fused gate|up projection)",
                                "bytes_per_launch": w4a16_bytes(args.batch, blk.gate_up.out_features, blk.gate_up.in_features)}
    del graph, stack
    torch.cuda.empty_cache()
    if world == 1:
        line["act_order"] = act_order_table(peak, tf_peak, f"cuda:{local}") if want("act_order") else {}
        line["attention"] = attention_table(dtype, torch.device(f"cuda:{local}"), peak, attention_cases(), args.attn_filter) if want("attention") else {}
        line["kivi_cache"] = kivi_cache_table(dtype, torch.device(f"cuda:{local}"), peak) if want("kivi_cache") else {}
        line["prefill_attention"] = prefill_attention_table(dtype, torch.device(f"cuda:{local}")) if want("prefill") else {}
        line["prompt"] = prompt_table(args, dtype, torch.device(f"cuda:{local}")) if want("prefill") else {}
    if not args.skip_70b and (not only or "70b" in only):
        res70 = stack_70b(args, world, local, peak)
        if rank == 0:
            line["shape_70b"] = res70
    if rank != 0:
        return
    if check is not None:
        line["tp_check"] = check
    if world == 1:
        try:
            if args.skip_cpu_baseline:
                raise RuntimeError("skipped by --skip-cpu-baseline")
            csec, info = cpu_step_seconds(SHAPES[args.shape], args.batch, args.context, args.layers, 1, 0, budget_s=20.0)
            line["cpu_baseline"] = {"value": args.batch / csec, "unit": UNIT, **info}
        except Exception as exc:  # the CPU arm must never hide the GPU result
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "error": repr(exc)}
    print(json.dumps(line), flush=True)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
