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
peak for every projection at M = 1/4/16; ``attention`` = the fused KIVI decode attention alone at
batch 1 and batch 16; ``prefill_layers`` = the tensor-core path at M = 64 / 256 as a fraction of the
measured dense bf16 peak; ``cpu_baseline`` = the reference's CPU op sequence
(oracle port) timed on the host cores on a bounded sample.  ``--impl reference`` prints only
that CPU arm.
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
# dram__bytes_read + dram__bytes_write of one gate|up GEMV launch (28672 x 4096, M = 1) from the ncu capture
# summarised in profiles/w4a16_gemv_persist_gate_up_m1.md
GATE_UP_DRAM_TRAFFIC = 66_100_000 + 540_000


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

def cpu_block_seconds(shape, batch: int, context: int, steps: int, warmup: int) -> tuple[float, dict]:
    """Median seconds for ONE decode block on the CPU (7 projections at M=batch in fp32 + one
    cache.update + SDPA at ``context`` tokens).  tok/s of the full stack = batch / (layers * that)."""
    from oracle import cpu_path

    hidden, ffn, hq, hkv, d, _ = shape
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)

    def layer(n, k):
        packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
        scale = torch.rand(n, k // 128, 1, generator=g) * 0.004 + 0.002
        zero = torch.randint(6, 11, (n, k // 128, 1), generator=g).float()
        return packed, scale, zero

    projs = [layer(hq * d, hidden), layer(hkv * d, hidden), layer(hkv * d, hidden), layer(hidden, hq * d),
             layer(ffn, hidden), layer(ffn, hidden), layer(hidden, ffn)]
    cache = cpu_path.TorchCache(4, 32, 128)
    k = torch.randn(batch, hkv, context, d, generator=g).half()
    v = torch.randn(batch, hkv, context, d, generator=g).half()
    cache.update(k, v)
    q = torch.randn(batch, hq, 1, d, generator=g).half()
    k1, v1 = k[:, :, :1].clone(), v[:, :, :1].clone()

    def one_block():
        t0 = time.perf_counter()
        for packed, scale, zero in projs:
            x = torch.randn(batch, packed.shape[1] * 2)
            cpu_path.linear_forward(x, packed, scale, zero)
        snap = (cache.comp, cache.rk, cache.rv)
        fk, fv = cache.update(k1, v1)
        cpu_path.attention(q, fk, fv)
        cache.comp, cache.rk, cache.rv = snap      # keep the context fixed from step to step
        return time.perf_counter() - t0

    for _ in range(warmup):
        one_block()
    times = sorted(one_block() for _ in range(steps))
    info = {"cores": cores, "kind": "port",
            "sample": f"1 of the stack's blocks per step (7 projections at M={batch} in fp32 + cache.update + fp32 SDPA "
                      f"at {context} tokens), scaled by the block count"}
    return times[len(times) // 2], info


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from pare_b200.decode import SHAPES
    shape = SHAPES[args.shape]
    steps = args.steps or 3
    warmup = args.warmup if args.warmup is not None else 1
    sec, info = cpu_block_seconds(shape, args.batch, args.context, steps, warmup)
    value = args.batch / (sec * args.layers)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * args.layers * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, **info},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
        # keep NCCL's version banner off stdout (one JSON line only): warnings only, and into a file
        os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", os.path.join(tempfile.gettempdir(), "nccl_%h_%p.log"))
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


def attention_table(dtype, device, peak: float,
                    cases=((1, 4096, 32, 4), (16, 4096, 8, 4), (16, 4096, 8, 2), (16, 4096, 8, 4, 32))) -> dict:
    """Fused KIVI decode attention alone (8 KV heads, 32 query heads, D = 128, g32, residual window 128):
    one CUDA graph over ``layers`` distinct caches (larger than L2 together), us per call and fraction of the HBM
    peak by the bytes the call must read (168 B per compressed token and KV head at 4 bits, 104 B at 2 bits,
    512 B per window token; with values in 32-channel groups -- a fifth element 32 in the case -- 24 B more per
    compressed token)."""
    from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache

    table = {}
    for case in cases:
        batch, ctx, layers, bits = case[:4]
        v_group = case[4] if len(case) > 4 else None
        cache = QuantizedKVCache(layers, KVCacheConfig(bits=bits, group_size=32, residual_length=128, v_group_size=v_group),
                                 max_seq_len=ctx + 256)
        g = torch.Generator(device=device).manual_seed(0)
        n0 = 128 + ((ctx - 128) // 32) * 32
        for layer in range(layers):
            k = torch.randn(batch, 8, n0, 128, device=device, generator=g).to(dtype)
            v = torch.randn(batch, 8, n0, 128, device=device, generator=g).to(dtype)
            cache._append(layer, k, v)
        q = torch.randn(batch, 32, 1, 128, device=device).to(dtype)
        k1 = torch.randn(batch, 8, 1, 128, device=device).to(dtype)
        v1 = torch.randn(batch, 8, 1, 128, device=device).to(dtype)

        def run():
            for layer in range(layers):
                cache.attend(layer, q, k1, v1)
                cache._stores[layer].r_len -= 1   # the same step again: the token lands in the same window slot

        gr, _ = capture(run)
        reps = 20
        sec = time_events(gr.replay, reps, 3, 1)
        us = sec / (reps * layers) * 1e6
        st = cache._stores[0]
        per_token = (168 if bits == 4 else 104) + (24 if v_group else 0)
        nbytes = batch * 8 * (st.n_comp * per_token + (st.r_len + 1) * 512) + batch * 32 * 128 * 4
        table[f"b{batch}_ctx{ctx}_{bits}bit" + (f"_vg{v_group}" if v_group else "")] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peak, 4)}
        del gr, cache
    return table


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

    if rank != 0:
        return
    tok_s = args.batch * steps / sec
    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": max(warmup, 3),
        "ms_per_step": sec / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
        "e2e": {"value": args.batch * steps / sec_e2e, "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": (LAUNCHES_PER_BLOCK + (2 if world > 1 and stack.peer_reduce is not None else 0)) * args.layers * steps,
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

    if world == 1:
        table = {} if args.skip_layer_table else layer_table(stack, peak, tuple(int(b) for b in args.table_batches.split(",")))
        line["layers"] = table
        line["attention"] = {} if args.skip_layer_table else attention_table(dtype, stack.device, peak)
        line["prefill_layers"] = {} if args.skip_layer_table else prefill_table(stack)
        line["prefill_attention"] = {} if args.skip_layer_table else prefill_attention_table(dtype, stack.device)
        line["prompt"] = {} if args.skip_layer_table else prompt_table(args, dtype, stack.device)
        key = f"gate_up_{blk.gate_up.out_features}x{blk.gate_up.in_features}_m{args.batch}"
        if key in table:
            achieved = table[key]["gbs"]
            line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                                "frac": round(achieved / peak, 4),
                                "traffic": GATE_UP_DRAM_TRAFFIC if (args.shape, args.batch) == ("llama-3.1-8b", 1) else None,
                                "peak_source": peak_kind,
                                "kernel": "w4a16_gemv_persist_kernel (fused gate|up projection)",
                                "bytes_per_launch": w4a16_bytes(args.batch, blk.gate_up.out_features, blk.gate_up.in_features)}
        try:
            if args.skip_cpu_baseline:
                raise RuntimeError("skipped by --skip-cpu-baseline")
            csec, info = cpu_block_seconds(SHAPES[args.shape], args.batch, args.context, 3, 1)
            line["cpu_baseline"] = {"value": args.batch / (csec * args.layers), "unit": UNIT, **info}
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
