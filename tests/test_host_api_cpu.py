"""Host-side mirror of the reference API, checked on CPU: layout contract, config validation,
QuantizedLinear state and eager branch, cache schedule, save/load, and the C-ABI export table.
(Modelled on the reference's tests/test_core.py:162-197, tests/test_schemes.py:101-147,
tests/test_triton_kernel.py:42-101, tests/test_model_io.py.)"""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

import pare_b200
from oracle import kivi as ok
from oracle import w4a16 as ow
from pare_b200 import KVCacheConfig, QuantConfig, QuantDtype, QuantizedKVCache, QuantizedLinear
from pare_b200.core import compute_scale, dequantize_tensor, pack_int4, quantize_tensor, unpack_int4
from pare_b200.core.pack import (pack_int4_signed, packed_size_bytes, repack_int4_for_kernel, unpack_int4_signed,
                                 unrepack_int4_from_kernel)
from pare_b200.kernels import _lib
from pare_b200.kv_cache import plan_update

ROOT = Path(__file__).resolve().parent.parent


# ---- layout contract -----------------------------------------------------------------------

def test_pack_layout_and_roundtrip():
    assert pack_int4(torch.arange(8).reshape(1, 8)).numpy().view("<u4")[0, 0] == 0x76543210
    q = torch.randint(0, 16, (7, 3, 64), dtype=torch.int32)
    p = pack_int4(q)
    assert p.dtype == torch.uint8 and p.shape == (7, 3, 32)
    assert torch.equal(unpack_int4(p), q)
    assert np.array_equal(p.numpy(), ow.pack_int4(q.numpy()))
    edge = torch.tensor([[0, 15, 15, 0, 8, 7]], dtype=torch.int32)
    assert torch.equal(unpack_int4(pack_int4(edge)), edge)
    s = torch.randint(-8, 8, (4, 16), dtype=torch.int32)
    assert torch.equal(unpack_int4_signed(pack_int4_signed(s)), s)
    with pytest.raises(ValueError):
        pack_int4(torch.zeros(2, 5, dtype=torch.int32))
    assert packed_size_bytes((4096, 4096), 4) == 8388608


def test_repack_for_kernel_roundtrip_and_group_isolation():
    q = torch.randint(0, 16, (8, 256), dtype=torch.int32)
    packed = pack_int4(q)
    rep = repack_int4_for_kernel(packed, 128)
    assert rep.shape == packed.shape and rep.dtype == torch.uint8
    b = rep.to(torch.int32)
    for t in range(2):                                   # low nibble = first half of the tile, high = second half
        tile = b[:, t * 64:(t + 1) * 64]
        assert torch.equal(tile & 0xF, q[:, t * 128:t * 128 + 64])
        assert torch.equal(tile >> 4, q[:, t * 128 + 64:(t + 1) * 128])
    assert torch.equal(unrepack_int4_from_kernel(rep, 128), packed)
    assert repack_int4_for_kernel(torch.zeros(4, 64, dtype=torch.uint8), 128).eq(0).all()


# ---- dtype / config / scale -------------------------------------------------------------------

def test_dtype_and_config():
    assert (QuantDtype.INT4.qmin, QuantDtype.INT4.qmax, QuantDtype.INT4.levels) == (0, 15, 16)
    assert (QuantDtype.INT8.qmin, QuantDtype.INT8.qmax) == (-128, 127)
    assert QuantDtype.from_bits(4) is QuantDtype.INT4 and QuantDtype.from_bits(8) is QuantDtype.INT8
    assert QuantDtype.FP8_E4M3 is not QuantDtype.FP8_E5M2
    with pytest.raises(TypeError):
        QuantDtype.NF4.qmax
    with pytest.raises(ValueError):
        QuantDtype.from_bits(5)
    cfg = QuantConfig()
    assert (cfg.bits, cfg.scheme, cfg.granularity, cfg.group_size, cfg.sym, cfg.exclude) == (4, "awq", "per_group", 128, False, ["lm_head"])
    assert cfg.effective_dtype is QuantDtype.INT4
    for bad in (dict(scheme="foo"), dict(granularity="x"), dict(bits=5), dict(calibration="nope")):
        with pytest.raises(ValueError):
            QuantConfig(**bad)
    assert QuantConfig(dtype=QuantDtype.NF4, granularity="per_group").granularity == "per_channel"


def test_compute_scale_shapes_and_quant_roundtrip():
    w = torch.randn(16, 256)
    s, z = compute_scale(w, QuantDtype.INT4, granularity="per_group", group_size=128)
    assert s.shape == (16, 2, 1) and z.shape == (16, 2, 1) and z.min() >= 0 and z.max() <= 15
    assert torch.equal(z, z.round())
    s1, _ = compute_scale(w, QuantDtype.INT4, granularity="per_channel")
    s0, _ = compute_scale(w, QuantDtype.INT4, granularity="per_tensor")
    assert s1.shape == (16, 1) and s0.dim() == 0
    q = quantize_tensor(w, s, z, QuantDtype.INT4)
    assert q.dtype == torch.int32 and q.min() >= 0 and q.max() <= 15
    rec = dequantize_tensor(q.reshape(16, 256), s, z).reshape(16, 256)   # flat codes, as QuantizedLinear stores them
    assert (rec - w).abs().max() <= 0.5 * s.max() + 1e-6
    with pytest.raises(ValueError):
        compute_scale(torch.randn(4, 100), QuantDtype.INT4, granularity="per_group", group_size=128)


# ---- QuantizedLinear on the host ---------------------------------------------------------------

def test_quantized_linear_matches_reference_fixture(golden):
    """Layer rebuilt from the reference's own stored tensors: dequantize and eager forward are bit-exact."""
    g = golden("w4a16_g128.npz")
    cfg = QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128)
    ql = QuantizedLinear.from_tensors(torch.from_numpy(g["packed"]), None, torch.from_numpy(g["scale"]),
                                      torch.from_numpy(g["zero"]), cfg, None, 256, 256)
    assert ql.use_kernel is False                       # the reference leaves this unset on loaded layers
    assert np.array_equal(ql.dequantize().numpy(), g["w"])
    with torch.no_grad():
        y = ql(torch.from_numpy(g["x"]).float())
    assert np.allclose(y.numpy(), g["y"], atol=2e-5, rtol=0)


def test_from_linear_reproduces_reference_quantization(golden):
    g = golden("w4a16_g128.npz")
    torch.manual_seed(0)
    ql = QuantizedLinear.from_linear(nn.Linear(256, 256, bias=False), QuantConfig(bits=4, scheme="rtn", group_size=128))
    assert ql.packed_weight.dtype == torch.uint8 and ql.packed_weight.shape == (256, 128) and ql.q_weight is None
    assert np.array_equal(ql.packed_weight.numpy(), g["packed"])
    assert np.array_equal(ql.scale.numpy(), g["scale"]) and np.array_equal(ql.zero.numpy(), g["zero"])
    ql.use_kernel = True                                # CPU input: eager branch, no error
    assert ql(torch.randn(4, 256)).shape == (4, 256)
    assert "_packed_weight_kernel" not in ql.state_dict() and not hasattr(ql, "_packed_weight_kernel")
    q8 = QuantizedLinear.from_linear(nn.Linear(64, 32), QuantConfig(bits=8, scheme="rtn", granularity="per_channel"))
    assert q8.q_weight.dtype == torch.int8 and q8.packed_weight is None and q8.bias is not None


def test_g_idx_and_input_scale_eager_semantics():
    torch.manual_seed(4)
    ql = QuantizedLinear.from_linear(nn.Linear(256, 64, bias=False), QuantConfig(bits=4, scheme="rtn", group_size=128))
    ident = (torch.arange(256) // 128).to(torch.int32)
    w0 = ql.dequantize()
    ql.g_idx = ident
    assert torch.equal(ql.dequantize(), w0)             # identity g_idx == plain grouping, bit for bit
    s = torch.rand(256) + 0.5
    ql.input_scale = s
    x = torch.randn(3, 256)
    assert torch.allclose(ql(x), nn.functional.linear(x / s, w0), atol=1e-5)
    assert {"g_idx", "input_scale"} <= set(ql.state_dict())


def test_quantize_rtn_and_save_load_roundtrip(tmp_path):
    model = nn.Sequential(nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 256))
    model.add_module("lm_head", nn.Linear(256, 10))
    pare_b200.quantize(model, QuantConfig(bits=4, scheme="rtn", group_size=128))
    assert isinstance(model[0], QuantizedLinear) and isinstance(model.lm_head, nn.Linear)   # default exclude
    x = torch.randn(2, 256)
    y = model(x)
    pare_b200.save_quantized(model, tmp_path / "ckpt")
    meta = __import__("json").loads((tmp_path / "ckpt" / "pare_config.json").read_text())
    assert set(meta["quantized_layers"]["0"]) == {"bits", "scheme", "granularity", "group_size", "sym", "smooth_alpha",
                                                   "in_features", "out_features", "quantize_inputs", "has_bias"}
    fresh = nn.Sequential(nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 256))
    fresh.add_module("lm_head", nn.Linear(256, 10))
    pare_b200.load_quantized(fresh, tmp_path / "ckpt")
    assert torch.equal(fresh(x), y)                     # bit-exact round trip
    with pytest.raises(ValueError):
        pare_b200.save_quantized(nn.Linear(4, 4), tmp_path / "none")
    with pytest.raises(NotImplementedError):
        pare_b200.quantize(nn.Linear(4, 4), QuantConfig(scheme="gptq"))


def test_load_quantized_tensor_parallel_slices(tmp_path):
    """Loading with a tensor-parallel plan reads each rank's slice from the file; the slices are those of
    ``shard_linear`` and together reproduce the unsharded model (column shards concatenate, row shards add)."""
    from pare_b200.parallel import shard_linear

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.up_proj = nn.Linear(256, 512, bias=True)
            self.down_proj = nn.Linear(512, 256, bias=True)

        def forward(self, x):
            return self.down_proj(torch.relu(self.up_proj(x)))

    torch.manual_seed(3)
    model = MLP()
    pare_b200.quantize(model, QuantConfig(bits=4, scheme="rtn", group_size=128))
    x = torch.randn(3, 256)
    y = model(x)
    pare_b200.save_quantized(model, tmp_path / "ckpt")
    plan = {"up_proj": "column", "down_proj": "row"}
    partial = []
    for rank in range(2):
        shard = MLP()
        pare_b200.load_quantized(shard, tmp_path / "ckpt", tp_plan=plan, tp_rank=rank, tp_world=2)
        assert shard.up_proj.out_features == 256 and shard.down_proj.in_features == 256
        for name, mode in plan.items():
            want = shard_linear(getattr(model, name), mode, rank, 2)
            got = getattr(shard, name)
            assert torch.equal(got.packed_weight, want.packed_weight) and torch.equal(got.scale, want.scale)
            assert torch.equal(got.zero, want.zero)
            assert (got.bias is None) == (want.bias is None) and (got.bias is None or torch.equal(got.bias, want.bias))
        partial.append(shard(x))     # up: this rank's columns -> relu -> down: this rank's partial sum
    assert torch.allclose(partial[0] + partial[1], y, atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError):
        pare_b200.load_quantized(MLP(), tmp_path / "ckpt", tp_plan={"up_proj": "diagonal"}, tp_rank=0, tp_world=2)


def test_awq_gemm_layout_roundtrip():
    """The AutoAWQ GEMM layout: nibble i of an int32 holds output column 8w + (0,2,4,6,1,3,5,7)[i]; export then
    import gives the same codes, zero points and (fp16-rounded) scales, hence the same dequantized weights."""
    from pare_b200.model.awq_format import ORDER, _pack_columns, _unpack_columns, from_awq_gemm, to_awq_gemm

    codes = torch.arange(16, dtype=torch.uint8).repeat(2)[:16].reshape(1, 16)       # columns 0..15 hold codes 0..15
    word = _pack_columns(codes)
    assert word.dtype == torch.int32 and word.shape == (1, 2)
    w0 = int(word[0, 0]) & 0xFFFFFFFF
    assert [(w0 >> (4 * i)) & 0xF for i in range(8)] == list(ORDER)                  # nibble i <- column ORDER[i]
    assert torch.equal(_unpack_columns(word), codes)
    hi = _pack_columns(torch.full((1, 8), 15, dtype=torch.uint8))                    # all nibbles set: wraps to -1
    assert int(hi[0, 0]) == -1 and torch.equal(_unpack_columns(hi), torch.full((1, 8), 15, dtype=torch.uint8))

    torch.manual_seed(5)
    lin = nn.Linear(256, 64, bias=True)
    ql = QuantizedLinear.from_linear(lin, QuantConfig(bits=4, scheme="rtn", group_size=128))
    t = to_awq_gemm(ql)
    assert t["qweight"].shape == (256, 8) and t["qzeros"].shape == (2, 8) and t["scales"].shape == (2, 64)
    back = from_awq_gemm(t["qweight"], t["qzeros"], t["scales"], t["bias"], group_size=128)
    assert torch.equal(back.packed_weight, ql.packed_weight) and torch.equal(back.zero, ql.zero)
    assert torch.equal(back.scale, ql.scale.half().float())
    assert torch.allclose(back.dequantize(), ql.dequantize(), rtol=2 ** -10, atol=0)   # scales went through fp16
    assert back.bias.dtype == torch.float16 and torch.equal(back.bias.float(), lin.bias.detach().half().float())
    with pytest.raises(ValueError):
        to_awq_gemm(QuantizedLinear.from_linear(nn.Linear(256, 64), QuantConfig(bits=4, scheme="rtn", granularity="per_channel")))


# ---- cache schedule ----------------------------------------------------------------------------------

def test_plan_update_matches_oracle_state_machine():
    for residual, group in ((128, 32), (64, 32), (0, 32), (100, 16)):
        ref = ok.Cache(4, group, residual)
        r_len = 0
        rng = np.random.default_rng(residual + group)
        for n_new in [200, 1, 1, 37, 1, 64, 5] + [1] * 70:
            x = rng.standard_normal((1, 1, n_new, 8)).astype(np.float32)
            ref.update(x, x)
            n_c, r_len = plan_update(r_len, n_new, residual, group)
            assert r_len == ref.n_res and n_c % group == 0
            assert residual <= r_len < residual + group or ref.n_comp == 0


def test_cache_host_api_without_gpu():
    cache = QuantizedKVCache(2, KVCacheConfig(bits=4, group_size=32, residual_length=64))
    assert cache.seq_len(0) == 0 and cache.memory_bytes(1) == {"compressed": 0, "residual": 0, "total": 0}
    assert cache._compressed == [None, None] and cache._residual_k == [None, None]
    with pytest.raises(RuntimeError):
        cache.update(0, torch.randn(1, 2, 4, 128), torch.randn(1, 2, 4, 128))     # CPU tensors: no fallback
    with pytest.raises(ValueError):
        QuantizedKVCache(1, KVCacheConfig(bits=3))
    cache.reset()


# ---- the C ABI ------------------------------------------------------------------------------------------

def test_library_exports_every_declared_symbol():
    """Loads the built library (no GPU needed) and checks the header, the ctypes table and the exports agree."""
    header = (ROOT / "include" / "pare_b200.h").read_text()
    declared = set(re.findall(r"\b(pare_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.LIB_PATH.exists(), "build with `python -m pare_b200.build`"
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(handle, name), name
    handle.pare_status_string.restype = ctypes.c_char_p
    assert handle.pare_version() >= 100
    assert handle.pare_status_string(0) == b"ok" and b"workspace" in handle.pare_status_string(4)
    handle.pare_w4a16_workspace_bytes.restype = ctypes.c_size_t
    assert handle.pare_w4a16_workspace_bytes(1, 4096, 4096, 128) >= 65536
    assert handle.pare_w4a16_workspace_bytes(0, 1, 1, 1) == 0


def test_rope_helpers_agree_with_the_oracle():
    """``rope_table`` / ``apply_rope`` (host side of the rotary step the attention kernel performs) against the numpy
    restatement: the same table up to libm rounding, the same rotation bit for bit, norm-preserving per pair,
    identity at position 0."""
    import numpy as np
    from oracle import kivi as ok
    from pare_b200.kv_cache import apply_rope, rope_table

    table = rope_table(300, 128, 500000.0)
    rows = ok.rope_rows(np.arange(300), 128, 500000.0)
    assert table.shape == (300, 128) and table.dtype == torch.float32
    assert np.allclose(table.numpy(), rows, rtol=0, atol=2e-6)
    x = torch.randn(2, 3, 5, 128, generator=torch.Generator().manual_seed(0))
    for dtype in (torch.float16, torch.bfloat16):
        xd = x.to(dtype)
        got = apply_rope(xd, table[100:105])
        ref = torch.from_numpy(ok.apply_rope(xd.float().numpy(), table[100:105].numpy())).to(dtype)
        assert torch.equal(got, ref)
        assert torch.equal(apply_rope(xd, table[0]), xd)
    y = ok.apply_rope(x.numpy(), rows[200])
    n0 = x.numpy()[..., :64] ** 2 + x.numpy()[..., 64:] ** 2
    n1 = y[..., :64] ** 2 + y[..., 64:] ** 2
    assert np.allclose(n0, n1, rtol=1e-5, atol=1e-6)


def test_reference_arm_prints_the_contract_line():
    """``bench.py --impl reference`` (the CPU op sequence of the reference, timed on the host) prints one JSON line with
    the keys the harness reads; under a multi-rank launch only rank 0 prints."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--layers", "1",
           "--context", "256"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["value"] > 0
    assert line["unit"] == "tok/s" and line["metric"].startswith("decode_tok_s")
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    other = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root, env=dict(os.environ, RANK="1", WORLD_SIZE="2"))
    assert other.returncode == 0 and other.stdout.strip() == ""
