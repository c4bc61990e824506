"""KIVI cache CUDA kernels vs the CPU oracle and the committed reference outputs (GPU).

Bars: codes, scales and zeros BIT-EXACT against the oracle (which is pinned bit-exact to the
reference); dense ``update()`` output bit-exact in the input dtype; fused attention within
max rel err <= 1e-2 and mean <= 1e-3 of fp32 attention over the dense cache the reference
would return (``|o - ref| / max(|ref|, 1e-2 * max|ref|)``).
"""

import numpy as np
import pytest
import torch

from oracle import kivi as ok
from oracle.w4a16 import rel_err
from pare_b200.kv_cache import (KVCacheConfig, QuantizedKVCache, _dequantize_keys, _dequantize_values,
                                _quantize_keys, _quantize_values)

pytestmark = pytest.mark.gpu

B, H, G, D = 1, 8, 32, 128


def _kv(n, seed=0, b=B, h=H, dtype=torch.float16, outliers=True):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(b, h, n, D, generator=g)
    v = torch.randn(b, h, n, D, generator=g)
    if outliers:
        k[..., 7] *= 10.0
    return k.to(dtype).cuda(), v.to(dtype).cuda()


# ---- primitives --------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [2, 4, 8])
def test_primitives_match_reference_fixture(bits, golden, cuda_lib):
    g = golden("kivi_prims.npz")
    k = torch.from_numpy(g["k"]).cuda()
    v = torch.from_numpy(g["v"]).cuda()
    kq, ks, kz = _quantize_keys(k, bits, 32)
    vq, vs, vz = _quantize_values(v, bits, 32)
    for name, got in (("kq", kq), ("ks", ks), ("kz", kz), ("vq", vq), ("vs", vs), ("vz", vz)):
        assert np.array_equal(got.cpu().numpy(), g[f"{name}{bits}"]), (name, bits)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits,group", [(4, 32), (2, 32), (8, 16), (4, 64), (4, 128)])
def test_primitives_bit_exact_vs_oracle(bits, group, dtype, cuda_lib):
    k, v = _kv(256, seed=bits + group, b=2, h=3, dtype=dtype)
    kq, ks, kz = _quantize_keys(k, bits, group)
    vq, vs, vz = _quantize_values(v, bits, group)
    assert kq.shape == (2, 3, 256, D) and kq.dtype == torch.uint8
    assert ks.shape == (2, 3, 256 // group, D) and vs.shape == (2, 3, 256, 1)
    ref_k = ok.quantize_keys(k.float().cpu().numpy(), bits, group)
    ref_v = ok.quantize_values(v.float().cpu().numpy(), bits, group)
    for got, ref in zip((kq, ks, kz, vq, vs, vz), ref_k + ref_v):
        assert np.array_equal(got.cpu().numpy(), ref)
    assert int(kq.max()) <= (1 << bits) - 1
    rec = _dequantize_keys(kq, ks, kz, group)
    assert ((rec - k.float()) ** 2).mean().item() < (0.5 if bits >= 4 else 5.0)
    assert _dequantize_values(vq, vs, vz).shape == v.shape


def test_constant_input_hits_scale_floor(cuda_lib):
    k = torch.full((1, 1, 32, D), 3.0, device="cuda", dtype=torch.float16)
    kq, ks, kz = _quantize_keys(k, 4, 32)
    assert torch.all(kq == 0) and torch.all(ks == 1e-8) and torch.all(kz == 3.0)


# ---- cache state machine (mirrors the reference's tests/test_kv_cache.py:159-273) -------

def test_residual_only_before_overflow(cuda_lib):
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128))
    k, v = _kv(64)
    fk, fv = cache.update(0, k, v)
    assert cache._compressed[0] is None
    assert fk.shape == (B, H, 64, D) and torch.equal(fk, k) and torch.equal(fv, v)


def test_compression_triggers_and_counts(cuda_lib):
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=64))
    k, v = _kv(128)
    cache.update(0, k, v)
    assert cache._compressed[0].k_quant.shape[2] == 64
    assert cache._residual_k[0].shape[2] == 64
    assert cache.seq_len(0) == 128
    mem = cache.memory_bytes(0)
    assert mem["compressed"] > 0 and mem["residual"] > 0 and mem["compressed"] + mem["residual"] == mem["total"]


def test_shapes_dtype_reset(cuda_lib):
    cache = QuantizedKVCache(2, KVCacheConfig(bits=4, group_size=32, residual_length=64))
    k, v = _kv(96)
    fk, _ = cache.update(0, k, v)
    assert fk.shape == (B, H, 96, D)
    for i in range(3):
        k1, v1 = _kv(1, seed=10 + i)
        fk, fv = cache.update(0, k1, v1)
    assert fk.shape == (B, H, 99, D) and fk.dtype == torch.float16
    cache.update(1, k, v)
    cache.reset(0)
    assert cache._compressed[0] is None and cache._residual_k[0] is None and cache._residual_k[1] is not None
    cache.reset()
    assert all(c is None for c in cache._compressed) and all(r is None for r in cache._residual_k)


def test_int8_residual_zero_reconstruction(cuda_lib):
    cache = QuantizedKVCache(1, KVCacheConfig(bits=8, group_size=32, residual_length=0))
    k, v = _kv(64, outliers=False)
    fk, fv = cache.update(0, k, v)
    assert ((fk.float() - k.float()) ** 2).mean().item() < 0.01
    assert ((fv.float() - v.float()) ** 2).mean().item() < 0.01


def test_reference_sequence_fixture(golden, cuda_lib):
    """96-token prefill + 40 decode steps: token counts, dense output and attention vs the reference's own run."""
    g = golden("kivi_cache.npz")
    k_all = torch.from_numpy(g["k_all"]).cuda()
    v_all = torch.from_numpy(g["v_all"]).cuda()
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=64))
    counts = []
    fk, fv = cache.update(0, k_all[:, :, :96], v_all[:, :, :96])
    counts.append((cache._compressed[0].k_quant.shape[2] if cache._compressed[0] is not None else 0,
                   cache._residual_k[0].shape[2]))
    for t in range(96, k_all.shape[2]):
        fk, fv = cache.update(0, k_all[:, :, t:t + 1], v_all[:, :, t:t + 1])
        counts.append((cache._compressed[0].k_quant.shape[2], cache._residual_k[0].shape[2]))
    assert np.array_equal(np.array(counts), g["counts"])
    assert np.array_equal(fk.cpu().numpy(), g["full_k"])
    assert np.array_equal(fv.cpu().numpy(), g["full_v"])

    # fused attention over the same final state (feed the last token through attend on a twin cache)
    twin = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=64))
    twin.update(0, k_all[:, :, :96], v_all[:, :, :96])
    for t in range(96, k_all.shape[2] - 1):
        twin.update(0, k_all[:, :, t:t + 1], v_all[:, :, t:t + 1])
    q = torch.from_numpy(g["q"]).cuda()
    out = twin.attend(0, q, k_all[:, :, -1:], v_all[:, :, -1:])
    ref_cache = ok.Cache(4, 32, 64)
    rk, rv = ref_cache.update(g["k_all"].astype(np.float32), g["v_all"].astype(np.float32))
    ref32 = ok.decode_attention(g["q"], rk, rv)
    _check_attn(out.float().cpu().numpy(), g["attn"], ref32, torch.float16)   # g["attn"]: the reference's own run


@pytest.mark.parametrize("bits", [4, 2])
def test_incremental_matches_batch_and_oracle(bits, cuda_lib):
    cfg = KVCacheConfig(bits=bits, group_size=32, residual_length=64)
    k_all, v_all = _kv(416, seed=99, b=2, h=2)
    one = QuantizedKVCache(1, cfg)
    fk1, fv1 = one.update(0, k_all, v_all)
    inc = QuantizedKVCache(1, cfg)
    for i in range(0, 416, 32):
        fk2, fv2 = inc.update(0, k_all[:, :, i:i + 32], v_all[:, :, i:i + 32])
    tok = QuantizedKVCache(1, cfg)
    tok.update(0, k_all[:, :, :300], v_all[:, :, :300])
    for i in range(300, 416):
        fk3, fv3 = tok.update(0, k_all[:, :, i:i + 1], v_all[:, :, i:i + 1])
    assert torch.equal(fk1, fk2) and torch.equal(fv1, fv2) and torch.equal(fk1, fk3) and torch.equal(fv1, fv3)
    ref = ok.Cache(bits, 32, 64)
    rk, rv = ref.update(k_all.float().cpu().numpy(), v_all.float().cpu().numpy())
    assert np.array_equal(fk1.cpu().numpy(), rk.astype(np.float16))
    assert np.array_equal(fv1.cpu().numpy(), rv.astype(np.float16))
    c = one._compressed[0]
    for got, want in zip(c, ref.comp):
        assert np.array_equal(got.cpu().numpy(), want)


def test_capacity_growth_keeps_contents(cuda_lib):
    cfg = KVCacheConfig(bits=4, group_size=32, residual_length=32)
    k_all, v_all = _kv(2600, seed=5, b=1, h=2)
    grow = QuantizedKVCache(1, cfg)                      # starts at 1024 tokens, must grow twice
    for i in range(0, 2600, 200):
        fk, fv = grow.update(0, k_all[:, :, i:i + 200], v_all[:, :, i:i + 200])
    big = QuantizedKVCache(1, cfg, max_seq_len=4096)
    fk2, fv2 = big.update(0, k_all, v_all)
    assert torch.equal(fk, fk2) and torch.equal(fv, fv2)


def test_cpu_tensors_rejected(cuda_lib):
    cache = QuantizedKVCache(1)
    with pytest.raises(RuntimeError):
        cache.update(0, torch.randn(1, 2, 4, D), torch.randn(1, 2, 4, D))


# ---- fused decode attention ------------------------------------------------------------------

def _attn_case(bsz, hkv, hq, ctx, dtype, residual=128, group=32, seed=0, bits=4):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(bsz, hkv, ctx, D, generator=g)
    v = torch.randn(bsz, hkv, ctx, D, generator=g)
    idx = torch.randperm(D, generator=g)[:2]
    k[..., idx] *= 10.0                                  # outlier channels
    q = torch.randn(bsz, hq, 1, D, generator=g)
    k, v, q = k.to(dtype).cuda(), v.to(dtype).cuda(), q.to(dtype).cuda()
    cfg = KVCacheConfig(bits=bits, group_size=group, residual_length=residual)
    cache = QuantizedKVCache(1, cfg, max_seq_len=ctx + 256)
    cache.update(0, k[:, :, :-1], v[:, :, :-1])
    out = cache.attend(0, q, k[:, :, -1:], v[:, :, -1:])
    ref_cache = ok.Cache(bits, group, residual)
    rk, rv = ref_cache.update(k.float().cpu().numpy(), v.float().cpu().numpy())
    cast = (lambda a: torch.from_numpy(a).to(dtype).float().numpy())
    qf = q.float().cpu().numpy()
    # ref: attention over the reconstruction in the cache dtype (what update() hands a caller);
    # ref32: over the fp32 reconstruction before that cast
    return out, ok.decode_attention(qf, cast(rk), cast(rv)), cache, ok.decode_attention(qf, rk, rv)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bsz,hkv,hq,ctx", [(1, 4, 28, 1000), (2, 2, 16, 4096), (1, 1, 8, 160), (3, 2, 8, 100), (1, 2, 2, 2500)])
def test_decode_attention_matches_oracle(bsz, hkv, hq, ctx, dtype, cuda_lib):
    out, ref, _, ref32 = _attn_case(bsz, hkv, hq, ctx, dtype)
    assert out.shape == (bsz, hq, 1, D) and out.dtype == dtype
    o = out.float().cpu().numpy()
    _check_attn(o, ref, ref32, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bsz,hkv,hq,ctx,group", [(1, 4, 28, 1000, 32), (2, 2, 16, 4096, 32), (1, 1, 8, 200, 16), (1, 2, 4, 700, 64)])
def test_decode_attention_two_bit_cache(bsz, hkv, hq, ctx, group, dtype, cuda_lib):
    """The same kernel over a 2-bit cache (16 codes per word, pairs (c_j, c_j+8)); same bars: the kernel's arithmetic
    is exact on the stored codes, so the coarser quantization is in the oracle's K^ / V^ as well."""
    out, ref, _, ref32 = _attn_case(bsz, hkv, hq, ctx, dtype, group=group, residual=64 if group == 64 else 128, bits=2, seed=ctx)
    _check_attn(out.float().cpu().numpy(), ref, ref32, dtype)


@pytest.mark.parametrize("bits", [4, 2])
def test_decode_attention_longest_benchmark_context(bits, cuda_lib):
    """The longest context of the benchmark grid (32768 tokens, 28 query / 4 KV heads, 128 compressed-token splits per
    head) against the oracle, same bars."""
    out, ref, cache, ref32 = _attn_case(1, 4, 28, 32768, torch.float16, bits=bits, seed=11)
    assert cache._stores[0].n_comp >= 32768 - 128 - 32
    _check_attn(out.float().cpu().numpy(), ref, ref32, torch.float16)


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("bsz,ctx", [(16, 4096), (4, 16384)])
def test_decode_attention_benchmark_grid_cells(bsz, ctx, bits, cuda_lib):
    """Cells of the benchmark grid that the smaller cases do not reach: batch 16 at 4096 tokens and batch 4 at
    16384 tokens, 28 query / 4 KV heads (seven query heads per KV head), 4- and 2-bit caches; same bars."""
    out, ref, cache, ref32 = _attn_case(bsz, 4, 28, ctx, torch.float16, bits=bits, seed=bsz + ctx)
    assert out.shape == (bsz, 28, 1, D)
    _check_attn(out.float().cpu().numpy(), ref, ref32, torch.float16)


def _check_attn(o, ref, ref32, dtype):
    """Two bars.  (1) Tight, against fp32 attention over the reference's reconstruction BEFORE its final
    cast (``_reconstruct``, pare/kv_cache.py:315-325): max <= 1e-2, mean <= 1e-3 (2.5e-3 for bf16
    outputs, 8 significant bits).  (2) Against attention over what ``update()`` returns, i.e. after the
    cast to fp16/bf16: that cast alone moves the reference by up to several 1e-2 on outlier channels
    (measured here as ref vs ref32), so the kernel must stay within 1.5x of that self-noise."""
    mx, mean = rel_err(o, ref32)
    assert mx <= 1e-2 and mean <= (2.5e-3 if dtype == torch.bfloat16 else 1e-3), (mx, mean)
    noise_mx, noise_mean = rel_err(ref, ref32)
    mx2, mean2 = rel_err(o, ref)
    assert mx2 <= 1.5 * noise_mx + 1e-2 and mean2 <= 1.5 * noise_mean + (2.5e-3 if dtype == torch.bfloat16 else 1e-3), \
        (mx2, mean2, noise_mx, noise_mean)


def test_decode_attention_other_groups_and_steps(cuda_lib):
    for group, residual in ((64, 64), (128, 128), (16, 32), (32, 0)):
        out, ref, _, ref32 = _attn_case(1, 2, 8, 700, torch.float16, residual=residual, group=group, seed=group)
        _check_attn(out.float().cpu().numpy(), ref, ref32, torch.float16)


def test_decode_attention_is_deterministic_and_steps(cuda_lib):
    out, ref, cache, _ = _attn_case(1, 2, 14, 3000, torch.float16, seed=3)
    g = torch.Generator().manual_seed(77)
    for _ in range(40):                                   # crosses a compression boundary
        k1 = torch.randn(1, 2, 1, D, generator=g).half().cuda()
        v1 = torch.randn(1, 2, 1, D, generator=g).half().cuda()
        q1 = torch.randn(1, 14, 1, D, generator=g).half().cuda()
        o1 = cache.attend(0, q1, k1, v1)
    o2 = cache.attend(0, q1, k1[:, :, :0], v1[:, :, :0])  # same state, nothing appended: bit-identical result
    assert torch.equal(o1, o2)
    c = cache._compressed[0]                              # fp32 reconstruction of the same state
    rk = torch.cat([ok_t(ok.dequantize_keys(c.k_quant.cpu().numpy(), c.k_scale.cpu().numpy(), c.k_zero.cpu().numpy(), 32)),
                    cache._residual_k[0].float().cpu()], dim=2).numpy()
    rv = torch.cat([ok_t(ok.dequantize_values(c.v_quant.cpu().numpy(), c.v_scale.cpu().numpy(), c.v_zero.cpu().numpy())),
                    cache._residual_v[0].float().cpu()], dim=2).numpy()
    fk, fv = cache.update(0, k1[:, :, :0], v1[:, :, :0])
    qn = q1.float().cpu().numpy()
    _check_attn(o1.float().cpu().numpy(), ok.decode_attention(qn, fk.float().cpu().numpy(), fv.float().cpu().numpy()),
                ok.decode_attention(qn, rk, rv), torch.float16)


def ok_t(a):
    return torch.from_numpy(a)


# ---- rotary embedding inside the attention launch ------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ctx", [200, 160])
def test_decode_attention_rotates_q_and_new_key(ctx, dtype, cuda_lib):
    """``attend(..., rope=row)``: q and the newest key get the rotary embedding inside the launch.  The stored key is
    bit-exact the oracle's rotation rounded to the dtype; the attention output meets the usual bars against the oracle
    on rotated inputs.  ctx = 200: the kernel appends (and rotates) the key itself; ctx = 160: the append compresses a
    group first, so the host side rotates the key and the kernel only the query."""
    from pare_b200.kv_cache import apply_rope, rope_table
    bsz, hkv, hq = 2, 2, 8
    g = torch.Generator().manual_seed(ctx)
    k = torch.randn(bsz, hkv, ctx, D, generator=g)
    v = torch.randn(bsz, hkv, ctx, D, generator=g)
    k[..., 5] *= 10.0
    q = torch.randn(bsz, hq, 1, D, generator=g)
    k, v, q = k.to(dtype).cuda(), v.to(dtype).cuda(), q.to(dtype).cuda()
    table = rope_table(ctx + 8, D, 500000.0, device="cuda")
    rows = ok.rope_rows(np.arange(ctx + 8), D, 500000.0)
    assert np.allclose(table.cpu().numpy(), rows, rtol=0, atol=2e-6)   # libm vs torch cos / sin of float64 angles
    rows = table.cpu().numpy()
    pos = ctx - 1
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128), max_seq_len=ctx + 256)
    cache.update(0, k[:, :, :-1], v[:, :, :-1])           # the older keys count as rotated already
    n_comp_before = cache._stores[0].n_comp
    out = cache.attend(0, q, k[:, :, -1:], v[:, :, -1:], rope=table[pos])
    assert (cache._stores[0].n_comp > n_comp_before) == (ctx == 160)

    cast = lambda a: torch.from_numpy(a).to(dtype).float().numpy()
    k_rot = cast(ok.apply_rope(k[:, :, -1:].float().cpu().numpy(), rows[pos]))
    q_rot = cast(ok.apply_rope(q.float().cpu().numpy(), rows[pos]))
    assert np.array_equal(cache._residual_k[0][:, :, -1:].float().cpu().numpy(), k_rot)     # stored key: bit-exact
    assert np.array_equal(apply_rope(k[:, :, -1:], table[pos]).float().cpu().numpy(), k_rot)  # the torch helper too
    k_all = np.concatenate([k[:, :, :-1].float().cpu().numpy(), k_rot], axis=2)
    ref_cache = ok.Cache(4, 32, 128)
    ref_cache.update(k_all[:, :, :-1], v[:, :, :-1].float().cpu().numpy())
    rk, rv = ref_cache.update(k_all[:, :, -1:], v[:, :, -1:].float().cpu().numpy())
    _check_attn(out.float().cpu().numpy(), ok.decode_attention(q_rot, cast(rk), cast(rv)), ok.decode_attention(q_rot, rk, rv), dtype)
    # position 0 is the identity
    cache2 = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128), max_seq_len=64)
    o_id = cache2.attend(0, q, k[:, :, :1], v[:, :, :1], rope=table[0])
    cache3 = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128), max_seq_len=64)
    assert torch.equal(o_id, cache3.attend(0, q, k[:, :, :1], v[:, :, :1]))


def test_rope_argument_checks(cuda_lib):
    from pare_b200.kv_cache import rope_table
    k, v = _kv(4, b=1, h=2)
    q = torch.randn(1, 4, 1, D).half().cuda()
    table = rope_table(16, D, device="cuda")
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128), max_seq_len=64)
    with pytest.raises(ValueError):
        cache.attend(0, q, k[:, :, :2], v[:, :, :2], rope=table[1])      # two new tokens
    with pytest.raises(ValueError):
        cache.attend(0, q, k[:, :, :1], v[:, :, :1], rope=table[1].half())


# ---- values quantized in 32-channel groups -------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_value_channel_groups_bit_exact_vs_oracle(bits, dtype, cuda_lib):
    """One (scale, zero) per token and 32 channels: codes, scales, zeros bit-exact against the oracle's
    ``quantize_values`` on the channel axis viewed as [D/32][32]; ``v_group_size = D`` is the reference's form."""
    _, v = _kv(128, seed=bits, b=2, h=3, dtype=dtype)
    vq, vs, vz = _quantize_values(v, bits, 32, v_group_size=32)
    assert vq.shape == (2, 3, 128, D) and vs.shape == (2, 3, 128, D // 32) and vz.shape == vs.shape
    for got, ref in zip((vq, vs, vz), ok.quantize_values(v.float().cpu().numpy(), bits, 32, 32)):
        assert np.array_equal(got.cpu().numpy(), ref)
    rec = _dequantize_values(vq, vs, vz)
    assert np.array_equal(rec.cpu().numpy(), ok.dequantize_values(vq.cpu().numpy(), vs.cpu().numpy(), vz.cpu().numpy()))
    whole = _quantize_values(v, bits, 32)
    same = _quantize_values(v, bits, 32, v_group_size=D)
    for a, b in zip(whole, same):
        assert torch.equal(a, b)
    err_g = ((rec - v.float()) ** 2).mean().item()
    err_w = ((_dequantize_values(*whole) - v.float()) ** 2).mean().item()
    assert err_g <= err_w                                   # finer groups never reconstruct worse


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("bsz,hkv,hq,ctx", [(1, 4, 28, 1000), (2, 2, 16, 4096), (1, 1, 8, 160)])
def test_value_channel_groups_cache_and_attention(bsz, hkv, hq, ctx, bits, dtype, cuda_lib):
    """The cache with 32-channel value groups: ``update()`` bit-exact against the oracle state machine, fused
    attention within the usual bars of fp32 attention over the oracle's reconstruction."""
    g = torch.Generator().manual_seed(ctx + bits)
    k = torch.randn(bsz, hkv, ctx, D, generator=g)
    v = torch.randn(bsz, hkv, ctx, D, generator=g)
    v[..., 40:44] *= 6.0                                    # a few loud value channels: where the finer groups matter
    k[..., 9] *= 10.0
    q = torch.randn(bsz, hq, 1, D, generator=g)
    k, v, q = k.to(dtype).cuda(), v.to(dtype).cuda(), q.to(dtype).cuda()
    cache = QuantizedKVCache(1, KVCacheConfig(bits=bits, group_size=32, residual_length=128, v_group_size=32), max_seq_len=ctx + 256)
    fk, fv = cache.update(0, k[:, :, :-1], v[:, :, :-1])
    ref_cache = ok.Cache(bits, 32, 128, v_group=32)
    rk, rv = ref_cache.update(k[:, :, :-1].float().cpu().numpy(), v[:, :, :-1].float().cpu().numpy())
    cast = (lambda a: torch.from_numpy(a).to(dtype).float().numpy())
    assert np.array_equal(fk.float().cpu().numpy(), cast(rk)) and np.array_equal(fv.float().cpu().numpy(), cast(rv))
    out = cache.attend(0, q, k[:, :, -1:], v[:, :, -1:])
    rk, rv = ref_cache.update(k[:, :, -1:].float().cpu().numpy(), v[:, :, -1:].float().cpu().numpy())
    qf = q.float().cpu().numpy()
    _check_attn(out.float().cpu().numpy(), ok.decode_attention(qf, cast(rk), cast(rv)), ok.decode_attention(qf, rk, rv), dtype)
    assert torch.equal(out, cache.attend(0, q, k[:, :, :0], v[:, :, :0]))     # deterministic
    m = cache.memory_bytes(0)
    n = cache._stores[0].n_comp
    assert m["compressed"] == bsz * hkv * (2 * n * D * bits // 8 + 2 * (n // 32) * D * 4 + 2 * n * 4 * 4)


def test_value_channel_group_argument_checks(cuda_lib):
    from pare_b200.kernels import _lib
    k, v = _kv(8, b=1, h=2)
    with pytest.raises(ValueError):
        QuantizedKVCache(1, KVCacheConfig(v_group_size=48)).update(0, k, v)
    cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=0, v_group_size=64), max_seq_len=256)
    k, v = _kv(64, b=1, h=2)
    fk, fv = cache.update(0, k, v)                          # the cache itself takes any multiple of 32
    assert fv.shape == v.shape
    q = torch.randn(1, 4, 1, D).half().cuda()
    with pytest.raises(_lib.KernelLibraryError):            # the fused attention only 32 or the whole head
        cache.attend(0, q, k[:, :, :0], v[:, :, :0])


# ---- prefill attention over full-precision K / V ---------------------------------------------------

def _bars_prefill(o, ref, dtype):
    mx, mean = rel_err(o, ref)
    assert mx <= 1e-2 and mean <= (2.5e-3 if dtype == torch.bfloat16 else 1e-3), (mx, mean)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bsz,hkv,hq,tq,tk,causal", [(1, 2, 8, 256, 256, True), (2, 1, 4, 100, 100, True), (1, 4, 28, 333, 333, True),
                                                      (1, 2, 4, 64, 200, True), (1, 1, 2, 1, 130, True), (2, 2, 2, 70, 70, False),
                                                      (1, 1, 1, 17, 17, True)])
def test_prefill_attention_matches_oracle(bsz, hkv, hq, tq, tk, causal, dtype, cuda_lib):
    """fp32 attention of the oracle on the same 16-bit inputs: max rel err <= 1e-2, mean <= 1e-3 (2.5e-3 for bf16
    outputs); ragged lengths, grouped-query sharing, queries that are the tail of a longer key sequence, and the
    first rows of a causal prompt (one or two visible keys) among the cases."""
    from pare_b200.kv_cache import prefill_attention
    g = torch.Generator().manual_seed(tq * 7 + tk)
    q = torch.randn(bsz, hq, tq, D, generator=g).to(dtype).cuda()
    k = torch.randn(bsz, hkv, tk, D, generator=g).to(dtype).cuda()
    v = torch.randn(bsz, hkv, tk, D, generator=g).to(dtype).cuda()
    out = prefill_attention(q, k, v, causal=causal)
    assert out.shape == q.shape and out.dtype == dtype
    ref = ok.causal_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), causal=causal)
    _bars_prefill(out.float().cpu().numpy(), ref, dtype)
    assert torch.equal(out, prefill_attention(q, k, v, causal=causal))          # deterministic
    # strided views (a fused q|k|v projection output) give the same bits
    qkv = torch.randn(bsz, max(tq, tk), (hq + 2 * hkv) * D, generator=g).to(dtype).cuda()
    q2 = qkv[:, :tq, : hq * D].unflatten(2, (hq, D)).transpose(1, 2)
    k2 = qkv[:, :tk, hq * D:(hq + hkv) * D].unflatten(2, (hkv, D)).transpose(1, 2)
    v2 = qkv[:, :tk, (hq + hkv) * D:].unflatten(2, (hkv, D)).transpose(1, 2)
    assert torch.equal(prefill_attention(q2, k2, v2, causal=causal),
                       prefill_attention(q2.contiguous(), k2.contiguous(), v2.contiguous(), causal=causal))


def test_prefill_attention_long_prompt(cuda_lib):
    """2048-token prompt (32 query tiles per head, 32 key tiles for the last of them): same bars."""
    from pare_b200.kv_cache import prefill_attention
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 8, 2048, D, generator=g).half().cuda()
    k = torch.randn(1, 2, 2048, D, generator=g).half().cuda()
    v = torch.randn(1, 2, 2048, D, generator=g).half().cuda()
    out = prefill_attention(q, k, v)
    ref = ok.causal_attention(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
    _bars_prefill(out.float().cpu().numpy(), ref, torch.float16)


def test_cache_prefill_then_decode(cuda_lib):
    """``prefill()`` = full-precision causal attention of the prompt + append; the decode step that follows sees the
    same cache as after ``update()``; a second chunk attends to the older tokens through the cache's reconstruction."""
    from pare_b200.kv_cache import apply_rope, rope_table
    g = torch.Generator().manual_seed(9)
    T = 300
    q = torch.randn(1, 8, T, D, generator=g).half().cuda()
    k = torch.randn(1, 2, T, D, generator=g).half().cuda()
    v = torch.randn(1, 2, T, D, generator=g).half().cuda()
    table = rope_table(T + 80, D, 500000.0, device="cuda")
    cfg = KVCacheConfig(bits=4, group_size=32, residual_length=128)
    a, b = QuantizedKVCache(1, cfg, max_seq_len=1024), QuantizedKVCache(1, cfg, max_seq_len=1024)
    out = a.prefill(0, q, k, v, rope=table[:T])
    kr, qr = apply_rope(k, table[:T]), apply_rope(q, table[:T])
    ref = ok.causal_attention(qr.float().cpu().numpy(), kr.float().cpu().numpy(), v.float().cpu().numpy())
    _bars_prefill(out.float().cpu().numpy(), ref, torch.float16)
    b.update(0, kr, v)
    assert a.seq_len(0) == b.seq_len(0) == T and a._stores[0].n_comp == b._stores[0].n_comp
    q1 = torch.randn(1, 8, 1, D, generator=g).half().cuda()
    k1 = torch.randn(1, 2, 1, D, generator=g).half().cuda()
    v1 = torch.randn(1, 2, 1, D, generator=g).half().cuda()
    assert torch.equal(a.attend(0, q1, k1, v1, rope=table[T]), b.attend(0, q1, k1, v1, rope=table[T]))
    # second chunk of 64 tokens on the non-empty cache
    q2 = torch.randn(1, 8, 64, D, generator=g).half().cuda()
    k2 = torch.randn(1, 2, 64, D, generator=g).half().cuda()
    v2 = torch.randn(1, 2, 64, D, generator=g).half().cuda()
    fk, fv = b.update(0, k2, v2)
    fk[:, :, -64:], fv[:, :, -64:] = k2, v2
    ref2 = ok.causal_attention(q2.float().cpu().numpy(), fk.float().cpu().numpy(), fv.float().cpu().numpy())
    out2 = a.prefill(0, q2, k2, v2)
    _bars_prefill(out2.float().cpu().numpy(), ref2, torch.float16)
    assert a.seq_len(0) == b.seq_len(0) == T + 1 + 64


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rope_kernel_bit_exact_on_strided_views(dtype, cuda_lib):
    """The prompt's rotary embedding in one launch (``apply_rope`` on 4-D CUDA tensors): on the q / k views of a fused
    q|k|v projection output (token-major rows, heads interleaved) it equals the fp32 restatement rounded to the dtype,
    bit for bit, and the element-wise torch formula it replaces."""
    from pare_b200.kv_cache import apply_rope, rope_table
    B, T, hq, hkv = 2, 70, 6, 2
    torch.manual_seed(4)
    qkv = torch.randn(B, T, (hq + 2 * hkv) * D, device="cuda").to(dtype)
    q = qkv[..., : hq * D].unflatten(2, (hq, D)).transpose(1, 2)
    k = qkv[..., hq * D:(hq + hkv) * D].unflatten(2, (hkv, D)).transpose(1, 2)
    table = rope_table(T + 5, D, 500000.0, device="cuda")
    rows = ok.rope_rows(np.arange(T + 5), D, 500000.0)
    off = torch.randn(B * hkv * T * D + 1, device="cuda").to(dtype)[1:].view(B, hkv, T, D)   # 2 bytes off: the scalar kernel
    assert off.data_ptr() % 16 != 0
    for x in (q, k, off):
        assert x is off or not x.is_contiguous()
        got = apply_rope(x, table[3:3 + T])
        assert got.shape == x.shape and got.dtype == dtype and got.is_contiguous()
        want = torch.from_numpy(ok.apply_rope(x.float().cpu().numpy(), rows[3:3 + T])).to(dtype)
        assert torch.equal(got.cpu(), want)
        half = D // 2
        cos, sin = table[3:3 + T, :half], table[3:3 + T, half:]
        a, b = x[..., :half].float(), x[..., half:].float()
        assert torch.equal(got, torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(dtype))
