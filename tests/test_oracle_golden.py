"""Pin the CPU oracle against outputs of the reference itself (committed fixtures)."""

import numpy as np

from oracle import kivi, w4a16


def test_w4a16_per_group_matches_reference(golden):
    g = golden("w4a16_g128.npz")
    w = w4a16.dequantize(g["packed"], g["scale"], g["zero"])
    assert np.array_equal(w, g["w"])                      # same fp32 formula -> bit-exact
    y = w4a16.linear(g["x"], g["packed"], g["scale"], g["zero"])
    assert np.allclose(y, g["y"], rtol=0, atol=2e-5)      # only the GEMM summation order differs


def test_w4a16_per_channel_bias_matches_reference(golden):
    g = golden("w4a16_channel.npz")
    w = w4a16.dequantize(g["packed"], g["scale"], g["zero"])
    assert np.array_equal(w, g["w"])
    y = w4a16.linear(g["x"], g["packed"], g["scale"], g["zero"], bias=g["bias"])
    assert np.allclose(y, g["y"], rtol=0, atol=2e-5)


def test_identity_g_idx_is_plain_dequantize(golden):
    g = golden("w4a16_g128.npz")
    k = g["packed"].shape[1] * 2
    idx = np.arange(k) // 128
    assert np.array_equal(w4a16.dequantize(g["packed"], g["scale"], g["zero"], g_idx=idx), g["w"])


def test_pack_roundtrip():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(5, 64), dtype=np.int32)
    assert np.array_equal(w4a16.unpack_int4(w4a16.pack_int4(q)), q)
    assert w4a16.pack_int4(np.arange(8)[None]).view("<u4")[0, 0] == 0x76543210


def test_kivi_primitives_bit_exact(golden):
    g = golden("kivi_prims.npz")
    for bits in (2, 4, 8):
        kq, ks, kz = kivi.quantize_keys(g["k"].astype(np.float32), bits, 32)
        vq, vs, vz = kivi.quantize_values(g["v"].astype(np.float32), bits, 32)
        for name, got in (("kq", kq), ("ks", ks), ("kz", kz), ("vq", vq), ("vs", vs), ("vz", vz)):
            assert np.array_equal(got, g[f"{name}{bits}"]), (name, bits)


def test_kivi_cache_sequence_matches_reference(golden):
    g = golden("kivi_cache.npz")
    cache = kivi.Cache(bits=4, group_size=32, residual_length=64)
    counts = []
    fk, fv = cache.update(g["k_all"][:, :, :96], g["v_all"][:, :, :96])
    counts.append((cache.n_comp, cache.n_res))
    for t in range(96, g["k_all"].shape[2]):
        fk, fv = cache.update(g["k_all"][:, :, t:t + 1], g["v_all"][:, :, t:t + 1])
        counts.append((cache.n_comp, cache.n_res))
    assert np.array_equal(np.array(counts), g["counts"])
    assert np.array_equal(fk.astype(np.float16), g["full_k"])
    assert np.array_equal(fv.astype(np.float16), g["full_v"])
    attn = kivi.decode_attention(g["q"], fk.astype(np.float16), fv.astype(np.float16))
    assert np.allclose(attn, g["attn"], rtol=0, atol=2e-6)


def test_kivi_dequant_roundtrip_error_bound():
    rng = np.random.default_rng(1)
    k = rng.standard_normal((1, 2, 64, 128)).astype(np.float32)
    q, s, z = kivi.quantize_keys(k, 4, 32)
    rec = kivi.dequantize_keys(q, s, z, 32)
    assert np.abs(rec - k).max() <= 0.5 * s.max() * (1 + 1e-5)


def test_value_channel_groups_restatement():
    """``quantize_values(.., v_group)`` is the reference's per-token function on the channel axis viewed as
    [D/v_group][v_group]: each group's codes / scale / zero equal the whole-row function applied to that slice."""
    import numpy as np
    from oracle import kivi as ok
    rng = np.random.default_rng(3)
    v = rng.standard_normal((2, 3, 64, 128)).astype(np.float32)
    for bits in (2, 4, 8):
        q, s, z = ok.quantize_values(v, bits, 32, 32)
        assert q.shape == v.shape and s.shape == (2, 3, 64, 4) and z.shape == s.shape
        for g in range(4):
            qg, sg, zg = ok.quantize_values(v[..., g * 32:(g + 1) * 32], bits, 32)
            assert np.array_equal(q[..., g * 32:(g + 1) * 32], qg)
            assert np.array_equal(s[..., g:g + 1], sg) and np.array_equal(z[..., g:g + 1], zg)
        whole = ok.quantize_values(v, bits, 32)
        for a, b in zip(whole, ok.quantize_values(v, bits, 32, 128)):
            assert np.array_equal(a, b)
        rec = ok.dequantize_values(q, s, z)
        assert np.abs(rec - v).max() <= np.abs(ok.dequantize_values(*whole) - v).max() + 1e-6


def test_timed_cpu_path_agrees_with_the_pinned_oracle():
    """``oracle/cpu_path.py`` (the torch op sequence the benchmark TIMES on the host) computes what the pinned numpy
    oracle computes: the linear within fp32 summation order (1e-5 relative), the cache bit for bit over a sequence of
    updates that crosses the residual boundary several times (codes are integers, the reconstruction is one fused
    multiply-add per element in both), attention within 1e-4."""
    import torch

    from oracle import cpu_path

    rng = np.random.default_rng(3)
    n, k, g = 96, 256, 128
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scale = (0.01 + rng.random((n, k // g, 1))).astype(np.float32)
    zero = rng.integers(0, 16, size=(n, k // g, 1)).astype(np.float32)
    x = rng.standard_normal((5, k)).astype(np.float32)
    want = w4a16.linear(x, packed, scale[..., 0], zero[..., 0])
    got = cpu_path.linear_forward(torch.from_numpy(x), torch.from_numpy(packed), torch.from_numpy(scale), torch.from_numpy(zero)).numpy()
    mx, _ = w4a16.rel_err(got, want)
    assert mx <= 1e-5, mx

    ref, tim = kivi.Cache(4, 32, 128), cpu_path.TorchCache(4, 32, 128)
    for t in (100, 60, 1, 1, 97, 1):
        kk = rng.standard_normal((2, 2, t, 128)).astype(np.float32)
        vv = rng.standard_normal((2, 2, t, 128)).astype(np.float32)
        rk, rv = ref.update(kk, vv)
        tk, tv = tim.update(torch.from_numpy(kk), torch.from_numpy(vv))
        assert tk.shape == rk.shape and tv.shape == rv.shape
        np.testing.assert_allclose(tk.numpy(), rk, rtol=0, atol=1e-6)   # same codes; q * scale + zero within an ulp
        np.testing.assert_allclose(tv.numpy(), rv, rtol=0, atol=1e-6)
    q = rng.standard_normal((2, 4, 1, 128)).astype(np.float32)
    a_ref = kivi.decode_attention(q, rk, rv)
    a_tim = cpu_path.attention(torch.from_numpy(q), tk, tv).numpy()
    mx, _ = w4a16.rel_err(a_tim, a_ref)
    assert mx <= 1e-4, mx   # fp32 softmax and sums in another order (measured 3e-5)
