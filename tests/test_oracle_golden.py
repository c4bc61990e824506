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
