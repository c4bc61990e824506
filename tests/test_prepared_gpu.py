"""Prepared activations (GPU): the hand-over format between the kernels of a decode step.

What is checked, and how tightly:
  * ``prepare`` + ``w4a16_forward_prepared`` is the M <= 16 path of ``w4a16_forward`` cut in two:
    bit-identical outputs;
  * RMSNorm / SwiGLU / attention writing prepared activations directly: the operand-order
    activations are bit-identical to ``prepare(plain output)``; the per-step sums are added in a
    different order (fp32), so they agree to 1e-5 relative and the linear's output to the oracle
    bars of test_w4a16_gpu.py (max rel <= 1e-2, mean <= 1e-3 fp16 / 2.5e-3 bf16);
  * a decode stack through the fused path vs the same stack through plain tensors: max rel <= 1e-2
    of the output scale, mean <= 1e-3 (fp16).
"""


import numpy as np
import pytest
import torch

from oracle import w4a16 as ow
from pare_b200.decode import DecodeStack
from pare_b200.kernels import _lib, w4a16_forward
from pare_b200.kernels.matmul_int4 import PreparedActivations, prepare, w4a16_forward_prepared
from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache

pytestmark = pytest.mark.gpu


def _layer(n, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    scale = torch.rand(n, k // 128, device="cuda", generator=g) * 0.01 + 0.001
    zero = torch.randint(0, 16, (n, k // 128), device="cuda", generator=g).float()
    return packed, scale, zero


def _split(prep):
    """(operand-order fp16 activations as int16, table (E, SX, g) as float32 [steps, rows, 3]) of a prepared buffer."""
    m, k = prep.rows, prep.k
    off = (m * k * 2 + 255) // 256 * 256
    xp = prep.buffer[: m * k * 2].view(torch.int16).reshape(m, k)
    tab = prep.buffer[off: off + (k // 128) * 16 * 16].view(torch.float32).reshape(k // 128, 16, 4)[:, :m, :3]
    return xp, tab


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (4, 28672, 4096), (16, 512, 1024), (3, 4096, 14336), (1, 9472, 3584), (2, 4096, 1792)])
def test_prepared_forward_is_the_plain_forward(m, n, k, dtype, cuda_lib):
    packed, scale, zero = _layer(n, k, seed=n + k)
    x = torch.randn(m, k, device="cuda").to(dtype)
    y_plain = w4a16_forward(x, packed, scale, zero, 128)
    y_prep = w4a16_forward_prepared(prepare(x), packed, scale, zero, 128)
    assert torch.equal(y_plain, y_prep)


def test_prepared_rejects_what_it_cannot_do(cuda_lib):
    with pytest.raises(ValueError):
        PreparedActivations(17, 1024, torch.float16, "cuda")
    with pytest.raises(ValueError):
        PreparedActivations(1, 1000, torch.float16, "cuda")
    packed, scale, zero = _layer(256, 640)          # K % 256 != 0: only the any-shape kernel serves it
    x = torch.randn(1, 640, device="cuda").half()
    with pytest.raises(_lib.KernelLibraryError):
        w4a16_forward_prepared(prepare(x), packed, scale, zero, 128)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,n", [(1, 4096), (4, 3584), (16, 1024)])
def test_rmsnorm_writes_prepared(rows, n, dtype, cuda_lib):
    L, code = cuda_lib, _lib.dtype_code(dtype)
    x = torch.randn(rows, n, device="cuda").to(dtype)
    delta = torch.randn(rows, n, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(n, device="cuda")).to(dtype)
    y = torch.empty_like(x)
    r1, r2 = torch.empty_like(x), torch.empty_like(x)
    s = _lib.current_stream(x.device)
    _lib.check(L.pare_rmsnorm_residual(x.data_ptr(), delta.data_ptr(), w.data_ptr(), r1.data_ptr(), y.data_ptr(), None,
                                       rows, n, 1e-5, code, s), "rmsnorm")
    prep = PreparedActivations(rows, n, dtype, "cuda")
    _lib.check(L.pare_rmsnorm_residual(x.data_ptr(), delta.data_ptr(), w.data_ptr(), r2.data_ptr(), None, prep.data_ptr(),
                                       rows, n, 1e-5, code, s), "rmsnorm")
    # the plain result against a torch fp32 reference of the same op (tolerance: one rounding of the output dtype)
    h = (x.float() + delta.float()).to(dtype).float()
    ref = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert torch.allclose(y.float(), ref, rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-3)
    assert torch.equal(r1, r2) and torch.equal(r1.float(), h)
    xp_a, tab_a = _split(prep)
    xp_b, tab_b = _split(prepare(y))
    assert torch.equal(xp_a, xp_b)
    assert torch.allclose(tab_a, tab_b, rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,n", [(1, 14336), (4, 1024)])
def test_silu_mul_writes_prepared(rows, n, dtype, cuda_lib):
    L, code = cuda_lib, _lib.dtype_code(dtype)
    gu = torch.randn(rows, 2 * n, device="cuda").to(dtype)
    out = torch.empty(rows, n, device="cuda", dtype=dtype)
    s = _lib.current_stream(gu.device)
    _lib.check(L.pare_silu_mul(gu.data_ptr(), out.data_ptr(), None, rows, n, 2 * n, code, s), "silu")
    prep = PreparedActivations(rows, n, dtype, "cuda")
    _lib.check(L.pare_silu_mul(gu.data_ptr(), None, prep.data_ptr(), rows, n, 2 * n, code, s), "silu")
    ref = torch.nn.functional.silu(gu[:, :n].float()) * gu[:, n:].float()
    assert torch.allclose(out.float(), ref, rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-3)
    xp_a, tab_a = _split(prep)
    xp_b, tab_b = _split(prepare(out))
    assert torch.equal(xp_a, xp_b)
    assert torch.allclose(tab_a, tab_b, rtol=1e-5, atol=1e-3)


def test_silu_mul_ragged_width(cuda_lib):
    """Widths that are not a multiple of 8 take the scalar path (no prepared output there)."""
    n = 1003
    gu = torch.randn(2, 2 * n + 3, device="cuda").half()[:, : 2 * n]
    out = torch.empty(2, n, device="cuda", dtype=torch.float16)
    _lib.check(cuda_lib.pare_silu_mul(gu.data_ptr(), out.data_ptr(), None, 2, n, gu.stride(0), _lib.F16,
                                      _lib.current_stream(gu.device)), "silu")
    ref = torch.nn.functional.silu(gu[:, :n].float()) * gu[:, n:].float()
    assert torch.allclose(out.float(), ref, rtol=2 ** -10, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_writes_prepared_and_appends(dtype, cuda_lib):
    bsz, hkv, hq, ctx, d = 2, 2, 8, 700, 128
    g = torch.Generator().manual_seed(11)
    k = torch.randn(bsz, hkv, ctx, d, generator=g).to(dtype).cuda()
    v = torch.randn(bsz, hkv, ctx, d, generator=g).to(dtype).cuda()
    q = torch.randn(bsz, hq, 1, d, generator=g).to(dtype).cuda()
    outs = []
    for fused in (False, True):
        cache = QuantizedKVCache(1, KVCacheConfig(bits=4, group_size=32, residual_length=128), max_seq_len=1024)
        cache.update(0, k[:, :, :-1], v[:, :, :-1])
        if fused:
            prep = PreparedActivations(bsz, hq * d, dtype, "cuda")
            assert cache.attend(0, q, k[:, :, -1:], v[:, :, -1:], prepared_out=prep) is None
            outs.append(prep)
        else:
            outs.append(cache.attend(0, q, k[:, :, -1:], v[:, :, -1:]))
        # the newest token is in the window whichever way it got there
        assert torch.equal(cache._residual_k[0][:, :, -1], k[:, :, -1])
        assert torch.equal(cache._residual_v[0][:, :, -1], v[:, :, -1])
    xp_a, tab_a = _split(outs[1])
    xp_b, tab_b = _split(prepare(outs[0].reshape(bsz, hq * d)))
    assert torch.equal(xp_a, xp_b)
    assert torch.allclose(tab_a, tab_b, rtol=1e-5, atol=1e-3)


def test_decode_stack_fused_equals_plain(cuda_lib, monkeypatch):
    """Two blocks of a small Llama-shaped stack, M = 2: hand-over through prepared activations vs plain tensors."""
    shape = (1024, 2048, 8, 2, 128, 2)

    def run(fused):
        torch.manual_seed(0)
        stack = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3)
        if not fused:
            for blk in stack.blocks:
                for lin in (blk.qkv, blk.o, blk.gate_up, blk.down):
                    monkeypatch.setattr(lin, "supports_prepared", lambda rows: False)
        stack.prefill_cache(2, 224)
        x = torch.randn(2, 1024, generator=torch.Generator().manual_seed(5)).half().cuda()
        y = None
        for _ in range(3):
            y = stack(x)
        return y.float().cpu().numpy()

    a, b = run(True), run(False)
    mx, mean = ow.rel_err(a, b)
    assert mx <= 1e-2 and mean <= 1e-3, (mx, mean)
    assert np.isfinite(a).all()


# ---- activations computed inside the streaming kernel ------------------------------------------

def _oracle_linear(x16, packed, scale, zero):
    return ow.linear(x16.float().cpu().numpy(), packed.cpu().numpy(), scale.cpu().numpy(), zero.cpu().numpy())


def _bars(y, ref, dtype):
    mx, mean = ow.rel_err(y.float().cpu().numpy(), ref)
    assert mx <= 1e-2 and mean <= (2.5e-3 if dtype == torch.bfloat16 else 1e-3), (mx, mean)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 1024, 1024), (4, 6144, 4096), (2, 9472, 1024), (1, 28672, 4096), (8, 1024, 1024)])
def test_linear_normalises_its_input_itself(m, n, k, dtype, cuda_lib):
    """rmsnorm(x + delta) * w -> linear in one launch (tile kernel, persistent kernel, and M = 8 through the
    stand-alone kernel) against the oracle on the fp32 reference of the norm rounded to the activation dtype;
    the new residual stream is exact."""
    from pare_b200.kernels.matmul_int4 import w4a16_forward_produced
    packed, scale, zero = _layer(n, k, seed=n + k + m)
    x = torch.randn(m, k, device="cuda").to(dtype)
    delta = torch.randn(m, k, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(k, device="cuda")).to(dtype)
    resid = torch.empty_like(x)
    y = w4a16_forward_produced(_lib.PRODUCER_RMSNORM, x, packed, scale, zero, 128, delta=delta, norm_weight=w,
                               resid_out=resid, eps=1e-5)
    h = (x.float() + delta.float()).to(dtype)
    assert torch.equal(resid, h)
    hn = (h.float() * torch.rsqrt((h.float() ** 2).mean(-1, keepdim=True) + 1e-5) * w.float()).to(dtype)
    _bars(y, _oracle_linear(hn, packed, scale, zero), dtype)
    # without a delta and without storing the stream
    y0 = w4a16_forward_produced(_lib.PRODUCER_RMSNORM, h, packed, scale, zero, 128, norm_weight=w, eps=1e-5)
    _bars(y0, _oracle_linear(hn, packed, scale, zero), dtype)
    y1 = w4a16_forward_produced(_lib.PRODUCER_RMSNORM, x, packed, scale, zero, 128, delta=delta, norm_weight=w,
                                resid_out=resid, eps=1e-5)
    assert torch.equal(y, y1)   # deterministic


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 1024, 2048), (3, 4096, 14336), (1, 10240, 1024), (6, 512, 1024), (2, 4096, 1792)])
def test_linear_applies_the_swiglu_gate_itself(m, n, k, dtype, cuda_lib):
    from pare_b200.kernels.matmul_int4 import w4a16_forward_produced
    packed, scale, zero = _layer(n, k, seed=n + k + m)
    gu = torch.randn(m, 2 * k + 8, device="cuda").to(dtype)[:, : 2 * k]     # a row stride larger than 2 K
    y = w4a16_forward_produced(_lib.PRODUCER_SILU_MUL, gu, packed, scale, zero, 128)
    act = (torch.nn.functional.silu(gu[:, :k].float()) * gu[:, k:].float()).to(dtype)
    _bars(y, _oracle_linear(act, packed, scale, zero), dtype)
    assert torch.equal(y, w4a16_forward_produced(_lib.PRODUCER_SILU_MUL, gu, packed, scale, zero, 128))


def test_produced_rejects_aliasing_and_odd_shapes(cuda_lib):
    from pare_b200.kernels.matmul_int4 import w4a16_forward_produced
    packed, scale, zero = _layer(256, 640)
    x = torch.randn(1, 640, device="cuda").half()
    w = torch.ones(640, device="cuda").half()
    with pytest.raises(_lib.KernelLibraryError):     # K % 512 != 0
        w4a16_forward_produced(_lib.PRODUCER_RMSNORM, x, packed, scale, zero, 128, norm_weight=w)
    packed, scale, zero = _layer(256, 1024)
    x = torch.randn(1, 1024, device="cuda").half()
    with pytest.raises(AssertionError):              # the stream must not be normalised in place
        w4a16_forward_produced(_lib.PRODUCER_RMSNORM, x, packed, scale, zero, 128, norm_weight=torch.ones(1024, device="cuda").half(),
                               resid_out=x)


def test_decode_stack_prefill_equals_token_by_token(cuda_lib):
    """A 72-token prompt (shorter than the residual window, so nothing is compressed and both routes see the same
    keys) through ``prefill()`` -- tensor-core linears, prefill attention -- against the same tokens fed one decode step
    at a time: hidden states within the kernels' tolerance, and the decode step that follows agrees too."""
    shape = (1024, 2048, 8, 2, 128, 2)
    T = 72
    x = torch.randn(1, T, 1024, generator=torch.Generator().manual_seed(11)).half().cuda()
    a = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3)
    b = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3)
    ya = a.prefill(x)
    yb = torch.cat([b(x[:, t]) for t in range(T)], dim=0).view(1, T, 1024)
    assert a.cache.seq_len(0) == b.cache.seq_len(1) == T
    mx, mean = ow.rel_err(ya.float().cpu().numpy(), yb.float().cpu().numpy())
    assert mx <= 3e-2 and mean <= 3e-3, (mx, mean)           # two blocks of 16-bit round trips on either route
    ka, kb = a.cache._residual_k[1].float(), b.cache._residual_k[1].float()
    assert torch.allclose(ka, kb, rtol=2e-2, atol=2e-2)
    nxt = torch.randn(1, 1024, generator=torch.Generator().manual_seed(12)).half().cuda()
    mx, mean = ow.rel_err(a(nxt).float().cpu().numpy(), b(nxt).float().cpu().numpy())
    assert mx <= 3e-2 and mean <= 3e-3, (mx, mean)
    # chunked prefill continues the sequence
    c = DecodeStack(shape, dtype=torch.float16, max_seq_len=512, seed=3)
    yc = torch.cat([c.prefill(x[:, :40]), c.prefill(x[:, 40:])], dim=1)
    mx, mean = ow.rel_err(yc.float().cpu().numpy(), ya.float().cpu().numpy())
    assert mx <= 3e-2 and mean <= 3e-3, (mx, mean)


@pytest.mark.parametrize("m", [1, 3])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_stack_step_against_restatement(m, dtype, cuda_lib):
    """Two blocks of a small Llama-shaped stack, one decode step, against a restatement of the block written here
    from the oracle's pieces (not against the stack's other route): RMSNorm -> q|k|v linear -> rotary embedding of q
    and the new key -> KIVI cache update -> attention over the cache -> o linear -> residual add -> RMSNorm -> gate|up
    linear -> SwiGLU -> down linear -> residual add.  Catches wiring errors both routes of the stack would share
    (residual ping-pong, head slicing, rotary position).  Every stage is computed in fp32 from the previous stage's
    result rounded to the activation dtype, which is where the kernels round too; what is left is the kernels' own
    error, eleven stages deep: max <= 3e-2, mean <= 2e-3 for fp16, 1.5e-1 / 1e-2 for bf16 (8 significant bits)."""
    from oracle import kivi as ok
    shape = (1024, 2048, 8, 2, 128, 2)
    hidden, ffn, hq, hkv, d, layers = shape
    ctx = 224 + 5                                              # 96 compressed tokens + a window that is not full
    stack = DecodeStack(shape, dtype=dtype, max_seq_len=512, seed=3)
    g = torch.Generator().manual_seed(21)
    caches = []
    for layer in range(layers):
        k = torch.randn(m, hkv, ctx, d, generator=g)
        v = torch.randn(m, hkv, ctx, d, generator=g)
        k[..., 17] *= 10.0
        k, v = k.to(dtype), v.to(dtype)
        stack.cache._append(layer, k.cuda(), v.cuda())
        c = ok.Cache(4, 32, 128)
        c.update(k.float().numpy(), v.float().numpy())
        caches.append(c)
    for blk in stack.blocks:                                    # non-trivial norm weights
        blk.norm1.copy_((1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype))
        blk.norm2.copy_((1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype))
    x = torch.randn(m, hidden, generator=g).to(dtype)
    y = stack(x.cuda()).float().cpu().numpy()

    rows = stack.rope.cpu().numpy()
    pos = ctx
    r = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()   # round to the dtype

    def rms(h, w):
        return r(h / np.sqrt((h * h).mean(-1, keepdims=True) + 1e-5) * w)

    def lin(layer, a):
        n = layer.out_features
        return r(ow.linear(a, layer.packed_weight.cpu().numpy(), layer.scale.cpu().numpy().reshape(n, -1),
                           layer.zero.cpu().numpy().reshape(n, -1)))

    h = x.float().numpy()
    delta = None
    for i, blk in enumerate(stack.blocks):
        if delta is not None:
            h = r(h + delta)
        qkv = lin(blk.qkv, rms(h, blk.norm1.float().cpu().numpy()))
        q = qkv[:, : hq * d].reshape(m, hq, 1, d)
        k1 = qkv[:, hq * d:(hq + hkv) * d].reshape(m, hkv, 1, d)
        v1 = qkv[:, (hq + hkv) * d:].reshape(m, hkv, 1, d)
        q, k1 = r(ok.apply_rope(q, rows[pos])), r(ok.apply_rope(k1, rows[pos]))
        fk, fv = caches[i].update(k1, v1)
        attn = r(ok.decode_attention(q, fk, fv).reshape(m, hq * d))
        h = r(h + lin(blk.o, attn))
        gu = lin(blk.gate_up, rms(h, blk.norm2.float().cpu().numpy()))
        gate, up = gu[:, :ffn], gu[:, ffn:]
        delta = lin(blk.down, r(gate / (1 + np.exp(-gate)) * up))
    want = r(h + delta)
    mx, mean = ow.rel_err(y, want)
    print("stack vs restatement", dtype, m, mx, mean)
    # The error is measured relative to max(|want|, 1e-2 max|want|).  Every hand-over rounds to the dtype, so one
    # element that lands on the other side of a rounding boundary differs by one unit in the last place: 2^-11 of
    # its own size in fp16, 2^-8 in bf16, i.e. up to 2^-8 / 1e-2 = 0.39 in this measure for a bf16 element of the
    # largest size.  The maximum bar allows exactly that single flip; the mean bar is what holds the kernels.
    bars = (3e-2, 2e-3) if dtype == torch.float16 else (0.4, 1e-2)
    assert mx <= bars[0] and mean <= bars[1], (mx, mean)
    assert stack.cache.seq_len(0) == stack.cache.seq_len(1) == ctx + 1
