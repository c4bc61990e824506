"""The workspace-free W4A16 entry point (collected last on purpose).

``pare_w4a16_forward_static`` serves callers that cannot allocate device memory — for example a
plugin invoked from inside another runtime's callback, where ``cudaMalloc`` is off limits, or a
binding that is handed nothing but input and output pointers.  It must give exactly what the
regular entry point gives (same kernel, same deterministic reduction), also on a second call that
finds the shared scratch array as the first one left it, and it must refuse layers that do not fit.
"""

import pytest
import torch
import torch.nn as nn

from pare_b200.config import QuantConfig
from pare_b200.kernels import _lib
from pare_b200.kernels.matmul_int4 import w4a16_forward
from pare_b200.layers.linear import QuantizedLinear

pytestmark = pytest.mark.gpu


def _layer(n, k, seed):
    torch.manual_seed(seed)
    ql = QuantizedLinear.from_linear(nn.Linear(k, n, bias=True), QuantConfig(bits=4, scheme="rtn", group_size=128))
    return ql.cuda()


def _static_forward(x, ql, bias):
    L = _lib.lib()
    n, k = ql.out_features, ql.in_features
    y = torch.empty(x.shape[0], n, device=x.device, dtype=x.dtype)
    scale = ql.scale.squeeze(-1).contiguous()
    zero = ql.zero.squeeze(-1).contiguous()
    status = L.pare_w4a16_forward_static(
        x.data_ptr(), _lib.dtype_code(x.dtype), x.stride(0), ql.packed_weight.data_ptr(),
        scale.data_ptr(), zero.data_ptr(), None, None, None, bias.data_ptr(),
        y.data_ptr(), y.stride(0), x.shape[0], n, k, 128, _lib.current_stream(x.device))
    torch.cuda.synchronize()
    return status, y


def test_static_entry_matches_regular_entry_twice(cuda_lib):
    # K = 14336 goes through the split-K reduction, i.e. through the counters in the shared array
    for (n, k, m, dtype) in ((1024, 4096, 1, torch.float16), (4096, 14336, 4, torch.bfloat16)):
        ql = _layer(n, k, seed=n + m)
        bias = ql.bias.detach().to(dtype)
        x = torch.randn(m, k, device="cuda", dtype=dtype)
        want = w4a16_forward(x, ql.packed_weight, ql.scale.squeeze(-1).contiguous(), ql.zero.squeeze(-1).contiguous(),
                             128, bias=bias)
        for call in range(2):                         # two calls in a row share the scratch array
            status, got = _static_forward(x, ql, bias)
            assert status == 0, (call, status)
            assert torch.equal(got, want), (n, k, m, call)   # same kernel, deterministic: bit-identical


def test_static_entry_rejects_what_does_not_fit(cuda_lib):
    L = _lib.lib()
    assert L.pare_w4a16_static_scratch_bytes() == 16 << 20
    ql = _layer(256, 512, seed=1)
    x = torch.randn(17, 512, device="cuda", dtype=torch.float16)
    status, _ = _static_forward(x, ql, ql.bias.detach().half())
    assert status == 5                                # M > 16: unsupported by this entry point
    # a layer whose scratch need exceeds the fixed array is refused before anything is launched
    big_n, big_k = 65536, 8192
    assert L.pare_w4a16_workspace_bytes(16, big_n, big_k, 128) > L.pare_w4a16_static_scratch_bytes()
    dummy = torch.empty(16, device="cuda", dtype=torch.uint8)
    status = L.pare_w4a16_forward_static(
        dummy.data_ptr(), 0, big_k, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, None, None, None,
        dummy.data_ptr(), big_n, 16, big_n, big_k, 128, _lib.current_stream(dummy.device))
    assert status == 4                                # PARE_ERR_WORKSPACE


def _static_call(x, ql, *, bias=None, meta_h2=None, col_perm=None, input_scale=None, group=128, sync=True):
    L = _lib.lib()
    n, k = ql.out_features, ql.in_features
    y = torch.empty(x.shape[0], n, device=x.device, dtype=x.dtype)
    scale = ql.scale.reshape(n, -1).contiguous()
    zero = ql.zero.reshape(n, -1).contiguous()
    status = L.pare_w4a16_forward_static(
        x.data_ptr(), _lib.dtype_code(x.dtype), x.stride(0), ql.packed_weight.data_ptr(),
        scale.data_ptr(), zero.data_ptr(), _lib.ptr(meta_h2), _lib.ptr(col_perm), _lib.ptr(input_scale), _lib.ptr(bias),
        y.data_ptr(), y.stride(0), x.shape[0], n, k, group, _lib.current_stream(x.device))
    if sync:
        torch.cuda.synchronize()
    return status, y, (scale, zero)


def test_static_entry_other_paths_bit_identical(cuda_lib):
    """The cases the two fast-path shapes above do not reach, each bit-identical to the regular entry point: the generic
    kernel (K % 256 != 0, which needs no scratch), a layer with an activation-order column permutation and a run-time
    input scale, packed half2 metadata, and the full 16 rows."""
    from pare_b200.kernels.matmul_int4 import pack_meta_h2
    g = torch.Generator(device="cuda").manual_seed(3)
    # generic path: K = 384 (not a multiple of 256), group 128
    ql = _layer(192, 384, seed=5)
    x = torch.randn(3, 384, device="cuda", dtype=torch.float16, generator=g)
    want = w4a16_forward(x, ql.packed_weight, ql.scale.reshape(192, -1).contiguous(), ql.zero.reshape(192, -1).contiguous(), 128)
    status, got, _ = _static_call(x, ql)
    assert status == 0 and torch.equal(got, want)
    # column permutation + input scale, M = 16, bf16
    ql = _layer(2048, 4096, seed=6)
    perm = torch.randperm(4096, generator=torch.Generator().manual_seed(1)).to(torch.int32).cuda()
    insc = (0.5 + torch.rand(4096, generator=torch.Generator().manual_seed(2))).cuda()
    x = torch.randn(16, 4096, device="cuda", dtype=torch.bfloat16, generator=g)
    sc, ze = ql.scale.reshape(2048, -1).contiguous(), ql.zero.reshape(2048, -1).contiguous()
    want = w4a16_forward(x, ql.packed_weight, sc, ze, 128, col_perm=perm, input_scale=insc)
    status, got, _ = _static_call(x, ql, col_perm=perm, input_scale=insc)
    assert status == 0 and torch.equal(got, want)
    # packed half2 metadata
    x = torch.randn(2, 4096, device="cuda", dtype=torch.float16, generator=g)
    h2 = pack_meta_h2(sc, ze)
    want = w4a16_forward(x, ql.packed_weight, sc, ze, 128, meta_h2=h2)
    status, got, _ = _static_call(x, ql, meta_h2=h2)
    assert status == 0 and torch.equal(got, want)
    assert _lib.lib().pare_w4a16_static_status(_lib.current_stream(x.device)) == 0


def test_static_entry_alternating_layers_queued_on_one_stream(cuda_lib):
    """The sharing case: two different layers take turns on one stream, 12 calls queued with no host synchronisation in
    between (consecutive calls overlap through programmatic dependent launch), one synchronise at the end; every
    result equals the regular entry point's bit for bit and the scratch's status word stays clean."""
    a, b = _layer(4096, 4096, seed=11), _layer(1024, 14336, seed=12)   # tile kernel / persistent split-K kernel
    g = torch.Generator(device="cuda").manual_seed(9)
    xa = [torch.randn(1 + i % 4, 4096, device="cuda", dtype=torch.float16, generator=g) for i in range(6)]
    xb = [torch.randn(1 + i % 3, 14336, device="cuda", dtype=torch.float16, generator=g) for i in range(6)]
    want = []
    for i in range(6):
        want.append(w4a16_forward(xa[i], a.packed_weight, a.scale.reshape(4096, -1).contiguous(), a.zero.reshape(4096, -1).contiguous(), 128))
        want.append(w4a16_forward(xb[i], b.packed_weight, b.scale.reshape(1024, -1).contiguous(), b.zero.reshape(1024, -1).contiguous(), 128))
    torch.cuda.synchronize()
    got, keep = [], []
    for i in range(6):
        for x, ql in ((xa[i], a), (xb[i], b)):
            status, y, tensors = _static_call(x, ql, sync=False)
            assert status == 0
            got.append(y)
            keep.append(tensors)
    torch.cuda.synchronize()
    for i, (y, w) in enumerate(zip(got, want)):
        assert torch.equal(y, w), i
    assert _lib.lib().pare_w4a16_static_status(_lib.current_stream(xa[0].device)) == 0


def test_bounded_wait_times_out_and_reports(cuda_lib):
    """A wait that nothing ends returns after its poll limit and leaves the time-out code in the workspace's status
    word; reading the word clears it, and the workspace then serves a normal call."""
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = _lib.workspace(dev, 1 << 20)
    stream = _lib.current_stream(dev)
    assert L.pare_workspace_status(ws.data_ptr(), stream) == 0
    assert L.pare_selftest_bounded_wait(ws.data_ptr(), 64, stream) == 0
    assert L.pare_workspace_status(ws.data_ptr(), stream) == 7        # PARE_ERR_TIMEOUT
    assert L.pare_workspace_status(ws.data_ptr(), stream) == 0        # read once, cleared
    assert L.pare_selftest_bounded_wait(ws.data_ptr(), 5000, stream) == 1   # PARE_ERR_SHAPE: only short waits are accepted
    ql = _layer(512, 1024, seed=2)
    x = torch.randn(2, 1024, device="cuda", dtype=torch.float16)
    y = ql(x)
    assert torch.isfinite(y).all() and _lib.workspace_status(dev) == 0
