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
