"""W4A16 fused dequantize-matmul — Python face of the CUDA kernels.

Drop-in for the reference's ``pare/kernels/matmul_int4.py``:

* :func:`matmul_w4a16` keeps the reference signature and semantics
  (``pare/kernels/matmul_int4.py:183-243``): fp16 activations ``[M, K]``, weights in the
  *kernel layout* of ``repack_int4_for_kernel``, fp16 result.  The CUDA kernels read the
  storage layout, so the kernel-layout argument is converted back once per tensor and
  cached.
* :func:`w4a16_forward` is the entry ``QuantizedLinear`` uses: storage-layout weights,
  fp16 or bf16 activations, optional bias / act-order column permutation / run-time
  input scale, all handled inside the kernel.
* :func:`triton_available` is kept by name for callers that gate on it; it now reports
  whether the CUDA library and a GPU are present.  Nothing here uses Triton and there is
  no CPU implementation behind these functions.
"""

from __future__ import annotations

import weakref

import torch
from torch import Tensor

from pare_b200.core.pack import unrepack_int4_from_kernel
from pare_b200.kernels import _lib


def kernel_available() -> bool:
    """True when libpare_b200.so is built and a CUDA device is visible."""
    return _lib.available()


def triton_available() -> bool:
    """Name kept from the reference (``pare/kernels/matmul_int4.py:246-248``)."""
    return kernel_available()


def _meta_2d(t: Tensor, n: int) -> Tensor:
    """Scale / zero in any of the reference's shapes → contiguous fp32 ``[N, groups]``."""
    t = t.float()
    if t.dim() == 0:
        t = t.reshape(1, 1).expand(n, 1)
    elif t.dim() == 1:
        t = t.unsqueeze(1)
    elif t.dim() == 3:
        t = t.squeeze(2)
    return t.contiguous()


def pack_meta_h2(scale: Tensor, zero: Tensor) -> Tensor:
    """Interleave fp16 (scale, zero) pairs into one int32 word per (row, group)."""
    s = scale.to(torch.float16).contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    z = zero.to(torch.float16).contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    return (s | (z << 16)).to(torch.int32).contiguous()


def w4a16_forward(
    x: Tensor,
    packed_weight: Tensor,
    scale: Tensor,
    zero: Tensor,
    group_size: int,
    *,
    bias: Tensor | None = None,
    col_perm: Tensor | None = None,
    input_scale: Tensor | None = None,
    meta_h2: Tensor | None = None,
    out: Tensor | None = None,
) -> Tensor:
    """``x [M, K] @ dequant(packed_weight [N, K/2]).T (+ bias)`` on the GPU.

    ``scale`` / ``zero`` are fp32 ``[N, K/group_size]`` (already 2-D and contiguous);
    ``meta_h2`` (from :func:`pack_meta_h2`) replaces them when given.  ``x`` may have a row
    stride larger than K.  The result has the dtype of ``x``.
    """
    if not x.is_cuda:
        raise RuntimeError("w4a16_forward requires CUDA tensors.")
    assert x.dim() == 2 and x.stride(1) == 1, "x must be [M, K] with unit inner stride"
    m, k = x.shape
    n, k_half = packed_weight.shape
    assert k == 2 * k_half, f"packed_weight has {k_half} columns, expected K//2={k // 2}"
    assert packed_weight.dtype == torch.uint8 and packed_weight.is_contiguous()
    if m == 0:
        return x.new_empty(0, n)
    code = _lib.dtype_code(x.dtype)
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    y = out if out is not None else torch.empty(m, n, device=x.device, dtype=x.dtype)
    L = _lib.lib()
    ws_bytes = L.pare_w4a16_workspace_bytes(m, n, k, group_size)
    ws = _lib.workspace(x.device, ws_bytes)
    status = L.pare_w4a16_forward(
        x.data_ptr(), code, x.stride(0),
        packed_weight.data_ptr(),
        _lib.ptr(scale), _lib.ptr(zero), _lib.ptr(meta_h2),
        _lib.ptr(col_perm), _lib.ptr(input_scale), _lib.ptr(bias),
        y.data_ptr(), y.stride(0),
        m, n, k, group_size,
        ws.data_ptr(), ws.numel(),
        _lib.current_stream(x.device),
    )
    _lib.check(status, "pare_w4a16_forward")
    return y


class PreparedActivations:
    """Activations of a W4A16 linear in the order its decode kernel consumes them.

    An opaque device buffer for ``rows <= 16`` activation rows of ``k`` columns (``k % 128 == 0``)
    of ``dtype``.  Kernels that compute an activation (RMSNorm, SwiGLU, the fused decode
    attention) can write into it directly; :func:`prepare` fills it from a plain tensor.
    """

    def __init__(self, rows: int, k: int, dtype: torch.dtype, device) -> None:
        nbytes = _lib.lib().pare_w4a16_prepared_bytes(rows, k)
        if nbytes == 0:
            raise ValueError(f"prepared activations need rows <= 16 and k % 128 == 0 (got {rows} x {k})")
        self.rows, self.k, self.dtype = rows, k, dtype
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def data_ptr(self) -> int:
        return self.buffer.data_ptr()


def prepare(x: Tensor, *, col_perm: Tensor | None = None, input_scale: Tensor | None = None,
            out: PreparedActivations | None = None) -> PreparedActivations:
    """Put ``x [M, K]`` (M <= 16) into operand order (what every M <= 16 ``w4a16_forward`` does first)."""
    assert x.is_cuda and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    prep = out if out is not None else PreparedActivations(m, k, x.dtype, x.device)
    assert (prep.rows, prep.k, prep.dtype) == (m, k, x.dtype)
    status = _lib.lib().pare_w4a16_prepare(x.data_ptr(), _lib.dtype_code(x.dtype), x.stride(0), _lib.ptr(col_perm),
                                           _lib.ptr(input_scale), m, k, prep.data_ptr(), _lib.current_stream(x.device))
    _lib.check(status, "pare_w4a16_prepare")
    return prep


def w4a16_forward_prepared(prep: PreparedActivations, packed_weight: Tensor, scale: Tensor | None, zero: Tensor | None,
                           group_size: int, *, bias: Tensor | None = None, meta_h2: Tensor | None = None,
                           out: Tensor | None = None, peer=None) -> Tensor:
    """:func:`w4a16_forward` for activations that already are in operand order.  ``peer`` (a
    :class:`pare_b200.parallel.PeerAllReduce`): the layer is a row-parallel shard and the result is the sum over the
    ranks, added inside the kernel's epilogue."""
    n, k_half = packed_weight.shape
    assert prep.k == 2 * k_half and packed_weight.dtype == torch.uint8 and packed_weight.is_contiguous()
    m, k = prep.rows, prep.k
    if bias is not None and bias.dtype != prep.dtype:
        bias = bias.to(prep.dtype)
    dev = packed_weight.device
    y = out if out is not None else torch.empty(m, n, device=dev, dtype=prep.dtype)
    L = _lib.lib()
    ws = _lib.workspace(dev, L.pare_w4a16_workspace_bytes(m, n, k, group_size))
    if peer is not None:
        status = L.pare_w4a16_forward_prepared_allreduce(
            prep.data_ptr(), _lib.dtype_code(prep.dtype), packed_weight.data_ptr(),
            _lib.ptr(scale), _lib.ptr(zero), _lib.ptr(meta_h2), _lib.ptr(bias),
            y.data_ptr(), y.stride(0), m, n, k, group_size, ws.data_ptr(), ws.numel(),
            peer.rank, peer.world, peer._ptrs, peer.buffer_bytes, _lib.current_stream(dev))
        _lib.check(status, "pare_w4a16_forward_prepared_allreduce")
        return y
    status = L.pare_w4a16_forward_prepared(
        prep.data_ptr(), _lib.dtype_code(prep.dtype), packed_weight.data_ptr(),
        _lib.ptr(scale), _lib.ptr(zero), _lib.ptr(meta_h2), _lib.ptr(bias),
        y.data_ptr(), y.stride(0), m, n, k, group_size, ws.data_ptr(), ws.numel(), _lib.current_stream(dev))
    _lib.check(status, "pare_w4a16_forward_prepared")
    return y


def w4a16_forward_produced(producer: int, a: Tensor, packed_weight: Tensor, scale: Tensor | None, zero: Tensor | None,
                           group_size: int, *, delta: Tensor | None = None, norm_weight: Tensor | None = None,
                           resid_out: Tensor | None = None, eps: float = 1e-5, bias: Tensor | None = None,
                           meta_h2: Tensor | None = None, out: Tensor | None = None, peer=None) -> Tensor:
    """The linear with its activations computed inside the streaming kernel (M <= 16).

    ``producer = _lib.PRODUCER_RMSNORM``: ``x = rmsnorm(a + delta) * norm_weight`` (``a [M, K]``; ``a + delta`` is
    stored to ``resid_out``, which must not be ``a``).  ``producer = _lib.PRODUCER_SILU_MUL``:
    ``x = silu(a[:, :K]) * a[:, K:2K]`` for a fused gate|up tensor ``a [M, >= 2K]``.
    """
    n, k_half = packed_weight.shape
    k = 2 * k_half
    m = a.shape[0]
    assert a.is_cuda and a.dim() == 2 and a.stride(1) == 1 and packed_weight.is_contiguous()
    if producer == _lib.PRODUCER_RMSNORM:
        assert a.shape[1] == k and norm_weight is not None and norm_weight.dtype == a.dtype
        assert delta is None or (delta.shape == a.shape and delta.stride() == a.stride() and delta.dtype == a.dtype)
        assert resid_out is None or (resid_out.shape == a.shape and resid_out.stride() == a.stride()
                                     and resid_out.data_ptr() != a.data_ptr())
    else:
        assert a.shape[1] >= 2 * k
    if bias is not None and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    y = out if out is not None else torch.empty(m, n, device=a.device, dtype=a.dtype)
    L = _lib.lib()
    ws = _lib.workspace(a.device, L.pare_w4a16_workspace_bytes(m, n, k, group_size))
    if peer is not None:   # row-parallel shard: the sum over the ranks is added inside the kernel
        status = L.pare_w4a16_forward_produced_allreduce(
            producer, a.data_ptr(), _lib.ptr(delta), _lib.ptr(norm_weight), _lib.ptr(resid_out), a.stride(0), float(eps),
            _lib.dtype_code(a.dtype), packed_weight.data_ptr(), _lib.ptr(scale), _lib.ptr(zero), _lib.ptr(meta_h2), _lib.ptr(bias),
            y.data_ptr(), y.stride(0), m, n, k, group_size, ws.data_ptr(), ws.numel(),
            peer.rank, peer.world, peer._ptrs, peer.buffer_bytes, _lib.current_stream(a.device))
        _lib.check(status, "pare_w4a16_forward_produced_allreduce")
        return y
    status = L.pare_w4a16_forward_produced(
        producer, a.data_ptr(), _lib.ptr(delta), _lib.ptr(norm_weight), _lib.ptr(resid_out), a.stride(0), float(eps),
        _lib.dtype_code(a.dtype), packed_weight.data_ptr(), _lib.ptr(scale), _lib.ptr(zero), _lib.ptr(meta_h2), _lib.ptr(bias),
        y.data_ptr(), y.stride(0), m, n, k, group_size, ws.data_ptr(), ws.numel(), _lib.current_stream(a.device))
    _lib.check(status, "pare_w4a16_forward_produced")
    return y


# kernel-layout tensor (as passed by reference-style callers) -> storage layout, cached per tensor
# object: keyed by id() (tensors do not hash/compare as dict keys) and dropped when it dies
_storage_cache: dict[int, tuple[int, int, Tensor]] = {}


def _storage_layout(kernel_layout: Tensor, group_size: int) -> Tensor:
    key = id(kernel_layout)
    hit = _storage_cache.get(key)
    if hit is not None and hit[0] == kernel_layout._version and hit[1] == group_size:
        return hit[2]
    storage = unrepack_int4_from_kernel(kernel_layout, group_size).contiguous()
    if hit is None:
        weakref.finalize(kernel_layout, _storage_cache.pop, key, None)
    _storage_cache[key] = (kernel_layout._version, group_size, storage)
    return storage


def matmul_w4a16(x: Tensor, packed_weight: Tensor, scales: Tensor, zeros: Tensor, group_size: int) -> Tensor:
    """Reference-compatible entry: ``packed_weight`` is in the *kernel layout*.

    Raises ``RuntimeError`` when the CUDA library is missing or ``x`` is not a CUDA tensor,
    ``AssertionError`` for non-contiguous / non-fp16 ``x`` or a K mismatch — the same
    conditions as the reference wrapper.
    """
    if not _lib.LIB_PATH.exists():
        raise RuntimeError("libpare_b200.so is not built. Run `python -m pare_b200.build`.")
    if not x.is_cuda:
        raise RuntimeError("matmul_w4a16 requires CUDA tensors.")
    assert x.is_contiguous(), "x must be contiguous"
    assert x.dtype == torch.float16, f"x must be float16, got {x.dtype}"
    m, k = x.shape
    n, k_half = packed_weight.shape
    assert k == k_half * 2, f"packed_weight has {k_half} columns, expected K//2={k // 2}"

    storage = _storage_layout(packed_weight, group_size)
    return w4a16_forward(x, storage, _meta_2d(scales, n), _meta_2d(zeros, n), group_size)
