"""``QuantizedLinear`` — quantized stand-in for ``nn.Linear`` with a CUDA fast path.

Same constructor, buffers, class methods and dispatch rule as the reference's
``pare/layers/linear.py:40-281``:

* buffers ``packed_weight`` (uint8 ``[out, in/2]``, INT4) or ``q_weight`` (int8), and
  ``scale`` / ``zero`` in fp32 with the reference's shapes (``[out, in/G, 1]`` per_group,
  ``[out, 1]`` per_channel, 0-d per_tensor); ``bias`` as a Parameter or ``None``;
* ``forward`` takes the kernel only if ``use_kernel`` and INT4 and not ``quantize_inputs``
  and the input is on a CUDA device; otherwise it dequantizes and calls ``F.linear``
  (that branch is the definition the kernel is tested against);
* ``dequantize`` returns ``(q - zero) * scale`` in fp32.

Differences, all additive:

* the kernel path reads ``packed_weight`` as stored — there is no repacking pass.
  ``_packed_weight_kernel`` still appears lazily on first kernel call (callers of the
  reference look for it); it is a *non-persistent buffer* holding the kernel-side view of
  the weights: the same tensor for plain layers, the group-sorted columns for act-order
  layers.  It follows ``.to()`` and stays out of ``state_dict()``.
* bf16 inputs run in bf16 (the reference silently computed them in fp16).
* ``from_tensors`` sets ``use_kernel = False`` (the reference leaves it unset, so a loaded
  layer raises ``AttributeError`` in ``forward``).
* optional ``g_idx`` (``[in]`` int32, group of every input column, GPTQ act-order) and
  ``input_scale`` (``[in]`` fp32, AWQ scale applied at run time) buffers; both default to
  ``None``, are ordinary buffers so they round-trip through ``state_dict()``, and are
  honoured by ``dequantize`` / the eager branch as well as by the kernel.
* ``kernel_meta_fp16 = True`` makes the kernel read fp16 copies of scale and zero
  (half the metadata traffic, scale rounded to 11 bits).
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from pare_b200.config import QuantConfig
from pare_b200.core.dtype import QuantDtype
from pare_b200.core.functional import dequantize_tensor, quantize_tensor
from pare_b200.core.pack import pack_int4, unpack_int4
from pare_b200.core.scale import compute_scale

_FP8 = (QuantDtype.FP8_E4M3, QuantDtype.FP8_E5M2)


class QuantizedLinear(nn.Module):
    def __init__(
        self,
        q_weight: Tensor,
        scale: Tensor,
        zero: Tensor,
        config: QuantConfig,
        bias: nn.Parameter | None,
        in_features: int,
        out_features: int,
        quantize_inputs: bool = False,
        use_kernel: bool = False,
        g_idx: Tensor | None = None,
        input_scale: Tensor | None = None,
    ) -> None:
        super().__init__()
        dtype = config.effective_dtype
        if dtype is QuantDtype.NF4 or dtype in _FP8:
            raise NotImplementedError(f"{dtype.name} layers are outside the INT4/INT8 affine path of this package")
        self._init_common(config, in_features, out_features, quantize_inputs, use_kernel)

        q2d = q_weight.reshape(out_features, in_features)
        if config.bits == 4:
            self.register_buffer("packed_weight", pack_int4(q2d))
            self.register_buffer("q_weight", None)
        else:
            self.register_buffer("q_weight", q2d.to(torch.int8))
            self.register_buffer("packed_weight", None)
        self.register_buffer("scale", scale.float())
        self.register_buffer("zero", zero.float())
        self._register_optional(g_idx, input_scale)
        self.bias = nn.Parameter(bias.data.clone()) if bias is not None else None

    # -- shared construction helpers ----------------------------------------
    def _init_common(self, config, in_features, out_features, quantize_inputs, use_kernel) -> None:
        self.config = config
        self.in_features = in_features
        self.out_features = out_features
        self.quantize_inputs = quantize_inputs
        self.use_kernel = use_kernel
        self.kernel_meta_fp16 = False

    def _register_optional(self, g_idx: Tensor | None, input_scale: Tensor | None) -> None:
        self.register_buffer("g_idx", None if g_idx is None else g_idx.to(torch.int32))
        self.register_buffer("input_scale", None if input_scale is None else input_scale.float())

    # -- dequantize / eager forward -----------------------------------------
    def _codes(self) -> Tensor:
        return unpack_int4(self.packed_weight) if self.config.bits == 4 else self.q_weight.to(torch.int32)

    def dequantize(self) -> Tensor:
        """Full fp32 weight ``[out, in]``: ``(q - zero) * scale`` (per column group if ``g_idx``)."""
        q = self._codes()
        if self.g_idx is not None:
            idx = self.g_idx.long()
            s = self.scale.reshape(self.out_features, -1)[:, idx]
            z = self.zero.reshape(self.out_features, -1)[:, idx]
            return (q.float() - z) * s
        return dequantize_tensor(q, self.scale, self.zero).reshape(self.out_features, self.in_features)

    def forward(self, x: Tensor) -> Tensor:
        if (
            self.use_kernel
            and self.config.effective_dtype is QuantDtype.INT4
            and not self.quantize_inputs
            and x.is_cuda
        ):
            return self._forward_kernel(x)

        weight = self.dequantize().to(x.dtype)
        if self.input_scale is not None:
            x = (x.float() / self.input_scale).to(x.dtype)
        if self.quantize_inputs:
            # per-token dynamic INT8 fake-quantization of the activations (SmoothQuant W8A8)
            step = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-6) / 127.0
            x = ((x / step).round().clamp(-128, 127) * step).to(x.dtype)
        bias = self.bias
        if bias is not None and bias.dtype != x.dtype:   # e.g. an imported fp16 bias under fp32 activations
            bias = bias.to(x.dtype)
        return nn.functional.linear(x, weight, bias)

    # -- CUDA path -----------------------------------------------------------
    def _kernel_group_size(self) -> int:
        return self.config.group_size if self.config.granularity == "per_group" else self.in_features

    def _prepare_kernel_buffers(self) -> None:
        """Create the derived, non-persistent tensors the kernel reads (first call only)."""
        from pare_b200.kernels.matmul_int4 import _meta_2d, pack_meta_h2

        n = self.out_features
        scale2d, zero2d = _meta_2d(self.scale, n), _meta_2d(self.zero, n)
        if self.config.granularity == "per_tensor":
            scale2d, zero2d = scale2d.contiguous(), zero2d.contiguous()
        packed, perm = self.packed_weight, None
        if self.g_idx is not None:
            # act-order: sort columns by group so every group is contiguous; the kernel gathers x
            perm = torch.argsort(self.g_idx.long(), stable=True)
            packed = pack_int4(unpack_int4(self.packed_weight)[:, perm]).contiguous()
            perm = perm.to(torch.int32).contiguous()
        self.register_buffer("_packed_weight_kernel", packed, persistent=False)
        self.register_buffer("_col_perm_kernel", perm, persistent=False)
        self.register_buffer("_scale_kernel", scale2d, persistent=False)
        self.register_buffer("_zero_kernel", zero2d, persistent=False)
        self.register_buffer("_meta_h2_kernel", pack_meta_h2(scale2d, zero2d), persistent=False)

    def _forward_kernel(self, x: Tensor) -> Tensor:
        from pare_b200.kernels.matmul_int4 import w4a16_forward

        if not hasattr(self, "_packed_weight_kernel"):
            self._prepare_kernel_buffers()
        shape = x.shape
        out_dtype = x.dtype
        x2d = x.reshape(-1, self.in_features)
        if x2d.dtype not in (torch.float16, torch.bfloat16):
            x2d = x2d.to(torch.float16)
        if x2d.stride(-1) != 1:
            x2d = x2d.contiguous()
        use_h2 = self.kernel_meta_fp16
        y = w4a16_forward(
            x2d,
            self._packed_weight_kernel,
            None if use_h2 else self._scale_kernel,
            None if use_h2 else self._zero_kernel,
            self._kernel_group_size(),
            bias=self.bias,
            col_perm=self._col_perm_kernel,
            input_scale=self.input_scale,
            meta_h2=self._meta_h2_kernel if use_h2 else None,
        )
        return y.to(out_dtype).reshape(*shape[:-1], self.out_features)

    def supports_prepared(self, rows: int) -> bool:
        """True if :meth:`forward_prepared` can serve ``rows`` activation rows of this layer."""
        return (self.use_kernel and self.config.dtype == QuantDtype.INT4 and not self.quantize_inputs
                and self.g_idx is None and self.input_scale is None and rows <= 16
                and self.in_features % 256 == 0 and self._kernel_group_size() % 128 == 0)

    def forward_prepared(self, prep, peer=None) -> Tensor:
        """Forward for activations handed over as :class:`PreparedActivations` (decode, rows <= 16):
        the producing kernel wrote them in operand order, so no preparation launch is needed.  ``peer`` (a
        ``PeerAllReduce``): this layer is a row-parallel shard; the result is the sum over the ranks, added inside
        the kernel."""
        from pare_b200.kernels.matmul_int4 import w4a16_forward_prepared

        if not self.supports_prepared(prep.rows):
            raise ValueError("this layer cannot take prepared activations (act-order, input scale, shape or row count)")
        if not hasattr(self, "_packed_weight_kernel"):
            self._prepare_kernel_buffers()
        use_h2 = self.kernel_meta_fp16
        return w4a16_forward_prepared(
            prep, self._packed_weight_kernel,
            None if use_h2 else self._scale_kernel, None if use_h2 else self._zero_kernel,
            self._kernel_group_size(), bias=self.bias, meta_h2=self._meta_h2_kernel if use_h2 else None, peer=peer)

    def _forward_produced(self, producer: int, a: Tensor, **kw) -> Tensor:
        from pare_b200.kernels.matmul_int4 import w4a16_forward_produced

        if not self.supports_prepared(a.shape[0]):
            raise ValueError("this layer cannot compute its activations in-kernel (act-order, input scale, shape or row count)")
        if not hasattr(self, "_packed_weight_kernel"):
            self._prepare_kernel_buffers()
        use_h2 = self.kernel_meta_fp16
        return w4a16_forward_produced(
            producer, a, self._packed_weight_kernel,
            None if use_h2 else self._scale_kernel, None if use_h2 else self._zero_kernel,
            self._kernel_group_size(), bias=self.bias, meta_h2=self._meta_h2_kernel if use_h2 else None, **kw)

    def forward_rmsnorm(self, x: Tensor, delta: Tensor | None, norm_weight: Tensor, resid_out: Tensor | None = None,
                        eps: float = 1e-5) -> Tensor:
        """``self(rmsnorm(x + delta) * norm_weight)`` for ``x [rows <= 16, in_features]`` in one launch: the
        streaming kernel normalises the row itself.  ``x + delta`` is stored to ``resid_out`` (not ``x``)."""
        from pare_b200.kernels import _lib

        return self._forward_produced(_lib.PRODUCER_RMSNORM, x, delta=delta, norm_weight=norm_weight, resid_out=resid_out, eps=eps)

    def forward_silu_mul(self, gate_up: Tensor, peer=None) -> Tensor:
        """``self(silu(gate) * up)`` for a fused ``gate_up [rows <= 16, 2 * in_features]`` in one launch; with ``peer`` (a
        ``PeerAllReduce``) summed over the ranks inside the kernel (this layer being a row-parallel shard)."""
        from pare_b200.kernels import _lib

        return self._forward_produced(_lib.PRODUCER_SILU_MUL, gate_up, peer=peer)

    # -- alternate constructors ----------------------------------------------
    @classmethod
    def from_tensors(
        cls,
        packed_weight: Tensor | None,
        q_weight: Tensor | None,
        scale: Tensor,
        zero: Tensor,
        config: QuantConfig,
        bias: Tensor | None,
        in_features: int,
        out_features: int,
        quantize_inputs: bool = False,
        g_idx: Tensor | None = None,
        input_scale: Tensor | None = None,
    ) -> "QuantizedLinear":
        """Rebuild a layer from stored tensors without re-packing (used by ``load_quantized``)."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self._init_common(config, in_features, out_features, quantize_inputs, use_kernel=False)
        self.register_buffer("packed_weight", packed_weight)
        self.register_buffer("q_weight", None if q_weight is None else q_weight.to(torch.int8))
        self.register_buffer("scale", scale.float())
        self.register_buffer("zero", zero.float())
        self._register_optional(g_idx, input_scale)
        self.bias = nn.Parameter(bias.clone()) if bias is not None else None
        return self

    @classmethod
    def from_linear(cls, linear: nn.Linear, config: QuantConfig) -> "QuantizedLinear":
        """Round-to-nearest quantization of an ``nn.Linear``."""
        w = linear.weight.data.float()
        dtype = config.effective_dtype
        scale, zero = compute_scale(w, dtype, granularity=config.granularity, group_size=config.group_size, sym=config.sym)
        q = quantize_tensor(w, scale, zero, dtype)
        return cls(q, scale, zero, config, linear.bias, linear.in_features, linear.out_features)

    def extra_repr(self) -> str:
        mode = "W+A" if self.quantize_inputs else "W"
        return (
            f"in={self.in_features}, out={self.out_features}, dtype={self.config.effective_dtype.name}, "
            f"scheme={self.config.scheme}, granularity={self.config.granularity}, mode={mode}"
        )
