"""Parity bars shared by the GPU tests (the tolerances the tests state, in one place).

``rel = |y - ref| / max(|ref|, 1e-2 * max|ref|)`` (``oracle.w4a16.rel_err``).

* Streaming kernels (up to 16 activation rows) compute with the fp32 weights ``(q - zero) * scale``:
  against the fp32 oracle max <= 1e-2, mean <= 1e-3 (bf16 outputs, 8 significant bits: mean <= 2.5e-3).
* The tensor-core kernel (more than 16 rows) feeds its MMA the weight cast to the activation dtype, exactly what the
  reference's eager path does (pare/layers/linear.py:129).  Bar 1, against the oracle with weights cast the same
  way: the bars above, unchanged.  Bar 2, against the fp32-weight oracle: the reference's own cast is the dominant
  error there; it is measured oracle against oracle, and the kernel must stay within 1.5x of it plus the bars above.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import w4a16 as ow

MAX_REL, MEAN_REL, MEAN_REL_BF16 = 1e-2, 1e-3, 2.5e-3


def layer_arrays(ql):
    n = ql.out_features
    return (ql.packed_weight.cpu().numpy(), ql.scale.detach().cpu().numpy().reshape(n, -1),
            ql.zero.detach().cpu().numpy().reshape(n, -1))


def cast(a: np.ndarray, dtype) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).float().numpy()


def oracle_pair(ql, x, dtype, g_idx=None, input_scale=None):
    """(fp32-weight oracle, oracle with weights cast to ``dtype``) of a layer on activations ``x`` (a tensor of
    ``dtype``); the bias enters both as the kernel sees it (cast to ``dtype``)."""
    packed, scale, zero = layer_arrays(ql)
    w = ow.dequantize(packed, scale, zero, g_idx)
    xin = x.float().cpu().numpy()
    xin_cast = xin
    if input_scale is not None:
        xin = xin / np.asarray(input_scale, dtype=np.float32)
        xin_cast = cast(xin, dtype)
    y32, y16 = xin @ w.T, xin_cast @ cast(w, dtype).T
    if ql.bias is not None:
        b = ql.bias.detach().to(dtype).float().cpu().numpy()
        y32, y16 = y32 + b, y16 + b
    return y32.astype(np.float32), y16.astype(np.float32)


def takes_tensor_cores(rows: int, ql) -> bool:
    """The routing rule of ``pare_w4a16_forward``: more than 16 rows, K a multiple of 512, groups a multiple of 128."""
    g = ql.config.group_size if ql.config.granularity == "per_group" else ql.in_features
    return rows > 16 and ql.in_features % 512 == 0 and g % 128 == 0


def check_linear(y, ql, x, dtype, max_rel: float = MAX_REL, **kw):
    """The bars above for ``y = ql(x)`` through the kernels, by the kernel the call is routed to."""
    yn = y.float().cpu().numpy().reshape(-1, ql.out_features)
    mean_bar = MEAN_REL_BF16 if dtype == torch.bfloat16 else MEAN_REL
    ref32, ref_cast = oracle_pair(ql, x.reshape(-1, ql.in_features), dtype, **kw)
    if not takes_tensor_cores(yn.shape[0], ql):
        mx, mean = ow.rel_err(yn, ref32)
        assert mx <= max_rel and mean <= mean_bar, (mx, mean)
        return
    mx, mean = ow.rel_err(yn, ref_cast)
    assert mx <= MAX_REL and mean <= mean_bar, (mx, mean)
    noise_mx, noise_mean = ow.rel_err(ref_cast, ref32)
    mx2, mean2 = ow.rel_err(yn, ref32)
    assert mx2 <= 1.5 * noise_mx + MAX_REL and mean2 <= 1.5 * noise_mean + mean_bar, (mx2, mean2, noise_mx, noise_mean)
