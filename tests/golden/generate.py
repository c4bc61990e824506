"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Usage (only where the reference checkout exists; the fixtures are committed):

    python tests/golden/generate.py /path/to/reference

The reference package is imported as ``pare`` from the given path; this repository's own
package is named ``pare_b200`` and is not imported here.  Every fixture is a small ``.npz``
holding seeded inputs and the outputs the reference produced for them on CPU:

  w4a16_g128.npz       256x256 RTN INT4 g128 layer built like the reference's kernel tests
                       (tests/test_triton_kernel.py:31-35), fp16 activations for M = 64,
                       reference ``QuantizedLinear.forward`` in fp32 and its dequantized weight
  w4a16_channel.npz    128x256 per_channel layer with bias, same outputs
  kivi_prims.npz       ``_quantize_keys`` / ``_quantize_values`` codes, scales, zeros for bits 2, 4, 8
  kivi_cache.npz       ``QuantizedKVCache.update`` over a 96-token prefill and 40 decode steps
                       (bits 4, G 32, residual 64): final dense K/V, token counts per step, and
                       fp32 grouped-query attention over the final cache
  ref_ckpt/            a directory written by the reference's ``save_quantized`` (``model.safetensors`` +
                       ``pare_config.json``) for a two-layer MLP (512 -> 768 -> 512, biases) quantized by the
                       reference's ``pare.quantize`` (RTN INT4 g128), and ``ref_ckpt_io.npz``: inputs for 1 and 64
                       rows with the outputs of the reference's own model on them (CPU, fp32)
  awq_gemm_layer.npz   the AutoAWQ GEMM tensors the reference's exporter (``pare/model/export_awq.py:75-94``)
                       makes of a 512 -> 256 layer with bias, the layer's own packed weight / scale / zero, inputs
                       and the reference layer's fp32 outputs
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import torch.nn as nn
    from pare.config import QuantConfig
    from pare.kv_cache import KVCacheConfig, QuantizedKVCache, _quantize_keys, _quantize_values
    from pare.layers.linear import QuantizedLinear

    torch.set_num_threads(1)

    # ---- W4A16, per_group 128 ------------------------------------------------
    torch.manual_seed(0)
    lin = nn.Linear(256, 256, bias=False)
    ql = QuantizedLinear.from_linear(lin, QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128))
    torch.manual_seed(1)
    x = torch.randn(64, 256, dtype=torch.float16)
    with torch.no_grad():
        y = ql.forward(x.float())
    np.savez_compressed(
        HERE / "w4a16_g128.npz",
        packed=ql.packed_weight.numpy(), scale=ql.scale.numpy(), zero=ql.zero.numpy(),
        x=x.numpy(), y=y.numpy(), w=ql.dequantize().numpy(),
    )

    # ---- W4A16, per_channel with bias -----------------------------------------
    torch.manual_seed(2)
    lin = nn.Linear(256, 128, bias=True)
    ql = QuantizedLinear.from_linear(lin, QuantConfig(bits=4, scheme="rtn", granularity="per_channel"))
    torch.manual_seed(3)
    x = torch.randn(7, 256, dtype=torch.float16)
    with torch.no_grad():
        y = ql.forward(x.float())
    np.savez_compressed(
        HERE / "w4a16_channel.npz",
        packed=ql.packed_weight.numpy(), scale=ql.scale.numpy(), zero=ql.zero.numpy(),
        bias=ql.bias.detach().numpy(), x=x.numpy(), y=y.numpy(), w=ql.dequantize().numpy(),
    )

    # ---- KIVI primitives ---------------------------------------------------------
    torch.manual_seed(4)
    k = torch.randn(1, 2, 64, 128, dtype=torch.float16)
    k[..., 7] *= 10.0
    v = torch.randn(1, 2, 64, 128, dtype=torch.float16)
    v[:, :, 3, :] *= 5.0
    out = {"k": k.numpy(), "v": v.numpy()}
    for bits in (2, 4, 8):
        kq, ks, kz = _quantize_keys(k.float(), bits, 32)
        vq, vs, vz = _quantize_values(v.float(), bits, 32)
        for name, t in (("kq", kq), ("ks", ks), ("kz", kz), ("vq", vq), ("vs", vs), ("vz", vz)):
            out[f"{name}{bits}"] = t.numpy()
    np.savez_compressed(HERE / "kivi_prims.npz", **out)

    # ---- KIVI cache sequence ------------------------------------------------------
    torch.manual_seed(5)
    B, H, HQ, D, total = 1, 2, 8, 128, 136
    k_all = torch.randn(B, H, total, D, dtype=torch.float16)
    v_all = torch.randn(B, H, total, D, dtype=torch.float16)
    k_all[..., 11] *= 10.0
    q = torch.randn(B, HQ, 1, D, dtype=torch.float16)
    cache = QuantizedKVCache(num_layers=1, config=KVCacheConfig(bits=4, group_size=32, residual_length=64))
    counts = []
    fk, fv = cache.update(0, k_all[:, :, :96], v_all[:, :, :96])
    counts.append((cache._compressed[0].k_quant.shape[2] if cache._compressed[0] is not None else 0,
                   cache._residual_k[0].shape[2]))
    for t in range(96, total):
        fk, fv = cache.update(0, k_all[:, :, t:t + 1], v_all[:, :, t:t + 1])
        counts.append((cache._compressed[0].k_quant.shape[2], cache._residual_k[0].shape[2]))
    rep = HQ // H
    attn = torch.nn.functional.scaled_dot_product_attention(
        q.float(), fk.float().repeat_interleave(rep, dim=1), fv.float().repeat_interleave(rep, dim=1))
    np.savez_compressed(
        HERE / "kivi_cache.npz",
        k_all=k_all.numpy(), v_all=v_all.numpy(), q=q.numpy(),
        full_k=fk.numpy(), full_v=fv.numpy(), counts=np.array(counts, dtype=np.int32), attn=attn.numpy(),
    )
    # ---- a checkpoint written by the reference's save_quantized ------------------------
    import pare
    from pare.model.io import save_quantized

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.up_proj = nn.Linear(512, 768, bias=True)
            self.down_proj = nn.Linear(768, 512, bias=True)

        def forward(self, x):
            return self.down_proj(torch.relu(self.up_proj(x)))

    torch.manual_seed(6)
    model = MLP()
    pare.quantize(model, QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128))
    assert isinstance(model.up_proj, QuantizedLinear) and isinstance(model.down_proj, QuantizedLinear)
    save_quantized(model, HERE / "ref_ckpt")
    torch.manual_seed(7)
    x1 = torch.randn(1, 512, dtype=torch.float16)
    x64 = torch.randn(64, 512, dtype=torch.float16)
    with torch.no_grad():
        np.savez_compressed(HERE / "ref_ckpt_io.npz", x1=x1.numpy(), x64=x64.numpy(),
                            y1=model(x1.float()).numpy(), y64=model(x64.float()).numpy(),
                            up1=model.up_proj(x1.float()).numpy(), up64=model.up_proj(x64.float()).numpy())

    # ---- the reference exporter's AutoAWQ GEMM tensors of one layer ------------------------
    from pare.model.export_awq import _to_awq_linear

    torch.manual_seed(8)
    lin = nn.Linear(512, 256, bias=True)
    ql = QuantizedLinear.from_linear(lin, QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128))
    awq = _to_awq_linear(ql, 128)
    torch.manual_seed(9)
    x = torch.randn(64, 512, dtype=torch.float16)
    with torch.no_grad():
        y = ql.forward(x.float())
    np.savez_compressed(
        HERE / "awq_gemm_layer.npz",
        qweight=awq.qweight.numpy(), qzeros=awq.qzeros.numpy(), scales=awq.scales.numpy(), bias=awq.bias.numpy(),
        packed=ql.packed_weight.numpy(), scale=ql.scale.numpy(), zero=ql.zero.numpy(), bias32=ql.bias.detach().numpy(),
        x=x.numpy(), y=y.numpy(),
    )
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
