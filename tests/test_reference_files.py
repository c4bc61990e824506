"""Files and tensors written BY THE REFERENCE, read by this package (fixtures of tests/golden/generate.py).

* ``tests/golden/ref_ckpt``: a directory from the reference's ``save_quantized`` (pare/model/io.py:52-123).
  ``load_quantized`` must rebuild it (the reference's own loader leaves ``use_kernel`` unset, so its
  loaded layers raise on ``forward``; pare/layers/linear.py:182-202 vs :122) and the rebuilt model must
  reproduce the outputs the reference's model gave -- on the CPU through the eager branch, on the GPU
  through the CUDA kernels at 1 row (streaming kernel) and 64 rows (tensor-core kernel).
* ``tests/golden/awq_gemm_layer.npz``: the AutoAWQ GEMM tensors from the reference's exporter
  (pare/model/export_awq.py:39-49, 75-94).  ``to_awq_gemm`` must produce the same bits, and
  ``from_awq_gemm`` of them must run through the kernels and agree with the reference layer's outputs.

Tolerances: the file's stated ones (max rel 1e-2, mean 1e-3 against the fp32 outputs of the reference).
"""

import numpy as np
import pytest
import torch
import torch.nn as nn

import pare_b200
from oracle.w4a16 import rel_err
from pare_b200.layers.linear import QuantizedLinear
from pare_b200.model.awq_format import from_awq_gemm, to_awq_gemm

from conftest import GOLDEN


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.up_proj = nn.Linear(512, 768, bias=True)
        self.down_proj = nn.Linear(768, 512, bias=True)

    def forward(self, x):
        return self.down_proj(torch.relu(self.up_proj(x)))


def _bars(y, ref):
    mx, mean = rel_err(np.asarray(y, dtype=np.float32), ref)
    assert mx <= 1e-2 and mean <= 1e-3, (mx, mean)


def _awq_oracle(g, x):
    """fp32 oracle on what the AutoAWQ tensors actually hold: the layer's codes and zero points, its scales and
    bias rounded to fp16 (the format's dtypes)."""
    from oracle import w4a16 as ow
    return ow.linear(x.astype(np.float32), g["packed"], g["scale"].reshape(256, -1).astype(np.float16).astype(np.float32),
                     g["zero"].reshape(256, -1), bias=g["bias32"].astype(np.float16).astype(np.float32))


# ---- CPU ---------------------------------------------------------------------------------------

def test_reference_checkpoint_loads_and_matches_on_cpu(golden):
    io = golden("ref_ckpt_io.npz")
    model = pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt")
    assert isinstance(model.up_proj, QuantizedLinear) and model.up_proj.use_kernel is False
    assert model.up_proj.packed_weight.shape == (768, 256) and model.up_proj.scale.shape == (768, 4, 1)
    with torch.no_grad():
        for m in ("1", "64"):
            y = model(torch.from_numpy(io["x" + m]).float())
            assert np.allclose(y.numpy(), io["y" + m], rtol=0, atol=2e-5)   # same fp32 op sequence as the reference


def test_awq_export_equals_reference_exporter_bits(golden):
    g = golden("awq_gemm_layer.npz")
    cfg = pare_b200.QuantConfig(bits=4, scheme="rtn", granularity="per_group", group_size=128)
    ql = QuantizedLinear.from_tensors(torch.from_numpy(g["packed"]), None, torch.from_numpy(g["scale"]),
                                      torch.from_numpy(g["zero"]), cfg, torch.from_numpy(g["bias32"]), 512, 256)
    t = to_awq_gemm(ql)
    for key in ("qweight", "qzeros", "scales", "bias"):
        assert t[key].dtype == torch.from_numpy(g[key]).dtype and np.array_equal(t[key].numpy(), g[key]), key
    back = from_awq_gemm(*(torch.from_numpy(g[k]) for k in ("qweight", "qzeros", "scales", "bias")), group_size=128)
    assert np.array_equal(back.packed_weight.numpy(), g["packed"]) and np.array_equal(back.zero.numpy(), g["zero"])
    with torch.no_grad():
        y = back(torch.from_numpy(g["x"]).float())
    assert np.allclose(y.numpy(), _awq_oracle(g, g["x"]), rtol=0, atol=2e-5)
    # the format stores fp16 scales (11 significant bits): against the reference layer's own fp32-scale outputs
    # that alone moves outputs near zero by more than 1e-2 of the floor, so the max bar is widened here
    mx, mean = rel_err(y.numpy(), g["y"])
    assert mx <= 5e-2 and mean <= 1e-3, (mx, mean)


# ---- GPU ---------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reference_checkpoint_runs_on_the_kernels(dtype, golden, cuda_lib):
    """The layers rebuilt from the reference-written file, on the CUDA path, against the oracle on the file's own
    tensors (bars of tests/parity.py: 1 row runs the streaming kernel, 64 rows the tensor-core kernel); the oracle
    itself reproduces the outputs the reference's model gave on the same fp16 inputs."""
    from parity import check_linear, oracle_pair
    io = golden("ref_ckpt_io.npz")
    model = pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt", use_kernel=True).cuda()
    assert model.up_proj.use_kernel and model.down_proj.use_kernel
    with torch.no_grad():
        for m in ("1", "64"):
            x = torch.from_numpy(io["x" + m]).cuda().to(dtype)
            up = model.up_proj(x)
            assert hasattr(model.up_proj, "_packed_weight_kernel") and up.dtype == dtype and up.shape == (int(m), 768)
            check_linear(up, model.up_proj, x, dtype)
            h = torch.relu(up)
            check_linear(model.down_proj(h), model.down_proj, h, dtype)
            if dtype == torch.float16:
                ref32, _ = oracle_pair(model.up_proj, x, dtype)
                b16 = model.up_proj.bias.detach().half().float().cpu().numpy() - model.up_proj.bias.detach().float().cpu().numpy()
                assert np.allclose(ref32 - b16, io["up" + m], rtol=0, atol=3e-5)     # oracle == the reference's own run
                mx, mean = rel_err(model(x).float().cpu().numpy(), io["y" + m])       # whole model, end to end
                assert mx <= 5e-2 and mean <= 2e-3, (mx, mean)                        # two layers, weights cast at 64 rows


@pytest.mark.gpu
def test_reference_checkpoint_tensor_parallel_slices_on_the_kernels(golden, cuda_lib):
    """Both ranks' slices of the reference-written file, each through the kernels on this GPU: the column shards'
    outputs concatenate to the unsharded layer's, the row shards' partial sums add up to it."""
    from parity import check_linear
    io = golden("ref_ckpt_io.npz")
    plan = {"up_proj": "column", "down_proj": "row"}
    whole = pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt", use_kernel=True).cuda()
    shards = [pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt", use_kernel=True, tp_plan=plan, tp_rank=r, tp_world=2).cuda()
              for r in range(2)]
    with torch.no_grad():
        for m in ("1", "64"):
            x = torch.from_numpy(io["x" + m]).cuda()
            ups = [s.up_proj(x) for s in shards]
            assert ups[0].shape == (int(m), 384)
            up = torch.cat(ups, dim=1)
            assert torch.equal(up, whole.up_proj(x))                 # output rows are independent: same bits
            h = torch.relu(up)
            parts = [s.down_proj(h[:, r * 384:(r + 1) * 384].contiguous()).float() for r, s in enumerate(shards)]
            total = (parts[0] + parts[1]).half()
            # rank 0 carries the bias; the sum of the two partial products is the unsharded product up to rounding.
            # Each partial is itself rounded to fp16 at its own (larger) magnitude before the sum: max <= 3e-2 here.
            check_linear(total, whole.down_proj, h, torch.float16, max_rel=3e-2)


@pytest.mark.gpu
def test_awq_gemm_import_runs_on_the_kernels(golden, cuda_lib):
    from parity import check_linear
    g = golden("awq_gemm_layer.npz")
    layer = from_awq_gemm(*(torch.from_numpy(g[k]) for k in ("qweight", "qzeros", "scales", "bias")), group_size=128).cuda()
    layer.use_kernel = True
    x = torch.from_numpy(g["x"]).cuda()
    with torch.no_grad():
        for m in (1, 4, 16, 64):
            y = layer(x[:m])
            assert y.dtype == torch.float16 and y.shape == (m, 256)
            check_linear(y, layer, x[:m], torch.float16)                  # on what the AutoAWQ tensors hold
            mx, mean = rel_err(y.float().cpu().numpy(), g["y"][:m])      # the reference layer's fp32-scale outputs:
            assert mx <= 5e-2 and mean <= 1.5e-3, (mx, mean)              # fp16 scales of the format, widened max
