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
    io = golden("ref_ckpt_io.npz")
    model = pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt", use_kernel=True).cuda()
    assert model.up_proj.use_kernel and model.down_proj.use_kernel
    with torch.no_grad():
        for m in ("1", "64"):
            x = torch.from_numpy(io["x" + m]).cuda().to(dtype)
            up = model.up_proj(x)
            assert hasattr(model.up_proj, "_packed_weight_kernel") and up.dtype == dtype
            if dtype == torch.float16:   # same inputs as the reference saw
                _bars(up.float().cpu().numpy(), io["up" + m])
                _bars(model(x).float().cpu().numpy(), io["y" + m])
            else:                        # bf16 rounds the input: compare with the eager branch on the same input
                model.up_proj.use_kernel = False
                ref = model.up_proj(x.float()).float().cpu().numpy()
                model.up_proj.use_kernel = True
                mx, mean = rel_err(up.float().cpu().numpy(), ref)
                assert mx <= 1e-2 and mean <= 2.5e-3, (mx, mean)


@pytest.mark.gpu
def test_reference_checkpoint_tensor_parallel_slices_on_the_kernels(golden, cuda_lib):
    """Both ranks' slices of the reference-written file, each through the kernels on this GPU: column shards
    concatenate, row shards add up to the reference's outputs."""
    io = golden("ref_ckpt_io.npz")
    plan = {"up_proj": "column", "down_proj": "row"}
    with torch.no_grad():
        for m in ("1", "64"):
            x = torch.from_numpy(io["x" + m]).cuda()
            total = None
            ups = []
            for rank in range(2):
                shard = pare_b200.load_quantized(MLP(), GOLDEN / "ref_ckpt", use_kernel=True, tp_plan=plan, tp_rank=rank,
                                                 tp_world=2).cuda()
                assert shard.up_proj.out_features == 384 and shard.down_proj.in_features == 384
                up = shard.up_proj(x)
                ups.append(up)
                part = shard.down_proj(torch.relu(up)).float()
                total = part if total is None else total + part
            _bars(torch.cat(ups, dim=1).float().cpu().numpy(), io["up" + m])
            _bars(total.cpu().numpy(), io["y" + m])


@pytest.mark.gpu
def test_awq_gemm_import_runs_on_the_kernels(golden, cuda_lib):
    g = golden("awq_gemm_layer.npz")
    layer = from_awq_gemm(*(torch.from_numpy(g[k]) for k in ("qweight", "qzeros", "scales", "bias")), group_size=128).cuda()
    layer.use_kernel = True
    x = torch.from_numpy(g["x"]).cuda()
    with torch.no_grad():
        for m in (1, 4, 16, 64):
            y = layer(x[:m])
            assert y.dtype == torch.float16 and y.shape == (m, 256)
            _bars(y.float().cpu().numpy(), _awq_oracle(g, g["x"][:m]))
            mx, mean = rel_err(y.float().cpu().numpy(), g["y"][:m])      # fp16 scales of the format: widened max
            assert mx <= 5e-2 and mean <= 1e-3, (mx, mean)
