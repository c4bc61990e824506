"""Save / load quantized models — file format of the reference, kernel-ready layers on load.

On-disk layout is the reference's (``pare/model/io.py:52-196``): a directory with
``model.safetensors`` (the de-duplicated ``state_dict()``: ``packed_weight`` / ``q_weight`` /
``scale`` / ``zero`` / ``bias`` of every ``QuantizedLinear`` plus all other tensors) and
``pare_config.json`` (per-layer ``bits, scheme, granularity, group_size, sym, smooth_alpha,
in_features, out_features, quantize_inputs, has_bias``).  Files written by either package load
in the other.  Additions: the optional ``g_idx`` / ``input_scale`` buffers travel as ordinary
tensors when present, and ``load_quantized(..., use_kernel=True)`` switches the rebuilt layers
to the CUDA path (the reference leaves ``use_kernel`` unset on loaded layers).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch.nn as nn
from torch import Tensor

CONFIG_FILE = "pare_config.json"
TENSORS_FILE = "model.safetensors"
_LAYER_KEYS = ("bits", "scheme", "granularity", "group_size", "sym", "smooth_alpha")


def save_quantized(model: nn.Module, path: str | Path) -> None:
    """Write ``path/model.safetensors`` and ``path/pare_config.json``."""
    from safetensors.torch import save_file

    from pare_b200.layers.linear import QuantizedLinear

    layers = {
        name: {
            **{k: getattr(m.config, k) for k in _LAYER_KEYS},
            "in_features": m.in_features,
            "out_features": m.out_features,
            "quantize_inputs": m.quantize_inputs,
            "has_bias": m.bias is not None,
        }
        for name, m in model.named_modules()
        if isinstance(m, QuantizedLinear)
    }
    if not layers:
        raise ValueError("No QuantizedLinear layers found in model. Quantize the model first with pare.quantize().")

    # safetensors refuses aliased storage (tied embeddings): keep the first name of each storage
    tensors: dict[str, Tensor] = {}
    seen: set[int] = set()
    for key, value in model.state_dict().items():
        value = value.contiguous().cpu()
        ptr = value.untyped_storage().data_ptr()
        if ptr not in seen:
            seen.add(ptr)
            tensors[key] = value

    out = Path(path)
    out.mkdir(parents=True, exist_ok=True)
    save_file(tensors, out / TENSORS_FILE)
    from pare_b200 import __version__
    (out / CONFIG_FILE).write_text(json.dumps({"pare_version": __version__, "quantized_layers": layers}, indent=2))
    print(f"[pare] Saved {len(layers)} quantized layers to {out}  ({(out / TENSORS_FILE).stat().st_size / 1e6:.0f} MB)")


def load_quantized(model: nn.Module, path: str | Path, use_kernel: bool = False) -> nn.Module:
    """Swap the named modules of ``model`` for ``QuantizedLinear`` layers rebuilt from ``path`` and
    load every other tensor; ``use_kernel=True`` puts the rebuilt layers on the CUDA path."""
    from safetensors.torch import load_file

    from pare_b200.config import QuantConfig
    from pare_b200.layers.linear import QuantizedLinear

    src = Path(path)
    meta = json.loads((src / CONFIG_FILE).read_text())["quantized_layers"]
    tensors = load_file(src / TENSORS_FILE)

    for name, info in meta.items():
        cfg = QuantConfig(**{k: info[k] for k in _LAYER_KEYS if k in info})
        t = lambda suffix: tensors.get(f"{name}.{suffix}")
        layer = QuantizedLinear.from_tensors(
            packed_weight=t("packed_weight"), q_weight=t("q_weight"),
            scale=tensors[f"{name}.scale"], zero=tensors[f"{name}.zero"],
            config=cfg, bias=t("bias"),
            in_features=info["in_features"], out_features=info["out_features"],
            quantize_inputs=info.get("quantize_inputs", False),
            g_idx=t("g_idx"), input_scale=t("input_scale"),
        )
        layer.use_kernel = use_kernel
        parent = model
        *parents, leaf = name.split(".")
        for part in parents:
            parent = getattr(parent, part)
        setattr(parent, leaf, layer)

    prefixes = tuple(n + "." for n in meta)
    rest = {k: v for k, v in tensors.items() if not k.startswith(prefixes)}
    _, unexpected = model.load_state_dict(rest, strict=False)
    if unexpected:
        print(f"[pare] load_quantized: {len(unexpected)} unexpected keys (ignored)")
    print(f"[pare] Loaded {len(meta)} quantized layers from {src}")
    return model
