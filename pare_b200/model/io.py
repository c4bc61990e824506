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

import torch
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


def load_quantized(model: nn.Module, path: str | Path, use_kernel: bool = False, *, tp_plan: dict[str, str] | None = None,
                   tp_rank: int = 0, tp_world: int = 1) -> nn.Module:
    """Swap the named modules of ``model`` for ``QuantizedLinear`` layers rebuilt from ``path`` and
    load every other tensor; ``use_kernel=True`` puts the rebuilt layers on the CUDA path.

    Tensor-parallel loading: ``tp_plan`` maps the last component of a layer name (``"q_proj"``, ``"down_proj"`` ...)
    to ``"column"`` (split output rows) or ``"row"`` (split input columns in whole groups); with ``tp_world > 1``
    every listed layer is rebuilt from this rank's slice only, which is read straight from the file
    (``safetensors`` slices, nothing else of the tensor is materialised).  The slices are those of
    :func:`pare_b200.parallel.shard_linear`.
    """
    from safetensors import safe_open
    from safetensors.torch import load_file

    from pare_b200.config import QuantConfig
    from pare_b200.layers.linear import QuantizedLinear
    from pare_b200.parallel import shard_range

    src = Path(path)
    meta = json.loads((src / CONFIG_FILE).read_text())["quantized_layers"]
    sharded = tp_world > 1 and bool(tp_plan)
    tensors = {} if sharded else load_file(src / TENSORS_FILE)
    handle = safe_open(src / TENSORS_FILE, framework="pt") if sharded else None
    keys = set(handle.keys()) if sharded else set(tensors)

    def whole(key):
        if key not in keys:
            return None
        return handle.get_tensor(key) if sharded else tensors[key]

    for name, info in meta.items():
        cfg = QuantConfig(**{k: info[k] for k in _LAYER_KEYS if k in info})
        n_out, n_in = info["out_features"], info["in_features"]
        mode = (tp_plan or {}).get(name.split(".")[-1]) if sharded else None
        if mode is None:
            t = lambda suffix: whole(f"{name}.{suffix}")
            parts = dict(packed_weight=t("packed_weight"), q_weight=t("q_weight"), scale=t("scale"), zero=t("zero"),
                         bias=t("bias"), g_idx=t("g_idx"), input_scale=t("input_scale"))
        else:
            if f"{name}.packed_weight" not in keys:
                raise ValueError(f"{name}: only INT4 (packed) layers can be loaded tensor-parallel")
            sl = lambda suffix: handle.get_slice(f"{name}.{suffix}") if f"{name}.{suffix}" in keys else None
            packed, scale, zero, bias = sl("packed_weight"), sl("scale"), sl("zero"), sl("bias")
            per_group = cfg.granularity == "per_group"
            zero_dim = len(scale.get_shape()) == 0
            if mode == "column":
                a, b = shard_range(n_out, tp_rank, tp_world)
                parts = dict(packed_weight=packed[a:b], q_weight=None,
                             scale=whole(f"{name}.scale") if zero_dim else scale[a:b],
                             zero=whole(f"{name}.zero") if zero_dim else zero[a:b],
                             bias=None if bias is None else bias[a:b],
                             g_idx=whole(f"{name}.g_idx"), input_scale=whole(f"{name}.input_scale"))
                n_out = b - a
            elif mode == "row":
                if f"{name}.g_idx" in keys:
                    raise ValueError(f"{name}: row-parallel loading of an act-order layer is not supported")
                group = cfg.group_size if per_group else 2
                a, b = shard_range(n_in, tp_rank, tp_world, multiple=group)
                isc = sl("input_scale")
                parts = dict(packed_weight=packed[:, a // 2:b // 2], q_weight=None,
                             scale=scale[:, a // group:b // group] if per_group else whole(f"{name}.scale"),
                             zero=zero[:, a // group:b // group] if per_group else whole(f"{name}.zero"),
                             bias=whole(f"{name}.bias") if tp_rank == 0 else None,
                             g_idx=None, input_scale=None if isc is None else isc[a:b])
                n_in = b - a
            else:
                raise ValueError(f"{name}: unknown tensor-parallel mode {mode!r}")
            parts = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in parts.items()}
        layer = QuantizedLinear.from_tensors(
            packed_weight=parts["packed_weight"], q_weight=parts["q_weight"], scale=parts["scale"], zero=parts["zero"],
            config=cfg, bias=parts["bias"], in_features=n_in, out_features=n_out,
            quantize_inputs=info.get("quantize_inputs", False), g_idx=parts["g_idx"], input_scale=parts["input_scale"],
        )
        layer.use_kernel = use_kernel
        parent = model
        *parents, leaf = name.split(".")
        for part in parents:
            parent = getattr(parent, part)
        setattr(parent, leaf, layer)

    if sharded:
        tensors = {k: handle.get_tensor(k) for k in keys if not k.startswith(tuple(n + "." for n in meta))}
    prefixes = tuple(n + "." for n in meta)
    rest = {k: v for k, v in tensors.items() if not k.startswith(prefixes)}
    _, unexpected = model.load_state_dict(rest, strict=False)
    if unexpected:
        print(f"[pare] load_quantized: {len(unexpected)} unexpected keys (ignored)")
    print(f"[pare] Loaded {len(meta)} quantized layers from {src}")
    return model
