"""pare_b200 — the quantized-inference hot path of Pare on B200 (sm_100a).

Same names as the reference's top-level package (``pare/__init__.py:7-18``) for everything on
the run-time path: ``QuantConfig``, ``QuantDtype``, ``QuantizedLinear`` (via
``pare_b200.layers``), ``save_quantized`` / ``load_quantized``, ``KVCacheConfig`` /
``QuantizedKVCache``.  ``quantize`` covers round-to-nearest only: the calibration-based
solvers (GPTQ, AWQ, SmoothQuant) are offline tools that end in the same ``QuantizedLinear``
buffers and are not part of this package.
"""

from __future__ import annotations

import re

import torch.nn as nn

__version__ = "0.1.3+b200.0"

from pare_b200.config import QuantConfig
from pare_b200.core.dtype import QuantDtype
from pare_b200.kv_cache import KVCacheConfig, QuantizedKVCache
from pare_b200.layers.linear import QuantizedLinear
from pare_b200.model.io import load_quantized, save_quantized

__all__ = [
    "QuantConfig", "QuantDtype", "QuantizedLinear", "quantize",
    "save_quantized", "load_quantized", "KVCacheConfig", "QuantizedKVCache", "__version__",
]


def quantize(model: nn.Module, config: QuantConfig, calibration_data=None, device: str = "cpu") -> nn.Module:
    """Replace ``nn.Linear`` layers by round-to-nearest ``QuantizedLinear`` layers, in place.

    Layer selection follows the reference (``pare/schemes/base.py:47-93``): names matching any
    ``config.modules`` regex (all linears when ``None``) and containing none of
    ``config.exclude``.  Only ``scheme="rtn"`` is implemented here.
    """
    if config.scheme != "rtn":
        raise NotImplementedError(
            f"scheme={config.scheme!r}: calibration-based schemes are offline tools outside this package; "
            "quantize with the reference and load the result with load_quantized()"
        )
    targets = []
    for name, mod in model.named_modules():
        if not isinstance(mod, nn.Linear):
            continue
        if any(ex in name for ex in config.exclude):
            continue
        if config.modules is not None and not any(re.search(pat, name) for pat in config.modules):
            continue
        targets.append((name, mod))
    for name, mod in targets:
        parent = model
        *parents, leaf = name.split(".")
        for part in parents:
            parent = getattr(parent, part)
        setattr(parent, leaf, QuantizedLinear.from_linear(mod, config))
    print(f"[pare] Quantized {len(targets)} linear layers (rtn, {config.bits}-bit)")
    return model
