"""``QuantConfig`` — field-for-field the configuration object of the reference.

Reference: ``pare/config.py:14-100``.  All fields are kept (including the ones only
the offline GPTQ / AWQ / SmoothQuant solvers read) so configs written for the
reference construct unchanged and ``save_quantized`` metadata stays compatible.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from pare_b200.core.dtype import QuantDtype

_SCHEMES = ("rtn", "gptq", "awq", "smoothquant")
_CALIBRATIONS = ("absmax", "percentile", "mse")
_GRANULARITIES = ("per_tensor", "per_channel", "per_group")
_FP8 = (QuantDtype.FP8_E4M3, QuantDtype.FP8_E5M2)


@dataclass
class QuantConfig:
    # core
    bits: int = 4
    dtype: QuantDtype | None = None
    scheme: str = "awq"
    granularity: str = "per_group"
    group_size: int = 128
    sym: bool = False
    modules: list[str] | None = None
    exclude: list[str] = field(default_factory=lambda: ["lm_head"])
    # calibration
    n_calibration_samples: int = 128
    calibration_seq_len: int = 2048
    calibration: str = "absmax"
    calibration_percentile: float = 99.99
    # gptq
    damp_percent: float = 0.01
    act_order: bool = False
    # awq
    awq_n_grid: int = 20
    # smoothquant
    smooth_alpha: float = 0.5
    # mixed precision
    sensitive_bits: int | None = None
    sensitivity_threshold: float = 0.05

    def __post_init__(self) -> None:
        if self.dtype is None:
            self.dtype = QuantDtype.from_bits(self.bits)
        for value, allowed, what in (
            (self.scheme, _SCHEMES, "scheme"),
            (self.calibration, _CALIBRATIONS, "calibration"),
            (self.granularity, _GRANULARITIES, "granularity"),
        ):
            if value not in allowed:
                raise ValueError(f"Unknown {what}: {value!r}")
        if self.bits not in (2, 3, 4, 8):
            raise ValueError(f"Unsupported bits: {self.bits}")
        if self.dtype is QuantDtype.NF4:          # per-row absmax codebook
            self.bits, self.granularity = 4, "per_channel"
        if self.dtype in _FP8:                    # per-row symmetric
            self.bits, self.granularity, self.sym = 8, "per_channel", True

    @property
    def effective_dtype(self) -> QuantDtype:
        assert self.dtype is not None
        return self.dtype
