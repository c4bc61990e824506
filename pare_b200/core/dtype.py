"""Quantization number formats and their integer ranges.

Mirrors the public surface of the reference's ``pare/core/dtype.py:32-97``
(``QuantDtype`` members, ``bits/is_float/signed/qmin/qmax/levels`` properties and
``QuantDtype.from_bits``) so code written against the reference keeps working.
Only the INT4 member reaches the CUDA path; the others exist for API parity.
"""

from __future__ import annotations

import enum
from typing import NamedTuple


class _Format(NamedTuple):
    tag: str          # unique name, keeps FP8_E4M3 and FP8_E5M2 from aliasing in the Enum
    bits: int
    is_float: bool
    signed: bool


class QuantDtype(enum.Enum):
    """Formats a weight can be quantized to."""

    INT2 = _Format("int2", 2, False, False)
    INT3 = _Format("int3", 3, False, False)
    INT4 = _Format("int4", 4, False, False)
    INT8 = _Format("int8", 8, False, True)
    FP8_E4M3 = _Format("fp8_e4m3", 8, True, True)
    FP8_E5M2 = _Format("fp8_e5m2", 8, True, True)
    NF4 = _Format("nf4", 4, True, True)

    # -- properties -------------------------------------------------------
    @property
    def bits(self) -> int:
        return self.value.bits

    @property
    def is_float(self) -> bool:
        return self.value.is_float

    @property
    def signed(self) -> bool:
        return self.value.signed

    @property
    def levels(self) -> int:
        return 1 << self.value.bits

    def _require_integer(self) -> None:
        if self.value.is_float:
            raise TypeError("float dtypes have no integer qmin/qmax")

    @property
    def qmin(self) -> int:
        self._require_integer()
        return -(1 << (self.bits - 1)) if self.signed else 0

    @property
    def qmax(self) -> int:
        self._require_integer()
        return (1 << (self.bits - 1)) - 1 if self.signed else (1 << self.bits) - 1

    # -- factory ----------------------------------------------------------
    @classmethod
    def from_bits(cls, bits: int, *, signed: bool = False) -> "QuantDtype":
        """Standard integer format for a bit-width (8-bit is always the signed INT8)."""
        table = {2: cls.INT2, 3: cls.INT3, 4: cls.INT4, 8: cls.INT8}
        if bits not in table or (signed and bits != 8):
            raise ValueError(f"No standard dtype for bits={bits}, signed={signed}")
        return table[bits]
