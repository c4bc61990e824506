from pare_b200.core.dtype import QuantDtype
from pare_b200.core.functional import dequantize_tensor, quantization_error, quantize_tensor
from pare_b200.core.pack import pack_int4, pack_int4_signed, unpack_int4, unpack_int4_signed
from pare_b200.core.scale import compute_scale

__all__ = [
    "QuantDtype", "quantize_tensor", "dequantize_tensor", "quantization_error", "compute_scale",
    "pack_int4", "unpack_int4", "pack_int4_signed", "unpack_int4_signed",
]
