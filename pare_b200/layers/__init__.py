from pare_b200.layers.linear import QuantizedLinear

__all__ = ["QuantizedLinear"]
