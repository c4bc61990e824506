from pare_b200.model.io import load_quantized, save_quantized

__all__ = ["save_quantized", "load_quantized"]
