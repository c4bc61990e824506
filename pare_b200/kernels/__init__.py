from pare_b200.kernels.matmul_int4 import kernel_available, matmul_w4a16, triton_available, w4a16_forward

__all__ = ["matmul_w4a16", "w4a16_forward", "triton_available", "kernel_available"]
