"""Element dtype codes of the C ABI (CUDAElementDType, device/cuda/internal/bridge/core.h:26-33)."""
Float32, Float16, BFloat16, Float64, Float8E4M3, Float8E5M2 = 0, 1, 2, 3, 4, 5

SIZE = {Float32: 4, Float16: 2, BFloat16: 2, Float64: 8, Float8E4M3: 1, Float8E5M2: 1}
NAME = {Float32: "f32", Float16: "f16", BFloat16: "bf16", Float64: "f64", Float8E4M3: "e4m3", Float8E5M2: "e5m2"}


def torch_dtype(code):
    import torch

    return {Float32: torch.float32, Float16: torch.float16, BFloat16: torch.bfloat16, Float64: torch.float64,
            Float8E4M3: torch.float8_e4m3fn, Float8E5M2: torch.float8_e5m2}[code]


def bits_dtype(code):
    """Integer numpy dtype that carries the raw bit pattern of an element."""
    import numpy as np

    return {Float32: np.uint32, Float16: np.uint16, BFloat16: np.uint16, Float8E4M3: np.uint8, Float8E5M2: np.uint8}[code]
