"""Hardware checks of the GEMM back ends (reference: modelopt/torch/quantization/backends/utils.py)."""
import torch

__all__ = ["fp8_compatible", "fp4_compatible"]


def _capability():
    return torch.cuda.get_device_capability() if torch.cuda.is_available() else (0, 0)


def fp8_compatible() -> bool:
    return _capability() >= (8, 9)


def fp4_compatible() -> bool:
    return _capability() >= (10, 0)
