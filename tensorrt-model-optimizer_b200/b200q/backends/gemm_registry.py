"""Registry of low-precision GEMM implementations (reference:
modelopt/torch/quantization/backends/gemm_registry.py:31-156).

An entry is a GEMM callable ``f(module, input, weight, bias, *args, **kwargs)`` plus a predicate
``check(module, input, args, kwargs)``; a ``RealQuantLinear`` asks the registry once for the first
entry whose predicate accepts it and keeps the answer.

The tensor-core kernels never synchronise: error bits of their bounded device-side waits collect in
a per-device status word, which ``backends.check_gemm_status(device)`` reads (and raises on)."""
from __future__ import annotations

from typing import Callable

from torch import nn

__all__ = ["GEMMRegistry", "gemm_registry", "enable_real_quant_gemm", "disable_real_quant_gemm",
           "is_real_quant_gemm_enabled"]


class GEMMRegistry:
    def __init__(self):
        self._registry: list[dict] = []

    def register(self, gemm_func: Callable, availability_check: Callable | None = None) -> None:
        self._registry.append({"gemm_func": gemm_func,
                               "availability_check": availability_check or (lambda module, input, args, kwargs: True)})

    def unregister(self, gemm_func: Callable) -> None:
        self._registry = [e for e in self._registry if e["gemm_func"] != gemm_func]

    def find_match(self, module: nn.Module, input, *args, **kwargs) -> Callable | None:
        for e in self._registry:
            if e["availability_check"](module, input, args, kwargs):
                return e["gemm_func"]
        return None

    def __contains__(self, gemm_func: Callable) -> bool:
        return any(e["gemm_func"] == gemm_func for e in self._registry)


gemm_registry = GEMMRegistry()


def _both_quantizers_enabled(module) -> bool:
    iq, wq = getattr(module, "input_quantizer", None), getattr(module, "weight_quantizer", None)
    return bool(iq is not None and wq is not None and iq.is_enabled and wq.is_enabled)


def enable_real_quant_gemm(model: nn.Module) -> None:
    """Mark every module whose input and weight quantisers are both enabled to use a registered
    real-quant GEMM."""
    for module in model.modules():
        if _both_quantizers_enabled(module):
            module._use_real_quant_gemm = True


def disable_real_quant_gemm(model: nn.Module) -> None:
    for module in model.modules():
        if hasattr(module, "_use_real_quant_gemm"):
            module._use_real_quant_gemm = False


def is_real_quant_gemm_enabled(model: nn.Module) -> bool:
    return any(getattr(module, "_use_real_quant_gemm", False) for module in model.modules())
