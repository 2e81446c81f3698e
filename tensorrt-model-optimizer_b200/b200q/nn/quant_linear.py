"""Quantised linear layer (reference: modelopt/torch/quantization/nn/modules/quant_linear.py:38-312
and quant_module.py:102-169).

``QuantLinear.convert`` patches the class of an existing ``nn.Linear`` in place (same parameters,
same state-dict keys) and adds ``input_quantizer``, ``weight_quantizer`` and ``output_quantizer``
children.  The forward is ``F.linear(input_quantizer(x), weight_quantizer(W), b)``.
"""
from __future__ import annotations

import warnings

import torch
import torch.nn.functional as F
from torch import nn

from ..config import QuantizerAttributeConfig
from ..qtensor import QTensorWrapper
from .tensor_quantizer import TensorQuantizer

__all__ = ["QuantModule", "QuantLinear", "RealQuantLinear", "is_quantized_linear"]


class QuantModule(nn.Module):
    """Marker base class of converted modules."""


class QuantLinear(nn.Linear, QuantModule):
    default_quant_desc_input = QuantizerAttributeConfig(num_bits=8)
    default_quant_desc_weight = QuantizerAttributeConfig(num_bits=8, axis=0)
    default_quant_desc_output = QuantizerAttributeConfig(num_bits=8)

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None, quant_desc_input=None,
                 quant_desc_weight=None, quant_desc_output=None):
        """Build a quantised linear layer directly (the reference's legacy constructor with
        ``quant_desc_*`` descriptors, nn/modules/quant_linear.py and quant_module.py); ``convert`` is the
        way an existing ``nn.Linear`` becomes one."""
        nn.Linear.__init__(self, in_features, out_features, bias=bias, device=device, dtype=dtype)
        self._original_cls = nn.Linear
        self._setup(quant_desc_input, quant_desc_weight, quant_desc_output)

    @classmethod
    def convert(cls, module: nn.Linear) -> "QuantLinear":
        """Turn ``module`` into a QuantLinear in place and return it."""
        assert isinstance(module, nn.Linear)
        module._original_cls = type(module)
        module.__class__ = cls
        module._setup()
        return module

    def _setup(self, quant_desc_input=None, quant_desc_weight=None, quant_desc_output=None):
        self.input_quantizer = TensorQuantizer(quant_desc_input or self.default_quant_desc_input)
        self.weight_quantizer = TensorQuantizer(quant_desc_weight or self.default_quant_desc_weight)
        self.output_quantizer = TensorQuantizer(quant_desc_output or self.default_quant_desc_output)
        self.output_quantizer.disable()
        dev = self.weight.device
        if dev.type != "meta":
            for q in (self.input_quantizer, self.weight_quantizer, self.output_quantizer):
                q.to(dev)

    def restore(self) -> nn.Linear:
        """Undo :meth:`convert` (drops the quantisers)."""
        for n in ("input_quantizer", "weight_quantizer", "output_quantizer"):
            delattr(self, n)
        self.__class__ = self._original_cls
        return self

    def _quantized_weight(self):
        w = self.weight
        if isinstance(w, QTensorWrapper):
            return self.weight_quantizer(w)
        return self.weight_quantizer(w)

    def forward(self, input, *args, **kwargs):
        x = self.input_quantizer(input)
        out = F.linear(x, self._quantized_weight(), self.bias)
        return self.output_quantizer(out)


class RealQuantLinear(QuantLinear):
    """QuantLinear whose weight is stored packed (after ``compress``).  The forward runs a
    registered real-quant GEMM on the packed weight when one is enabled and applies
    (``backends.enable_real_quant_gemm``; reference quant_linear.py:191-239), else dequantises the
    weight through the weight quantiser."""

    allow_real_quant_gemm = True

    @property
    def _should_run_real_quant_gemm(self):
        iq = self.input_quantizer
        return (getattr(self, "_use_real_quant_gemm", False) and self.allow_real_quant_gemm
                and not (iq.is_enabled and iq._if_calib))

    def has_real_quant_gemm_impl(self, input, *args, **kwargs) -> bool:
        if not hasattr(self, "_real_quant_gemm_impl"):      # matched once, then kept
            from .. import backends
            self._real_quant_gemm_impl = backends.gemm_registry.find_match(self, input, *args, **kwargs)
            if self._real_quant_gemm_impl is None:
                warnings.warn(f"RealQuantLinear: no real-quant GEMM found: {self}.")
        return self._real_quant_gemm_impl is not None

    def forward(self, input, *args, **kwargs):
        from ..utils import is_torch_export_mode

        if is_torch_export_mode():      # torch.export traces the fake-quantisation forward
            return super().forward(input, *args, **kwargs)
        if (self._should_run_real_quant_gemm and input.numel() > 1
                and self.has_real_quant_gemm_impl(input, *args, **kwargs)):
            out = self._real_quant_gemm_impl(self, input, self.weight, self.bias, *args, **kwargs)
            return self.output_quantizer(out)
        return super().forward(input, *args, **kwargs)

    def _quantized_weight(self):
        w = self.weight
        if isinstance(w, QTensorWrapper):
            return self.weight_quantizer(w)
        return super()._quantized_weight()


def is_quantized_linear(module) -> bool:
    return (isinstance(module, QuantModule) and isinstance(getattr(module, "input_quantizer", None), TensorQuantizer)
            and hasattr(module, "weight_quantizer") and getattr(module, "weight", None) is not None
            and module.weight.dim() == 2)
