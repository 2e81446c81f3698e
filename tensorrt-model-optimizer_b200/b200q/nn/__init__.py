"""Quantised modules (reference: modelopt/torch/quantization/nn/)."""
from .tensor_quantizer import SequentialQuantizer, TensorQuantizer
from .quant_linear import QuantLinear, RealQuantLinear, QuantModule, is_quantized_linear

__all__ = ["TensorQuantizer", "SequentialQuantizer", "QuantLinear", "RealQuantLinear", "QuantModule",
           "is_quantized_linear"]
