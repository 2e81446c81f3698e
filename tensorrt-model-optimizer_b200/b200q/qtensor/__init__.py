"""Real-quantised tensor classes with the interface of ``modelopt/torch/quantization/qtensor``."""
from .base_qtensor import BaseQuantizedTensor, QTensorWrapper, pack_real_quantize_weight
from .fp8_tensor import FP8QTensor
from .int4_tensor import INT4QTensor
from .int8_tensor import INT8QTensor
from .mxfp4_tensor import MXFP4QTensor
from .nvfp4_tensor import NVFP4QTensor

__all__ = ["BaseQuantizedTensor", "QTensorWrapper", "pack_real_quantize_weight", "NVFP4QTensor",
           "INT4QTensor", "FP8QTensor", "INT8QTensor", "MXFP4QTensor"]
