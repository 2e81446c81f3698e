"""Base classes of the real-quantised tensors (reference:
modelopt/torch/quantization/qtensor/base_qtensor.py:39-229)."""
from __future__ import annotations

import torch

__all__ = ["BaseQuantizedTensor", "QTensorWrapper", "pack_real_quantize_weight"]


class BaseQuantizedTensor:
    """Packed data plus the shape and dtype of the tensor it came from."""

    _quantized_data: torch.Tensor

    def __init__(self, original_shape, original_dtype, quantized_data):
        self.metadata = {"shape": original_shape, "dtype": original_dtype}
        self._quantized_data = quantized_data

    @classmethod
    def quantize(cls, input, block_size):
        raise NotImplementedError

    def dequantize(self, dtype=None, **kwarg):
        raise NotImplementedError


class QTensorWrapper(torch.nn.Parameter):
    """Makes a quantised tensor usable as ``module.weight`` (an ``nn.Parameter`` over the packed
    bytes that carries the metadata needed to rebuild the quantised-tensor object)."""

    def __new__(cls, qtensor, metadata: dict | None = None):
        data = qtensor._quantized_data if isinstance(qtensor, BaseQuantizedTensor) else qtensor
        inst = super().__new__(cls, data, requires_grad=False)
        if metadata is None:
            inst.metadata = qtensor.metadata
            inst.metadata["qtensor_class"] = qtensor.__class__
        else:
            assert all(k in metadata for k in ("qtensor_class", "shape", "dtype")), f"metadata: {metadata}"
            inst.metadata = metadata
        return inst

    def dim(self):
        return len(self.metadata["shape"])

    def to(self, *args, **kwargs):
        device, dtype, *_ = torch._C._nn._parse_to(*args, **kwargs)
        if device:
            self.data = self.data.to(device=device)
        dtype = dtype if dtype else self.metadata["dtype"]
        return QTensorWrapper(self.metadata["qtensor_class"](self.metadata["shape"], dtype, self.data))

    def get_qtensor(self):
        return self.metadata["qtensor_class"](self.metadata["shape"], self.metadata["dtype"], self.data)

    def get_state(self):
        return {"metadata": self.metadata, "quantized_data.shape": self.data.shape,
                "quantized_data.dtype": self.data.dtype}


def pack_real_quantize_weight(module, force_quantize: bool = False):
    """Replace the weight of every sub-module whose weight quantiser is in real-quant mode by its
    packed form (the quantiser keeps the scales as buffers)."""
    from ..nn import SequentialQuantizer

    with torch.no_grad():
        for name, m in module.named_modules():
            wq = getattr(m, "weight_quantizer", None)
            if wq is None or getattr(m, "weight", None) is None or m.weight.is_meta:
                continue
            if isinstance(wq, SequentialQuantizer):
                wq = wq[0]
            if wq.is_enabled and not wq._fake_quant and m.weight.element_size() > 1:
                if force_quantize:
                    wq._dequantize = False
                m.weight = QTensorWrapper(wq(m.weight))
