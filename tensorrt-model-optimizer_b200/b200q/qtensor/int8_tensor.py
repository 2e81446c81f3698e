"""INT8 quantised tensor (reference: modelopt/torch/quantization/qtensor/int8_tensor.py:28-124)."""
from __future__ import annotations

import torch

from .. import ops
from . import _scaled8
from .base_qtensor import BaseQuantizedTensor

__all__ = ["INT8QTensor"]


class INT8QTensor(BaseQuantizedTensor):
    @classmethod
    def quantize(cls, input, scales=None, axis=None, block_sizes=None):
        """-> (INT8QTensor, scales); scales = amax / 127 unless given."""
        x, scales, view = _scaled8.prepare(input, scales, axis, block_sizes, 127.0)
        if view is not None:
            q = ops.int8_quantize(x, scales, *view)
        else:
            q = ops.int8_quantize(x / _scaled8.expand(scales, x, block_sizes).to(x.dtype),
                                  torch.ones(1, dtype=x.dtype, device=x.device), 1, 1, x.numel())
        return cls(input.shape, input.dtype, q), scales

    def dequantize(self, dtype=None, **kwarg):
        dtype = dtype or self.metadata["dtype"]
        assert "scale" in kwarg, "Require scale for INT8 dequantization."
        scales, block_sizes = kwarg["scale"], kwarg.get("block_sizes")
        q = self._quantized_data
        if block_sizes:
            scales = _scaled8.expand(scales, q, block_sizes)
        sl = tuple(slice(0, d) for d in self.metadata["shape"])
        return (q.view(torch.int8).to(dtype) * scales.to(q.device).to(dtype))[sl]
