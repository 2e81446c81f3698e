"""FP8 E4M3 quantised tensor (reference: modelopt/torch/quantization/qtensor/fp8_tensor.py:33-151)."""
from __future__ import annotations

import torch

from .. import ops
from ..utils import reduce_block_padding
from . import _scaled8
from .base_qtensor import BaseQuantizedTensor

__all__ = ["FP8QTensor"]


class FP8QTensor(BaseQuantizedTensor):
    @classmethod
    def quantize(cls, input, scales=None, axis=None, block_sizes=None):
        """-> (FP8QTensor, scales); scales = amax / 448 unless given."""
        x, scales, view = _scaled8.prepare(input, scales, axis, block_sizes, 448.0)
        if view is not None:
            q = ops.fp8_quantize(x, scales, *view)
        else:  # N-D blocks: divide by the expanded scales, then the same cast kernel with scale 1
            q = ops.fp8_quantize(x / _scaled8.expand(scales, x, block_sizes).to(x.dtype),
                                 torch.ones(1, dtype=x.dtype, device=x.device), 1, 1, x.numel())
        q = q[tuple(slice(0, d) for d in input.shape)]
        return cls(input.shape, input.dtype, q), scales

    def dequantize(self, dtype=None, **kwarg):
        dtype = dtype or self.metadata["dtype"]
        assert "scale" in kwarg, "Require scale for FP8 dequantization."
        scales, block_sizes = kwarg["scale"], kwarg.get("block_sizes")
        q = self._quantized_data
        if block_sizes:
            q = reduce_block_padding(q.view(torch.uint8), block_sizes).view(torch.float8_e4m3fn)
            scales = _scaled8.expand(scales, q, block_sizes)
        sl = tuple(slice(0, d) for d in self.metadata["shape"])
        return (q.to(dtype) * scales.to(q.device).to(dtype))[sl]
