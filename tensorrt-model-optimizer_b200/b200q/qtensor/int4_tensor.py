"""INT4 (AWQ) quantised tensor (reference: modelopt/torch/quantization/qtensor/int4_tensor.py:28-130)."""
from __future__ import annotations

import math

import torch

from .. import ops
from ..utils import reduce_block_padding
from .base_qtensor import BaseQuantizedTensor

__all__ = ["INT4QTensor"]


class INT4QTensor(BaseQuantizedTensor):
    @classmethod
    def quantize(cls, input: torch.Tensor, block_size: int):
        """-> (INT4QTensor, scales [nblocks, 1] in the input dtype, scales = 7 / block_amax)."""
        assert input.shape[-1] % 2 == 0, "Input tensor must have even number on last dimension."
        flat = reduce_block_padding(input.reshape(-1), {-1: block_size})
        packed, scales = ops.int4_quantize(flat, block_size)
        packed = packed.reshape(*input.shape[:-1], -1)
        return cls(input.shape, input.dtype, packed), scales

    def dequantize(self, dtype=None, **kwarg):
        dtype = dtype or self.metadata["dtype"]
        scales, block = kwarg["scale"], kwarg["block_sizes"][-1]
        out = ops.int4_dequantize(self._quantized_data.reshape(-1), scales.to(self._quantized_data.device), block)
        n = math.prod(self.metadata["shape"])
        return out[:n].reshape(self.metadata["shape"]).to(dtype)
