"""MXFP4 quantised tensor (reference: modelopt/torch/quantization/qtensor/mxfp4_tensor.py:28-143):
E2M1 values packed two per byte with one E8M0 (power-of-two) scale byte per block of 32."""
from __future__ import annotations

import torch

from .. import ops
from .base_qtensor import BaseQuantizedTensor

__all__ = ["MXFP4QTensor"]


class MXFP4QTensor(BaseQuantizedTensor):
    E2M1_max = 6.0
    E2M1_values = [0, 0.5, 1, 1.5, 2, 3, 4, 6]

    @classmethod
    def quantize(cls, input: torch.Tensor, block_size: int | None):
        """-> (MXFP4QTensor, e8m0 scale bytes [numel/block, 1])."""
        block_size = block_size or 32
        packed, scales = ops.mxfp4_quantize(input, block_size)
        return cls(input.shape, input.dtype, packed), scales

    def dequantize(self, dtype: torch.dtype = None, **kwarg):
        """value = sign * E2M1 magnitude * 2^(scale byte - 127), per block of ``block_sizes[-1]``."""
        dtype = dtype or self.metadata["dtype"]
        scale, block = kwarg["scale"], kwarg["block_sizes"][-1]
        q = self._quantized_data
        codes = torch.stack([q & 0x0F, (q >> 4) & 0x0F], dim=-1).reshape(*q.shape[:-1], -1)
        sign = 1 - 2 * ((codes & 0b1000) >> 3).to(torch.float32)
        values = torch.tensor(self.E2M1_values, device=q.device)
        x = sign * values[(codes & 0b0111).long()]
        shape = x.shape
        x = x.reshape(-1, block) * torch.exp2(scale.reshape(-1, 1).float() - 127)
        return x.reshape(shape).to(dtype)
