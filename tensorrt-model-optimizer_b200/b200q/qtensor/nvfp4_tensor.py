"""NVFP4 quantised tensor (reference: modelopt/torch/quantization/qtensor/nvfp4_tensor.py:31-297):
E2M1 values packed two per byte, an E4M3 scale per 16 elements, an fp32 scale per tensor."""
from __future__ import annotations

import torch

from .. import ops
from ..utils import reduce_amax, reduce_block_padding
from .base_qtensor import BaseQuantizedTensor

__all__ = ["NVFP4QTensor"]


def _scale2_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """amax / (6 * 448) in fp32 as a true division.  (Dividing a CUDA tensor by a Python number is
    evaluated by torch as a multiplication with the rounded reciprocal, which can differ from the
    quotient in the last bit; a tensor divisor keeps the IEEE division on every device.)"""
    a = amax.float()
    return a / torch.full((), 6.0 * 448.0, dtype=torch.float32, device=a.device)


class NVFP4QTensor(BaseQuantizedTensor):
    @classmethod
    def get_weights_scaling_factor_2_from_quantizer(cls, weight_quantizer):
        assert hasattr(weight_quantizer, "_amax"), "Weight quantizer does not have attribute amax"
        return _scale2_from_amax(weight_quantizer._amax)

    @classmethod
    def get_weights_scaling_factor_2(cls, input: torch.Tensor):
        """amax / (6 * 448) as fp32."""
        return _scale2_from_amax(reduce_amax(input))

    @classmethod
    def get_weights_scaling_factor(cls, input, block_size, weights_scaling_factor_2=None,
                                   keep_high_precision=False):
        """(per-block scale as float8_e4m3fn [..., K/block], weights_scaling_factor_2)."""
        assert input.shape[-1] % block_size == 0, (
            "Weight shape is not divisible for block size for block quantization.")
        if weights_scaling_factor_2 is None:
            weights_scaling_factor_2 = cls.get_weights_scaling_factor_2(input)
        if keep_high_precision:
            amax = ops.amax_blocks(input, block_size).reshape(*input.shape[:-1], -1)
            s = amax / (6.0 * weights_scaling_factor_2.to(amax.device))
            s[s == 0] = 1.0
            return s, weights_scaling_factor_2
        _, scales, _ = ops.nvfp4_quantize(input, scale2=weights_scaling_factor_2, block=block_size)
        return scales, weights_scaling_factor_2

    @classmethod
    def get_activation_scaling_factor(cls, quantizer):
        if not quantizer.is_enabled:
            return None
        amax = quantizer.export_amax()
        if amax is None:
            return None
        s = amax.float() / (quantizer.maxbound * 448.0)
        assert torch.all(s > 0), f" activation scaling factor {s} not positive."
        return s

    @classmethod
    def quantize(cls, input, block_size, weights_scaling_factor=None, weights_scaling_factor_2=None,
                 keep_high_precision=False, try_tensorrt=False):
        """-> (NVFP4QTensor, per-block scale float8_e4m3fn, per-tensor scale fp32).  One fused
        kernel (plus the abs-max pass when no per-tensor scale is given)."""
        shape, dtype = input.shape, input.dtype
        x = reduce_block_padding(input, {-1: block_size})
        if keep_high_precision:   # the scaled values before the 4-bit cast (a debugging aid of the reference)
            s2 = weights_scaling_factor_2 if weights_scaling_factor_2 is not None else cls.get_weights_scaling_factor_2(x)
            sc = weights_scaling_factor
            if sc is None:
                sc = cls.get_weights_scaling_factor(x, block_size, s2)[0]
            xb = x.reshape(*x.shape[:-1], -1, block_size)
            return (xb.float() / (sc.to(torch.float32) * s2.to(x.device)).unsqueeze(-1)).reshape(x.shape)
        packed, scales, s2 = ops.nvfp4_quantize(x, scale2=weights_scaling_factor_2,
                                                scales_in=weights_scaling_factor, block=block_size)
        if weights_scaling_factor is not None:
            scales = weights_scaling_factor
        if weights_scaling_factor_2 is not None:
            s2 = weights_scaling_factor_2
        return cls(shape, dtype, packed), scales, s2

    @classmethod
    def _cast_fp4(cls, weight: torch.Tensor) -> torch.Tensor:
        """The 4-bit E2M1 code (sign bit 8, magnitude index 0..7) of every element as uint8, ties between two
        grid values going to the even index (reference qtensor/nvfp4_tensor.py ``_cast_fp4``): the
        quantisation kernel run with unit scales, its packed pairs taken apart again."""
        block = 16
        x = reduce_block_padding(weight, {-1: block})
        ones = torch.ones(*x.shape[:-1], x.shape[-1] // block, device=x.device).to(torch.float8_e4m3fn)
        packed = cls.quantize(x, block, ones, torch.ones((), dtype=torch.float32, device=x.device))[0]._quantized_data
        codes = torch.stack((packed & 0xF, packed >> 4), dim=-1).reshape(x.shape)
        return codes[..., : weight.shape[-1]].contiguous()

    def dequantize(self, dtype=None, fast=False, **kwarg):
        """Needs ``scale`` (E4M3 per block), ``double_scale`` (fp32) and ``block_sizes``."""
        dtype = dtype or self.metadata["dtype"]
        out = ops.nvfp4_dequantize(self._quantized_data, kwarg["scale"], kwarg["double_scale"], dtype,
                                   block=kwarg["block_sizes"][-1])
        shape = self.metadata["shape"]
        if out.shape[-1] != shape[-1]:
            out = out[..., : shape[-1]]
        return out.reshape(shape)
