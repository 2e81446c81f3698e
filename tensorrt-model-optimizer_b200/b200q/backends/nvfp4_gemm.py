"""NVFP4 linear layer on the tensor cores (reference:
modelopt/torch/quantization/backends/nvfp4_gemm.py:31-257).

The reference hands this to TensorRT-LLM (``fp4_quantize`` + ``nvfp4_gemm``); here the activation is
quantised by the NVFP4 kernel of this package (two-level scaling with the input quantiser's amax,
the arithmetic of ``NVFP4QTensor.quantize``), its block scales are tiled by
``ops.nvfp4_swizzle_scales`` and one block-scaled tcgen05 kernel computes
``out = alpha * (a4 * sfa) @ (w4 * sfb).T`` (``ops.nvfp4_gemm``), alpha the product of the two
per-tensor scales."""
from __future__ import annotations

import torch
from torch.autograd import Function

from .. import ops
from ..config import NVFP4_DEFAULT_CFG
from ..qtensor import NVFP4QTensor, QTensorWrapper
from .gemm_registry import gemm_registry
from .utils import fp4_compatible

__all__ = ["nvfp4_gemm", "Nvfp4Linear"]


def _weight_operand(quant_module):
    """(packed codes [n, k/2], tiled block scales, per-tensor scale) of the module's weight; the
    tiled scales of a compressed weight are cached until its ``_scale`` buffer is replaced."""
    wq, weight = quant_module.weight_quantizer, quant_module.weight
    if isinstance(weight, QTensorWrapper):
        assert weight.metadata["qtensor_class"] is NVFP4QTensor
        key = (wq._scale.data_ptr(), wq._scale._version)
        cached = getattr(quant_module, "_weight_scale_tiled", None)
        if cached is None or cached[0] != key:
            cached = (key, ops.nvfp4_swizzle_scales(wq._scale.reshape(-1, wq._scale.shape[-1])))
            quant_module._weight_scale_tiled = cached
        return weight.data.reshape(-1, weight.data.shape[-1]), cached[1], wq._double_scale.detach().float().reshape(())
    w = weight.detach()
    if w.dtype == torch.float32:
        w = w.to(torch.float16)
    packed, scales, s2 = ops.nvfp4_quantize(w, amax=wq.amax)
    return packed, ops.nvfp4_swizzle_scales(scales), s2


def nvfp4_gemm(quant_module, input_tensor, bias=None):
    """``input [..., k]`` times the module's weight ``[n, k]`` through the NVFP4 GEMM."""
    if input_tensor.dtype == torch.float32:
        input_tensor = input_tensor.to(torch.float16)
    x2 = input_tensor.reshape(-1, input_tensor.shape[-1])
    # activations may exceed the calibrated amax: their block scales saturate, as in the fake-quant path
    a4, sfa, s2a = ops.nvfp4_quantize(x2, amax=quant_module.input_quantizer.amax, saturate_scales=True)
    b4, sfb_tiled, s2b = _weight_operand(quant_module)
    quant_module.alpha = s2a * s2b
    out = ops.nvfp4_gemm(a4, ops.nvfp4_swizzle_scales(sfa), b4, sfb_tiled, quant_module.alpha, bias, x2.dtype)
    return out.reshape(*input_tensor.shape[:-1], out.shape[-1])


def _matches(quantizer, cfg: dict) -> bool:
    return all(hasattr(quantizer, k) and getattr(quantizer, k) == v for k, v in cfg.items() if k != "enable")


def _nvfp4_availability_check(module, input, args, kwargs) -> bool:
    from ..nn import RealQuantLinear

    cfg = NVFP4_DEFAULT_CFG["quant_cfg"]
    if not (torch.cuda.is_available() and fp4_compatible() and input.is_cuda):
        return False
    if not isinstance(module, RealQuantLinear):
        return False
    if not (hasattr(module, "input_quantizer") and hasattr(module, "weight_quantizer")):
        return False
    if not (_matches(module.input_quantizer, cfg["*input_quantizer"])
            and _matches(module.weight_quantizer, cfg["*weight_quantizer"])):
        return False
    # the shapes the reference's back end accepts, which the kernel's own limits (k % 32, n % 8) include
    if input.shape[-1] % 64 != 0 or module.weight.shape[0] % 32 != 0:
        return False
    return module.input_quantizer.block_sizes[-1] == 16 and module.weight_quantizer.block_sizes[-1] == 16


class Nvfp4Linear(Function):
    """Autograd wrapper: forward through the NVFP4 GEMM, backward in high precision."""

    @staticmethod
    def forward(ctx, quant_module, input_tensor, weight, bias=None, allreduce_dgrad=False, tp_group=None):
        wq = quant_module.weight_quantizer
        ctx.save_for_backward(input_tensor if weight.requires_grad else None,
                              weight if input_tensor.requires_grad else None,
                              getattr(wq, "_scale", None), getattr(wq, "_double_scale", None))
        ctx.compute_bias_grad = bias is not None and bias.requires_grad
        ctx.allreduce_dgrad, ctx.tp_group = allreduce_dgrad, tp_group
        return nvfp4_gemm(quant_module, input_tensor, bias)

    @staticmethod
    def backward(ctx, grad_outputs):
        input_tensor, weight, scale, double_scale = ctx.saved_tensors
        grad_input = grad_weight = grad_bias = None
        if weight is not None:
            if isinstance(weight, QTensorWrapper):
                weight = weight.get_qtensor().dequantize(scale=scale, double_scale=double_scale,
                                                         block_sizes={-1: 16})
            grad_input = grad_outputs @ weight
        if input_tensor is not None:
            g2 = grad_outputs.reshape(-1, grad_outputs.shape[-1])
            grad_weight = g2.T @ input_tensor.reshape(-1, input_tensor.shape[-1])
        if ctx.compute_bias_grad:
            grad_bias = grad_outputs.sum(dim=list(range(grad_outputs.dim() - 1)))
        if ctx.allreduce_dgrad and grad_input is not None:
            torch.distributed.all_reduce(grad_input, group=ctx.tp_group)
        return None, grad_input, grad_weight, grad_bias, None, None

    @classmethod
    def apply(cls, *args, **kwargs):
        return super().apply(*args, *kwargs.values())


gemm_registry.register(gemm_func=Nvfp4Linear.apply, availability_check=_nvfp4_availability_check)
