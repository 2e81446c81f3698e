"""FP8 per-tensor linear layer on the tensor cores (reference:
modelopt/torch/quantization/backends/fp8_per_tensor_gemm.py:35-207).

The activation is cast to E4M3 with scale ``amax / 448`` (``ops.fp8_gemm_operand``), the weight is
the compressed ``FP8QTensor`` (or is cast the same way), and one tcgen05 kernel computes
``out = a8 @ w8.T * scale_a * scale_b + bias`` (``ops.fp8_gemm``) in place of ``torch._scaled_mm``.
The cast follows the eager arithmetic of the reference's expression (fp32 scale, quotient rounded to
the activation's dtype, clamp, E4M3 cast; pinned by a fixture of the reference run on the CPU);
``ops.fp8_gemm_operand(..., fused=True)`` keeps the quotient in fp32 as a compiled graph does."""
from __future__ import annotations

import torch
from torch.autograd import Function

from .. import ops
from ..config import FP8_DEFAULT_CFG
from ..qtensor import FP8QTensor, QTensorWrapper
from .gemm_registry import gemm_registry
from .utils import fp8_compatible

__all__ = ["fp8_per_tensor_gemm", "Fp8PerTensorLinear"]


def _scale_from(quantizer, tensor) -> torch.Tensor:
    amax = quantizer.amax
    if amax is None:
        amax = ops.amax_tensor(tensor)
    return amax.detach().float().reshape(()).to(tensor.device) / 448.0


def fp8_per_tensor_gemm(quant_module, input, bias=None):
    """``input [..., k]`` times the module's weight ``[n, k]`` through the FP8 GEMM."""
    iq, wq = quant_module.input_quantizer, quant_module.weight_quantizer
    if not (hasattr(quant_module, "_scale_a") and iq.amax is not None):      # dynamic scales are not cached
        quant_module._scale_a = _scale_from(iq, input)
    weight = quant_module.weight
    compressed = isinstance(weight, QTensorWrapper)
    if compressed:
        quant_module._scale_b = wq._scale.detach().float().reshape(())
        weight_fp8 = weight.data
    else:
        if not (hasattr(quant_module, "_scale_b") and wq.amax is not None):
            quant_module._scale_b = _scale_from(wq, weight)
        weight_fp8 = ops.fp8_gemm_operand(weight.detach(), quant_module._scale_b)
    out_dtype = input.dtype
    x2 = input.reshape(-1, input.shape[-1])
    a8 = ops.fp8_gemm_operand(x2, quant_module._scale_a)
    out = ops.fp8_gemm(a8, weight_fp8.reshape(-1, weight_fp8.shape[-1]), quant_module._scale_a, quant_module._scale_b,
                       bias, out_dtype)
    return out.reshape(*input.shape[:-1], out.shape[-1])


def _matches(quantizer, cfg: dict) -> bool:
    return all(hasattr(quantizer, k) and getattr(quantizer, k) == v for k, v in cfg.items() if k != "enable")


def _fp8_availability_check(module, input, args, kwargs) -> bool:
    from ..nn import RealQuantLinear

    cfg = FP8_DEFAULT_CFG["quant_cfg"]
    if not (torch.cuda.is_available() and fp8_compatible() and input.is_cuda):
        return False
    if not isinstance(module, RealQuantLinear):
        return False
    if not (hasattr(module, "input_quantizer") and hasattr(module, "weight_quantizer")):
        return False
    if not (_matches(module.input_quantizer, cfg["*input_quantizer"])
            and _matches(module.weight_quantizer, cfg["*weight_quantizer"])):
        return False
    w = module.weight
    if isinstance(w, QTensorWrapper) and w.metadata["qtensor_class"] is not FP8QTensor:
        return False
    # the kernel's own limits: 16-byte operand rows and output vectors
    return input.shape[-1] % 16 == 0 and module.weight.shape[0] % 8 == 0


class Fp8PerTensorLinear(Function):
    """Autograd wrapper: forward through the FP8 GEMM, backward in high precision (the saved
    activation for the weight gradient, the dequantised weight for the input gradient)."""

    @staticmethod
    def forward(ctx, quant_module, input_tensor, weight, bias=None, allreduce_dgrad=False, tp_group=None):
        wq = quant_module.weight_quantizer
        ctx.save_for_backward(input_tensor if weight.requires_grad else None,
                              weight if input_tensor.requires_grad else None, getattr(wq, "_scale", None))
        ctx.compute_bias_grad = bias is not None and bias.requires_grad
        ctx.block_sizes = getattr(wq, "_block_sizes", None)
        ctx.allreduce_dgrad, ctx.tp_group = allreduce_dgrad, tp_group
        return fp8_per_tensor_gemm(quant_module, input_tensor, bias)

    @staticmethod
    def backward(ctx, grad_outputs):
        input_tensor, weight, scale = ctx.saved_tensors
        grad_input = grad_weight = grad_bias = None
        if weight is not None:
            if isinstance(weight, QTensorWrapper):
                weight = weight.get_qtensor().dequantize(scale=scale, block_sizes=ctx.block_sizes)
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


gemm_registry.register(gemm_func=Fp8PerTensorLinear.apply, availability_check=_fp8_availability_check)
