"""Functional fake-quantisation layer with the names and argument order of
``modelopt/torch/quantization/tensor_quant.py``: ``fake_tensor_quant``, ``scaled_e4m3``,
``dynamic_block_quant`` (autograd functions with the straight-through backward, lines 293-571)
over torch custom ops ``b200q::quantize_op`` / ``b200q::dynamic_block_quantize_op`` (lines 226-273),
which call the CUDA kernels.  CUDA tensors only."""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import ops

__all__ = ["normalized_hadamard_transform", "fake_tensor_quant", "scaled_e4m3", "dynamic_block_quant", "quantize_op",
           "dynamic_block_quantize_op"]


@torch.library.custom_op("b200q::quantize_op", mutates_args=())
def quantize_op(input: torch.Tensor, amax: torch.Tensor, num_bits: int = 8, exponent_bits: int = 0,
                unsigned: bool = False, narrow_range: bool = True) -> torch.Tensor:
    if input.dtype == torch.float64:
        # the reference kernels take a double tensor and compute on its float cast
        # (modelopt/torch/quantization/src/tensor_quant_gpu.cu:29-44,64-78): same here, around the fp32 kernel
        return quantize_op(input.float(), amax, num_bits, exponent_bits, unsigned, narrow_range).double()
    if num_bits == 8 and exponent_bits == 4:
        return ops.fake_e4m3(input, amax)
    if exponent_bits == 0:
        return ops.fake_int(input, amax, num_bits, unsigned, narrow_range)
    raise ValueError(f"Invalid combination of (num_bits, exponent_bits): ({num_bits}, {exponent_bits}).")


@quantize_op.register_fake
def _(input, amax, num_bits=8, exponent_bits=0, unsigned=False, narrow_range=True):
    return torch.empty_like(input)


@torch.library.custom_op("b200q::e4m3_cast_op", mutates_args=())
def e4m3_cast_op(input: torch.Tensor) -> torch.Tensor:
    return ops.fake_e4m3(input, None)


@e4m3_cast_op.register_fake
def _(input):
    return torch.empty_like(input)


@torch.library.custom_op("b200q::dynamic_block_quantize_op", mutates_args=())
def dynamic_block_quantize_op(input: torch.Tensor, block_size: int, amax: torch.Tensor, num_bits: int,
                              exponent_bits: int, scale_num_bits: int,
                              scale_exponent_bits: int) -> torch.Tensor:
    fmt = (exponent_bits, num_bits - exponent_bits - 1)
    scale_fmt = (scale_exponent_bits, scale_num_bits - scale_exponent_bits - 1)
    if fmt == (2, 1) and scale_fmt == (4, 3) and block_size % 2 == 0:
        shape = input.shape
        x = input
        pad = (-shape[-1]) % block_size
        if pad:
            x = torch.nn.functional.pad(x, (0, pad))
        y = ops.nvfp4_fake(x, amax, block=block_size)
        return y[..., : shape[-1]].contiguous() if pad else y
    if scale_fmt == (8, 0):  # MX formats: power-of-two block scales, no global amax
        key = num_bits if exponent_bits == 0 else fmt
        if key in ops.MX_FORMATS:
            return ops.mx_fake(input, block_size, key)
    raise NotImplementedError(
        f"Unsupported num_bits: {fmt}, scale_bits: {scale_fmt}, block {block_size} for dynamic block "
        "quantization (built: NVFP4 = (2,1) values with (4,3) scales, and the MX formats with (8,0) scales).")


@dynamic_block_quantize_op.register_fake
def _(input, block_size, amax, num_bits, exponent_bits, scale_num_bits, scale_exponent_bits):
    return torch.empty_like(input)


def _backward(ctx, grad_outputs, num_args):
    """Straight-through estimator, clipped to |x| <= amax when the inputs were saved."""
    saved = ctx.saved_tensors
    if len(saved) == 0:
        return (grad_outputs,) + (None,) * (num_args - 1)
    inputs, amax = saved
    grad = torch.where(inputs.abs() <= amax, grad_outputs, grad_outputs.new_zeros(1))
    return (grad,) + (None,) * (num_args - 1)


def _save(ctx, pass_through_bwd, inputs, amax):
    if not pass_through_bwd and amax is not None:
        if not isinstance(amax, torch.Tensor):
            amax = torch.tensor(amax, device=inputs.device, dtype=inputs.dtype)
        ctx.save_for_backward(inputs, amax)


def _as_tensor(amax, like):
    if isinstance(amax, torch.Tensor):
        return amax
    return torch.tensor(float(amax), device=like.device, dtype=torch.float32)


class FakeTensorQuantFunction(Function):
    """Integer fake quantisation (reference: FakeTensorQuantFunction, tensor_quant.py:322-402)."""

    @staticmethod
    def forward(ctx, inputs, amax, bias=None, num_bits=8, unsigned=False, narrow_range=True,
                trt_high_precision_dtype=None, pass_through_bwd=False, block_size=None, axis=None):
        if bias is not None:
            inputs = inputs - bias
        _save(ctx, pass_through_bwd, inputs, amax)
        # amax is validated (non-negative, finite) where it is produced: a check here would cost a
        # device synchronisation on every call
        outputs = quantize_op(inputs, _as_tensor(amax, inputs), num_bits, 0, unsigned, narrow_range)
        if bias is not None:
            outputs = outputs + bias
        return outputs

    @staticmethod
    def backward(ctx, grad_outputs):
        return _backward(ctx, grad_outputs, 10)


class ScaledE4M3Function(Function):
    """FP8 E4M3 fake quantisation (reference: ScaledE4M3Function, tensor_quant.py:405-463)."""

    @staticmethod
    def forward(ctx, inputs, amax, bias, E, M, trt_high_precision_dtype=None, pass_through_bwd=False):  # noqa: N803
        if E != 4 or M != 3:
            raise NotImplementedError("Only support E=4 & M=3 for now.")
        if bias is not None:
            inputs = inputs - bias
        _save(ctx, pass_through_bwd, inputs, amax)
        if amax is None:
            outputs = e4m3_cast_op(inputs)
        else:
            outputs = quantize_op(inputs, _as_tensor(amax, inputs), 8, 4, False, False)
        if bias is not None:
            outputs = outputs + bias
        return outputs

    @staticmethod
    def backward(ctx, grad_outputs):
        return _backward(ctx, grad_outputs, 7)


class DynamicBlockQuantizationFunction(Function):
    """Dynamic block fake quantisation (reference: tensor_quant.py:466-571)."""

    @staticmethod
    def forward(ctx, inputs, block_size, amax, bias, num_bits, scale_bits, trt_high_precision_dtype=None,
                onnx_quantizer_type="dynamic", pass_through_bwd=True):
        _save(ctx, pass_through_bwd, inputs, amax)
        if isinstance(num_bits, int):
            exponent_bits, nb = 0, num_bits
        else:
            exponent_bits, nb = num_bits[0], num_bits[0] + num_bits[1] + 1
        if amax is None:  # MX formats carry no global amax; the op needs a tensor argument
            amax = (ops.amax_tensor(inputs) if tuple(scale_bits) != (8, 0)
                    else torch.zeros((), dtype=torch.float32, device=inputs.device))
        return dynamic_block_quantize_op(inputs, block_size, _as_tensor(amax, inputs), nb, exponent_bits,
                                         scale_bits[0] + scale_bits[1] + 1, scale_bits[0])

    @staticmethod
    def backward(ctx, grad_outputs):
        return _backward(ctx, grad_outputs, 9)


class _HadamardFunction(Function):
    """H x along the last dimension; H is symmetric, so the backward is the same transform."""

    @staticmethod
    def forward(ctx, inputs, scale):
        ctx.scale = scale
        return ops.hadamard(inputs, scale)

    @staticmethod
    def backward(ctx, grad):
        return ops.hadamard(grad.contiguous(), ctx.scale), None


def normalized_hadamard_transform(inputs: torch.Tensor) -> torch.Tensor:
    """Hadamard rotation of the last dimension, scaled by 1/sqrt(n) (reference:
    modelopt/torch/quantization/nn/functional.py:75-109, which calls the third-party
    ``fast_hadamard_transform`` CUDA package and divides its output by sqrt(n))."""
    n = inputs.shape[-1]
    assert n & (n - 1) == 0, "Fast hadamard only works for inputs.shape[-1] == power of 2."
    return _HadamardFunction.apply(inputs, 1.0 / (n ** 0.5))


fake_tensor_quant = FakeTensorQuantFunction.apply
scaled_e4m3 = ScaledE4M3Function.apply
dynamic_block_quant = DynamicBlockQuantizationFunction.apply


def _register_reference_op_names():
    """Also expose the ops under the reference's names (``tensorrt::quantize_op``,
    ``tensorrt::dynamic_block_quantize_op`` and its ``.overload`` without a global amax,
    tensor_quant.py:226-273) so that code and exported
    graphs that refer to ``torch.ops.tensorrt.*`` resolve to these kernels.  Skipped when that
    namespace already defines them (the reference itself is imported in the same process)."""
    try:
        lib = torch.library.Library("tensorrt", "FRAGMENT")
        lib.define("quantize_op(Tensor input, Tensor amax, int num_bits, int exponent_bits, "
                   "bool unsigned, bool narrow_range) -> Tensor")
        lib.define("dynamic_block_quantize_op(Tensor input, int block_size, Tensor amax, int num_bits, "
                   "int exponent_bits, int scale_num_bits, int scale_exponent_bits) -> Tensor")
        lib.impl("quantize_op", lambda i, a, nb, eb, u, nr: quantize_op(i, a, nb, eb, u, nr), "CUDA")
        lib.impl("dynamic_block_quantize_op",
                 lambda i, bs, a, nb, eb, snb, seb: dynamic_block_quantize_op(i, bs, a, nb, eb, snb, seb), "CUDA")
        lib.define("dynamic_block_quantize_op.overload(Tensor input, int block_size, None amax, int num_bits, "
                   "int exponent_bits, int scale_num_bits, int scale_exponent_bits) -> Tensor")

        def _none_amax(i, bs, a, nb, eb, snb, seb):
            # no global amax: the MX formats need none, NVFP4 takes the tensor's own abs-max
            am = (torch.zeros((), dtype=torch.float32, device=i.device) if (seb, snb - seb - 1) == (8, 0)
                  else ops.amax_tensor(i))
            return dynamic_block_quantize_op(i, bs, am, nb, eb, snb, seb)

        lib.impl("dynamic_block_quantize_op.overload", _none_amax, "CUDA")
        lib.impl("dynamic_block_quantize_op.overload", lambda i, bs, a, nb, eb, snb, seb: torch.empty_like(i), "Meta")
        lib.impl("quantize_op", lambda i, a, nb, eb, u, nr: torch.empty_like(i), "Meta")
        lib.impl("dynamic_block_quantize_op", lambda i, bs, a, nb, eb, snb, seb: torch.empty_like(i), "Meta")
        return lib
    except RuntimeError:
        return None


_tensorrt_lib = _register_reference_op_names()
