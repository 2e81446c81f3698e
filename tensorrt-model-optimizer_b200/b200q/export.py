"""Export-side weight packers (reference: modelopt/torch/export/quant_utils.py:68-91,697-834):
the on-disk layouts deployment frameworks read, produced by the same kernels as the in-memory
real-quant tensors plus the transposed INT4 packer."""
from __future__ import annotations

import torch

from . import ops
from .qtensor import FP8QTensor, NVFP4QTensor, QTensorWrapper

__all__ = ["get_scaling_factor_from_weight", "pack_int4_in_uint8", "to_quantized_weight",
           "QUANTIZATION_FP8", "QUANTIZATION_INT8_SQ", "QUANTIZATION_INT8_WO", "QUANTIZATION_INT4_AWQ",
           "QUANTIZATION_W4A8_AWQ", "QUANTIZATION_NVFP4", "QUANTIZATION_NVFP4_AWQ", "QUANTIZATION_FP8_PB_WO",
           "QUANTIZATION_FP8_PC_PT"]

QUANTIZATION_FP8 = "fp8"
QUANTIZATION_INT8_SQ = "int8_sq"
QUANTIZATION_INT8_WO = "int8_wo"
QUANTIZATION_INT4_AWQ = "int4_awq"
QUANTIZATION_W4A8_AWQ = "w4a8_awq"
QUANTIZATION_NVFP4 = "nvfp4"
QUANTIZATION_NVFP4_AWQ = "nvfp4_awq"
QUANTIZATION_FP8_PB_WO = "fp8_pb_wo"
QUANTIZATION_FP8_PC_PT = "fp8_pc_pt"


def _true_div(a: torch.Tensor, value: float) -> torch.Tensor:
    return a / torch.full((), value, dtype=a.dtype, device=a.device)


def get_scaling_factor_from_weight(weight, group_size) -> torch.Tensor:
    """fp32 amax / 7 per (row, group) for int4_awq (group_size > 0) or amax / 127 per row."""
    n, k = weight.shape
    if group_size != 0:
        if k % group_size != 0:
            raise NotImplementedError("Weight shape is not divisible for block size for block quantization.")
        amax = ops.amax_blocks(weight, group_size).reshape(n, k // group_size)
        maxbound = 7.0
    else:
        amax = ops.amax_axis3(weight, 1, n, k)
        maxbound = 127.0
    s = _true_div(amax, maxbound)
    s[s == 0] = 1.0
    return s


def pack_int4_in_uint8(weight, weights_scaling_factor):
    """uint8 [out/2, in]: two output channels per byte (low nibble = even row), signed nibbles."""
    out_dim = weight.shape[-2]
    assert out_dim % 2 == 0, f"Cannot pack weight. Out dimension {out_dim} is not an even number."
    if weight.dim() == 3:
        return torch.stack([ops.int4_export_pack(weight[e], weights_scaling_factor[e])
                            for e in range(weight.shape[0])])
    return ops.int4_export_pack(weight, weights_scaling_factor)


def _quotient(weight, scale):
    """``weight / scale`` with torch's type promotion, formed as an fp32 division rounded to the
    result type — what the CPU kernels compute.  (On CUDA torch would first round a 0-dim fp32
    scale to a 16-bit weight's type, which changes the last bit of the quotient.)"""
    rt = torch.result_type(weight, scale)
    return (weight.float() / scale.float()).to(rt).contiguous()


def _fp8(weight, scale_broadcast):
    """torch's e4m3 cast of the promoted quotient, through the cast kernel."""
    q = _quotient(weight, scale_broadcast)
    one = torch.ones(1, dtype=q.dtype, device=q.device)
    return ops.fp8_quantize(q, one, 1, 1, q.numel()).reshape(weight.shape)


def to_quantized_weight(weight, weights_scaling_factor, quantization: str, weights_scaling_factor2=None,
                        block_size=None):
    """Convert a weight to its packed checkpoint form for ``quantization``."""
    if weights_scaling_factor is not None:
        weights_scaling_factor = weights_scaling_factor.to(weight.device)
    if weights_scaling_factor2 is not None:
        weights_scaling_factor2 = weights_scaling_factor2.to(weight.device)
    if isinstance(weight, QTensorWrapper):
        return weight.data
    if quantization == QUANTIZATION_FP8:
        if weight.dtype == torch.float8_e4m3fn:
            return weight
        s = weights_scaling_factor.unsqueeze(-1) if weight.dim() == 3 else weights_scaling_factor
        return _fp8(weight, s)
    if quantization in (QUANTIZATION_INT8_SQ, QUANTIZATION_INT8_WO):
        q = _quotient(weight, weights_scaling_factor[:, None])
        one = torch.ones(1, dtype=q.dtype, device=q.device)
        return ops.int8_quantize(q, one, 1, 1, q.numel()).reshape(weight.shape)
    if quantization == QUANTIZATION_FP8_PB_WO:
        return FP8QTensor.quantize(weight, weights_scaling_factor.squeeze(),
                                   block_sizes={-1: block_size, -2: block_size})[0]._quantized_data
    if quantization == QUANTIZATION_FP8_PC_PT:
        return _fp8(weight, weights_scaling_factor[:, None])
    if quantization in (QUANTIZATION_INT4_AWQ, QUANTIZATION_W4A8_AWQ):
        return pack_int4_in_uint8(weight, weights_scaling_factor)
    if quantization in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        assert block_size is not None, "Block size not passed. Unable to quantize to NVFP4 format."
        assert weights_scaling_factor2 is not None, (
            "Weights scaling factor 2 not passed. Unable to quantize to NVFP4 format")
        return NVFP4QTensor.quantize(weight, block_size, weights_scaling_factor,
                                     weights_scaling_factor2)[0]._quantized_data
    raise NotImplementedError(f"quantization format {quantization} not supported")
