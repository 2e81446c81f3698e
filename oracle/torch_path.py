"""TEST AND BENCHMARK INFRASTRUCTURE ONLY — never imported by the product.

The reference's CPU path for NVFP4 weight quantisation restated as the sequence of torch tensor
operations it executes (modelopt/torch/quantization/qtensor/nvfp4_tensor.py:62-97,119-232 with
reduce_amax / reduce_block_amax of modelopt/torch/quantization/utils.py:52-98,155-188): about ten
passes over the tensor with fp32 temporaries.  It is what "ModelOpt's CPU torch path" costs on the
host cores, so ``bench.py --impl reference`` times it; the golden vectors pin its bytes
(tests/test_oracle_golden.py)."""
from __future__ import annotations

import torch

_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32)


def _amax_all(x: torch.Tensor) -> torch.Tensor:
    return torch.maximum(torch.abs(torch.max(x)), torch.abs(torch.min(x)))          # utils.py:176-179


def _amax_blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    a = x.clone().reshape(*x.shape[:-1], x.shape[-1] // block, block)                # utils.py:73,89
    return torch.maximum(torch.abs(torch.amax(a, dim=-1)), torch.abs(torch.amin(a, dim=-1)))


def _cast_fp4(v: torch.Tensor) -> torch.Tensor:
    sign = (v < 0).to(torch.uint8)                                                     # nvfp4_tensor.py:125
    a = v.abs_()
    ordn = torch.searchsorted(_BOUNDS, a, out_int32=True).to(torch.uint8)
    ties = torch.any(a.unsqueeze(-1) == _BOUNDS[[1, 3, 5]], dim=-1).to(torch.uint8)
    return (sign << 3) + ordn + ties


@torch.no_grad()
def nvfp4_quantize(x: torch.Tensor, block: int = 16):
    """x [.., K] (K % block == 0) on the CPU -> (packed uint8 [.., K/2], scales float8_e4m3fn
    [.., K/block], scale2 fp32 0-dim), operation by operation as the reference's torch path."""
    s2 = _amax_all(x).float() / (6.0 * 448.0)
    per_block = _amax_blocks(x, block).float() / (6.0 * s2)
    per_block[per_block == 0] = 1.0
    scales = per_block.to(torch.float8_e4m3fn)
    shape = x.shape
    xb = x.view(*shape[:-1], -1, block)
    scaled = (xb / (scales.to(torch.float32) * s2).unsqueeze(-1)).view(shape)
    q = _cast_fp4(scaled)
    packed = (q[..., 1::2] << 4) | q[..., 0::2]
    return packed, scales, s2
