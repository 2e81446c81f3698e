"""Amax reductions with the signatures of ``modelopt/torch/quantization/utils.py`` (lines 52-188),
computed by the single-pass CUDA reductions."""
from __future__ import annotations

import contextlib

import torch
import torch.nn.functional as F

from . import ops

__all__ = ["export_torch_mode", "is_torch_export_mode", "reduce_amax", "reduce_block_amax", "reduce_block_padding",
           "convert_quantization_axis_to_reduce_axis"]


def convert_quantization_axis_to_reduce_axis(input, axis):
    """Quantisation axis (kept) -> list of axes to reduce; ``None`` = reduce everything."""
    if axis is None:
        return None
    axis = axis if isinstance(axis, (list, tuple)) else [axis]
    return [i for i in range(input.dim()) if i not in axis and (i - input.dim()) not in axis]


@torch.no_grad()
def reduce_amax(input, axis=None, keepdims=True, squeeze_scalar=True):
    """max(|max|, |min|) over ``axis`` (the axes to reduce), in the input's dtype."""
    x = input.detach()
    if axis is None:
        return ops.amax_tensor(x).to(x.dtype)
    if isinstance(axis, int):
        axis = (axis,)
    nd = x.dim()
    red = sorted({a % nd for a in axis})
    keep = [d for d in range(nd) if d not in red]
    if not keep:
        out = ops.amax_tensor(x).to(x.dtype)
        return out.reshape([1] * nd) if keepdims and not squeeze_scalar else out
    contiguous_run = keep == list(range(keep[0], keep[-1] + 1))
    if not contiguous_run:
        # bring the kept axes together; the reduction itself still runs in one pass
        x = x.permute(*keep, *red).contiguous()
        outer, inner = 1, 1
        for d in red:
            inner *= input.shape[d]
    else:
        outer = 1
        for d in range(keep[0]):
            outer *= x.shape[d]
        inner = 1
        for d in range(keep[-1] + 1, nd):
            inner *= x.shape[d]
    n_axis = 1
    for d in keep:
        n_axis *= input.shape[d]
    out = ops.amax_axis3(x, outer, n_axis, inner).to(input.dtype)
    if keepdims:
        out = out.reshape([input.shape[d] if d in keep else 1 for d in range(nd)])
    else:
        out = out.reshape([input.shape[d] for d in keep])
    if squeeze_scalar and out.numel() == 1:
        out = out.squeeze()
    return out


@torch.no_grad()
def reduce_block_amax(input_tensor: torch.Tensor, block_sizes: dict):
    """Per-block abs-max; a single last-dimension block size runs as one fused kernel, several
    blocked dimensions are reduced one after the other like the reference does."""
    items = [(d if d >= 0 else input_tensor.dim() + d, b) for d, b in block_sizes.items()]
    x = input_tensor.detach()
    if len(items) == 1 and items[0][0] == x.dim() - 1:
        b = items[0][1]
        assert x.shape[-1] % b == 0, f"Tensor dimension {x.shape[-1]} is not divisible by {b}"
        out = ops.amax_blocks(x, b).to(x.dtype)
        return out.reshape(*x.shape[:-1], x.shape[-1] // b)
    amax = x
    for dim, b in items:
        assert amax.shape[dim] % b == 0, f"Tensor dimension {amax.shape[dim]} is not divisible by {b}"
        shape = [*amax.shape[:dim], amax.shape[dim] // b, b, *amax.shape[dim + 1:]]
        amax = reduce_amax(amax.reshape(shape), dim + 1, keepdims=False, squeeze_scalar=False)
    return amax


def reduce_block_padding(input: torch.Tensor, block_sizes: dict, pad_value: float = 0):
    """Right-pad each listed dimension to a multiple of its block size."""
    with torch.no_grad():
        x = input
        nd = x.dim()
        for dim, block in block_sizes.items():
            d = dim if dim >= 0 else nd + dim
            rem = x.size(d) % block
            if rem:
                pad = [0] * (2 * nd)
                pad[(nd - 1 - d) * 2 + 1] = block - rem
                x = F.pad(x, pad, value=pad_value)
        return x


# ---- torch.export ---------------------------------------------------------------------------------------
_EXPORT_MODE = False


@contextlib.contextmanager
def export_torch_mode():
    """While active, quantised modules run the forms ``torch.export`` can trace: packed layers take the
    fake-quantisation forward instead of a registered GEMM, amax buffers are read detached (reference
    modelopt/torch/quantization/utils.py:360-374)."""
    global _EXPORT_MODE
    saved, _EXPORT_MODE = _EXPORT_MODE, True
    try:
        yield
    finally:
        _EXPORT_MODE = saved


def is_torch_export_mode() -> bool:
    return _EXPORT_MODE
