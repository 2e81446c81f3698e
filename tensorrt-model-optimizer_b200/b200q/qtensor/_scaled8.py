"""Shared scale handling of the 8-bit quantised tensors: per tensor, per axis, or N-D blocks."""
from __future__ import annotations

import math

import torch

from ..utils import (convert_quantization_axis_to_reduce_axis, reduce_amax, reduce_block_amax,
                     reduce_block_padding)


def prepare(input, scales, axis, block_sizes, divisor):
    """-> (padded input, scales, (outer, n_axis, inner) or None when the scale layout needs the
    expanded-scale fallback)."""
    x = reduce_block_padding(input, block_sizes) if block_sizes else input
    if scales is None:
        if block_sizes:
            amax = reduce_block_amax(x, block_sizes)
        else:
            amax = reduce_amax(x, axis=convert_quantization_axis_to_reduce_axis(x, axis))
        # tensor divisor: a true division on every device (see nvfp4_tensor._scale2_from_amax)
        scales = amax / torch.full((), divisor, dtype=amax.dtype, device=amax.device)
    if block_sizes:
        expected = list(x.shape)
        for dim, b in block_sizes.items():
            d = dim if dim >= 0 else x.dim() + dim
            assert x.shape[d] % b == 0
            expected[d] = x.shape[d] // b
        if scales.shape != tuple(expected) and scales.numel() == math.prod(expected):
            scales = scales.reshape(expected)
        assert scales.shape == tuple(expected), f"Mismatch in expected scale shape: {scales.shape} vs {tuple(expected)}"
        dims = [d if d >= 0 else x.dim() + d for d in block_sizes]
        if dims == [x.dim() - 1]:
            return x, scales, (1, scales.numel(), block_sizes[list(block_sizes)[0]])
        return x, scales, None
    if scales.numel() == 1:
        return x, scales, (1, 1, x.numel())
    sshape = [s for s in scales.shape]
    if len(sshape) == x.dim():
        nz = [i for i, s in enumerate(sshape) if s != 1]
        if len(nz) == 1 and sshape[nz[0]] == x.shape[nz[0]]:
            a = nz[0]
            return x, scales, (math.prod(x.shape[:a]), x.shape[a], math.prod(x.shape[a + 1:]))
    return x, scales, None


def expand(scales, x, block_sizes):
    e = scales
    if block_sizes:
        for dim, b in block_sizes.items():
            e = e.repeat_interleave(b, dim=dim)
    return e
