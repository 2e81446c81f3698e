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


# ---- the other formats' CPU paths, operation by operation (timed as the reference's side of bench.py) ----

@torch.no_grad()
def reduce_amax(x: torch.Tensor, axis=None) -> torch.Tensor:
    """utils.py:155-188: two reductions (max, min) in the input dtype, keepdims."""
    if axis is None:
        return torch.maximum(torch.abs(torch.max(x)), torch.abs(torch.min(x)))
    red = [i for i in range(x.dim()) if i != axis % x.dim()]
    return torch.maximum(torch.abs(torch.amax(x, dim=red, keepdim=True)), torch.abs(torch.amin(x, dim=red, keepdim=True)))


@torch.no_grad()
def fake_int(x: torch.Tensor, amax: torch.Tensor, num_bits=8, unsigned=False, narrow_range=True) -> torch.Tensor:
    """_tensor_quant (tensor_quant.py:574-612), the fallback FakeTensorQuantFunction runs on CPU tensors."""
    dtype = x.dtype
    x, amax = x.float(), amax.float()
    min_amax = amax.min()
    if min_amax < 0:
        raise ValueError("Negative values in amax")
    max_bound = torch.tensor((2.0 ** (num_bits - 1 + int(unsigned))) - 1.0)
    min_bound = 0 if unsigned else (-max_bound if narrow_range else -max_bound - 1)
    scale = max_bound / amax
    eps = 1.0 / (1 << 24)
    if min_amax <= eps:
        mask = amax <= eps
        scale[mask] = 0
    out = torch.clamp((x * scale).round_(), min_bound, max_bound)
    if min_amax <= eps:
        scale[mask] = 1.0
    return (out / scale).to(dtype)


@torch.no_grad()
def max_calibrate_collect(x: torch.Tensor, running, axis=None):
    """MaxCalibrator.collect (calib/max.py:59-83): reduce_amax, three validity checks, running maximum."""
    a = reduce_amax(x, axis).detach()
    assert torch.all(a >= 0) and not torch.any(torch.isinf(a)) and not torch.any(torch.isnan(a))
    return a if running is None else torch.max(running, a)


@torch.no_grad()
def fp8_eager(x: torch.Tensor, amax: torch.Tensor) -> torch.Tensor:
    """_fp8_eager (tensor_quant.py:45-54), what ScaledE4M3Function runs on CPU tensors."""
    dtype = x.dtype
    scale = 448.0 / amax.to(torch.float32)
    inv = 1 / scale
    y = (x.to(torch.float32) * scale).to(torch.float8_e4m3fn)
    return (y.to(torch.float32) * inv).to(dtype)


class HistogramPath:
    """HistogramCalibrator.collect with torch_hist=True (calib/histogram.py:77-130) and the percentile
    read-out (:328-343)."""

    def __init__(self, num_bins=2048):
        self.num_bins, self.hist, self.edges = num_bins, None, None

    @torch.no_grad()
    def collect(self, x: torch.Tensor):
        if torch.min(x) < 0.0:
            x = x.abs()
        x = x.float()
        x_max = x.max().item()
        if self.hist is None:
            self.hist = torch.histc(x, bins=self.num_bins, min=0, max=x_max)
            self.edges = torch.linspace(0, x_max, self.num_bins + 1)
        else:
            if x_max > self.edges[-1]:
                width = self.edges[1] - self.edges[0]
                self.num_bins = int((x_max / width).ceil().item())
                self.edges = torch.arange(0, x_max + width, width)
            h = torch.histc(x, bins=self.num_bins, min=0, max=self.edges[-1])
            h[: self.hist.numel()] += self.hist
            self.hist = h

    def percentile(self, p: float) -> float:
        import numpy as np

        hist, edges = self.hist.int().numpy(), self.edges.numpy()
        cdf = np.cumsum(hist / hist.sum())
        return float(edges[np.searchsorted(cdf, p / 100)])


@torch.no_grad()
def awq_lite_candidate(w: torch.Tensor, x: torch.Tensor, out_actual: torch.Tensor, a_scale, w_scale, alpha, block=128):
    """One alpha of the patched forward of awq_lite (model_calib.py:671-685 with get_scale :608-621 and
    update_loss :623-627): the scales, the pre-quant-scale multiplies, dynamic block amax, INT4 fake quant
    (``_tensor_quant``), the linear layer and the loss."""
    s = (a_scale.pow(alpha) / (w_scale.pow(1 - alpha) + torch.finfo(torch.float32).tiny)).clamp(min=1e-4, max=1e4)
    s = s / (s.max() * s.min()).sqrt()
    ws = (w * s.to(w.dtype)).view(-1, block)
    amax = reduce_amax(ws, axis=0)
    wq = fake_int(ws, amax, 4, False, False).view(w.shape)
    out = torch.nn.functional.linear(x * (1 / s).to(x.dtype), wq)
    return (out - out_actual).float().pow(2).mean()
