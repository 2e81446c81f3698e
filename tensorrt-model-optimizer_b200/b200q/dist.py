"""Data-parallel exchange steps of calibration, batched.

The reference all-reduces every quantiser's ``_amax`` separately
(modelopt/torch/quantization/model_calib.py:87-102; nn/modules/tensor_quantizer.py:1074-1086) —
hundreds of tiny collectives per model — and does not combine histograms across ranks at all
(calib/histogram.py:158-163 only warns).  Here all amaxes travel in ONE flat fp32 buffer through
one MAX all-reduce, and all histograms in ONE int64 buffer through one SUM all-reduce; both work
with NCCL (GPU tensors, NVLink) and with Gloo (CPU tensors, used by the tests).

Histograms of different ranks are only summable if they share the bin width, so the ranks first
agree on a common range (``agree_histogram_ranges``: rank 0's first-batch maximum, the value the
sequential reference would have used, broadcast in one buffer) before any batch is binned.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

__all__ = ["sync_amax", "sync_histograms", "agree_histogram_ranges", "flat_all_reduce"]


def _quantizers(model):
    from .nn import TensorQuantizer

    if isinstance(model, TensorQuantizer):
        return [("", model)]
    return [(n, m) for n, m in model.named_modules() if isinstance(m, TensorQuantizer)]


def flat_all_reduce(tensors, op, group=None):
    """All-reduce a list of same-dtype tensors through one flat buffer; results are copied back
    in place.  Returns the number of collectives issued (1, or 0 for an empty list)."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return 0
    flat = torch.cat([t.detach().reshape(-1) for t in tensors])
    dist.all_reduce(flat, op=op, group=group)
    off = 0
    for t in tensors:
        n = t.numel()
        t.data.copy_(flat[off:off + n].reshape(t.shape))
        off += n
    return 1


def sync_amax(model: nn.Module, group=None) -> int:
    """MAX all-reduce of every quantiser's ``_amax`` over ``group`` in one collective per dtype.
    Every rank must hold the same set of calibrated quantisers.  Returns the collective count."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    by_dtype = {}
    for _, q in _quantizers(model):
        a = getattr(q, "_amax", None)
        if a is not None and not a.is_meta:
            by_dtype.setdefault(a.dtype, []).append(a)
    n = 0
    for dt in sorted(by_dtype, key=str):
        n += flat_all_reduce(by_dtype[dt], dist.ReduceOp.MAX, group)
    return n


def _hist_calibrators(model):
    from .calib import HistogramCalibrator

    out = []
    for name, q in _quantizers(model):
        c = getattr(q, "_calibrator", None)
        if isinstance(c, HistogramCalibrator) and not q._disabled:
            out.append((name, c))
    return out


def agree_histogram_ranges(model: nn.Module, first_batch_max: dict, device, group=None, src: int = 0):
    """Give every rank's histogram calibrators the range rank ``src`` observed in its first batch.

    ``first_batch_max`` maps quantiser name -> abs-max (float or 0-dim tensor) of this rank's first
    batch; the values of rank ``src`` are broadcast (one buffer) and applied with ``set_range``.
    """
    cals = _hist_calibrators(model)
    if not cals:
        return
    buf = torch.tensor([float(first_batch_max[n]) for n, _ in cals], dtype=torch.float32, device=device)
    if dist.is_available() and dist.is_initialized():
        dist.broadcast(buf, src=src, group=group)
    for (_, c), v in zip(cals, buf.tolist()):
        c.set_range(v, device)


def sync_histograms(model: nn.Module, group=None) -> int:
    """SUM all-reduce of all histogram counters in one int64 buffer.

    Ranks may have grown their histograms to different lengths (same bin width, see
    ``agree_histogram_ranges``): a MAX all-reduce of the lengths comes first, every histogram is
    padded to the common length, then one SUM all-reduce adds the counts.  Returns the number of
    collectives (2, or 0 without calibrators / process group)."""
    cals = _hist_calibrators(model)
    if not cals or not (dist.is_available() and dist.is_initialized()):
        return 0
    dev = cals[0][1]._calib_hist.device
    for _, c in cals:
        c._resolve()
    lens = torch.tensor([c._num_bins for _, c in cals], dtype=torch.int64, device=dev)
    dist.all_reduce(lens, op=dist.ReduceOp.MAX, group=group)
    lens = lens.tolist()
    flat = torch.zeros(sum(lens), dtype=torch.int64, device=dev)
    off = 0
    for (_, c), n in zip(cals, lens):
        flat[off:off + c._num_bins] = c._calib_hist[: c._num_bins]
        off += n
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for (_, c), n in zip(cals, lens):
        c._load_counts(flat[off:off + n])
        off += n
    return 2
