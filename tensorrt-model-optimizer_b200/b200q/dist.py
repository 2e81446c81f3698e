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

__all__ = ["sync_amax", "sync_histograms", "agree_histogram_ranges", "flat_all_reduce", "sync_awq_statistics"]


def _quantizers(model):
    from .nn import TensorQuantizer

    if isinstance(model, TensorQuantizer):
        return [("", model)]
    return [(n, m) for n, m in model.named_modules() if isinstance(m, TensorQuantizer)]


def flat_all_reduce(tensors, op, group=None):
    """All-reduce a list of same-dtype tensors; results land in place.  Tensors that are adjacent slices
    of one allocation (the buffers of a calibration arena) are reduced where they are, as one run per
    allocation; anything else travels through one flat staging buffer.  Returns the number of collectives
    issued."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return 0
    runs = _contiguous_runs(tensors)
    if len(runs) == 1 and runs[0] is not None:
        dist.all_reduce(runs[0], op=op, group=group)
        return 1
    flat = torch.cat([t.detach().reshape(-1) for t in tensors])
    dist.all_reduce(flat, op=op, group=group)
    parts = flat.split([t.numel() for t in tensors])
    torch._foreach_copy_([t.data for t in tensors], [p.view(t.shape) for p, t in zip(parts, tensors)])
    return 1


def _contiguous_runs(tensors):
    """[view] if the tensors are back-to-back contiguous slices of one storage (in order), else [None]."""
    first = tensors[0]
    if not all(t.is_contiguous() and t.dtype == first.dtype and t.device == first.device
               and t.untyped_storage().data_ptr() == first.untyped_storage().data_ptr() for t in tensors):
        return [None]
    off = first.storage_offset()
    for t in tensors:
        if t.storage_offset() != off:
            return [None]
        off += t.numel()
    total = off - first.storage_offset()
    return [torch.as_strided(first, (total,), (1,), first.storage_offset())]


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


def _arenas(cals):
    seen, out = set(), []
    for _, c in cals:
        a = getattr(c, "_arena", None)
        if a is not None and id(a) not in seen:
            seen.add(id(a))
            out.append(a)
    return out


def agree_histogram_ranges(model: nn.Module, first_batch_max: dict | None = None, device=None, group=None,
                           src: int = 0, broadcast=None):
    """Give every rank's histogram calibrators the range rank ``src`` observed in its first batch.

    Calibrators that live in a ``HistogramArena`` have observed their first batch already
    (``observe_range``): their range slots are broadcast in place, one collective per arena, nothing passes
    through the host.  For the others ``first_batch_max`` maps quantiser name -> abs-max (float or 0-dim
    tensor) of this rank's first batch; the values of rank ``src`` are broadcast (one buffer) and applied
    with ``set_range``.  ``broadcast(tensor)`` replaces the collective (tests)."""
    cals = _hist_calibrators(model)
    if not cals:
        return
    active = dist.is_available() and dist.is_initialized()
    bc = broadcast or ((lambda t: dist.broadcast(t, src=src, group=group)) if active else (lambda t: None))
    for a in _arenas(cals):
        a.flush()
        if a.ranges is not None:
            bc(a.ranges)
    loose = [(n, c) for n, c in cals if getattr(c, "_arena", None) is None]
    if not loose:
        return
    buf = torch.tensor([float(first_batch_max[n]) for n, _ in loose], dtype=torch.float32, device=device)
    bc(buf)
    for (_, c), v in zip(loose, buf.tolist()):
        c.set_range(v, device)


def sync_histograms(model: nn.Module, group=None, all_reduce=None) -> int:
    """SUM all-reduce of all histogram counters.

    Arena calibrators: the arena's counters (and out-of-range counters) are reduced IN PLACE, one
    collective each; histograms of different live length need no padding because every row has the
    arena's capacity.  Other calibrators: ranks may have grown their histograms to different lengths (same
    bin width, see ``agree_histogram_ranges``): a MAX all-reduce of the lengths comes first, every
    histogram is padded to the common length in one int64 buffer, then one SUM all-reduce adds the counts.
    ``all_reduce(tensor, op)`` replaces the collective (tests).  Returns the number of collectives."""
    cals = _hist_calibrators(model)
    active = dist.is_available() and dist.is_initialized()
    if not cals or not (active or all_reduce is not None):
        return 0
    ar = all_reduce or (lambda t, op: dist.all_reduce(t, op=op, group=group))
    n = 0
    for a in _arenas(cals):
        a.flush()
        if a.counts is None:
            continue
        ar(a.counts, dist.ReduceOp.SUM)
        ar(a.overflow, dist.ReduceOp.SUM)
        a._stale = True
        n += 2
    loose = [(nm, c) for nm, c in cals if getattr(c, "_arena", None) is None]
    if not loose:
        return n
    dev = loose[0][1]._calib_hist.device
    for _, c in loose:
        c._resolve()
    lens = torch.tensor([c._num_bins for _, c in loose], dtype=torch.int64, device=dev)
    ar(lens, dist.ReduceOp.MAX)
    lens = lens.tolist()
    flat = torch.zeros(sum(lens), dtype=torch.int64, device=dev)
    off = 0
    for (_, c), ln in zip(loose, lens):
        flat[off:off + c._num_bins] = c._calib_hist[: c._num_bins]
        off += ln
    ar(flat, dist.ReduceOp.SUM)
    off = 0
    for (_, c), ln in zip(loose, lens):
        c._load_counts(flat[off:off + ln])
        off += ln
    return n + 2


def sync_awq_statistics(act_scales: list, has_nan: list, group=None) -> list:
    """Data-parallel step of awq_lite between its two passes (reference model_calib.py:711-741): every
    layer's ``act_scale`` becomes the mean over the ranks, and a layer is disabled on all ranks if its
    statistics hold a NaN on any.  ``act_scales`` are fp32 tensors (updated in place), ``has_nan`` one bool
    per layer; one SUM all-reduce carries everything (a layer's flag travels as one extra element).
    Returns the list of flags after the exchange."""
    if not (dist.is_available() and dist.is_initialized()) or not act_scales:
        return list(has_nan)
    world = dist.get_world_size(group)
    dev = act_scales[0].device
    flags = torch.tensor([1.0 if f else 0.0 for f in has_nan], dtype=torch.float32, device=dev)
    # NaN statistics must not poison the other layers' sums: they travel as zeros, their flag says so
    clean = [torch.where(torch.isnan(a), torch.zeros_like(a), a).reshape(-1) for a in act_scales]
    flat = torch.cat(clean + [flags])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    out_flags = (flat[-len(has_nan):] > 0).tolist()
    for a, bad in zip(act_scales, out_flags):
        n = a.numel()
        if not bad:
            a.copy_((flat[off:off + n] / world).reshape(a.shape))
        off += n
    return out_flags
