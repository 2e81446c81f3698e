"""Calibration algorithms (reference: modelopt/torch/quantization/model_calib.py): ``max_calibrate``
(:65-185) and ``awq_lite`` (:530-785) with their helpers.

Differences in execution, not in results: amax collection is one kernel per quantiser call with
no host synchronisation, the data-parallel amax exchange is one all-reduce over a flat buffer
(``b200q.dist.sync_amax``) instead of one per quantiser, and the AWQ search evaluates each alpha
with a fused scale+block-quantise kernel feeding the GEMM.
"""
from __future__ import annotations

import warnings

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from . import dist as qdist
from . import ops
from .calib import MseCalibrator
from .nn import SequentialQuantizer, TensorQuantizer, is_quantized_linear

__all__ = ["max_calibrate", "mse_calibrate", "histogram_calibrate", "awq_lite", "awq_clip", "smoothquant", "awq", "enable_stats_collection", "finish_stats_collection", "load_calib_amax_all",
           "weight_only_quantize", "apply_pre_quant_scale_and_smooth", "disable_pre_quant_scale_and_resmooth"]


def enable_stats_collection(model: nn.Module):
    for _, m in model.named_modules():
        if isinstance(m, TensorQuantizer) and not m._disabled:
            if m._calibrator is not None:
                m.disable_quant()
                m.enable_calib()
            else:
                m.disable()


def load_calib_amax_all(items):
    """Load the calibrated amax of many quantisers with ONE validity read.  ``items``: (name, quantiser,
    args, kwargs) with the arguments of ``calibrator.compute_amax``.  Quantisers whose calibrator has
    seen nothing are skipped.  The reference loads and validates quantiser by quantiser
    (model_calib.py:145-185), one device->host read each; here the values are tested together, per
    device, and the error names every offending quantiser."""
    from .calib import HistogramCalibrator, MaxCalibrator

    loaded = {}       # device -> [(name, quantiser)]
    checks = {}       # device -> fp32 tensors holding every value loaded on it
    batched = {}      # (device, percentile) -> histogram calibrators read out by one launch
    running_max = {}  # (device, dtype) -> max calibrators whose running maxima are converted together

    def took(name, q, values_fp32=None):
        dev = q._amax.device
        loaded.setdefault(dev, []).append((name, q))
        checks.setdefault(dev, []).append(q._amax.detach().reshape(-1).float() if values_fp32 is None else values_fp32)

    for name, q, args, kwargs in items:
        cal = q._calibrator
        if (isinstance(cal, HistogramCalibrator) and tuple(args) == ("percentile",) and set(kwargs) <= {"percentile"}
                and cal._calib_hist is not None and cal._calib_hist.is_cuda
                and (cal._arena is None or cal._ranged)):
            pct = kwargs.get("percentile", 99.99)
            if pct < 0 or pct > 100:
                raise ValueError("Invalid percentile. Must be in range 0 <= percentile <= 100.")
            cal._resolve()
            batched.setdefault((cal._calib_hist.device, pct), []).append((name, q))
            continue
        if type(cal) is MaxCalibrator and not args and not kwargs and cal._acc is not None and cal._acc.is_cuda:
            running_max.setdefault((cal._acc.device, cal._dtype), []).append((name, q))
            continue
        extra = {"check": False} if isinstance(cal, MaxCalibrator) else {}
        value = cal.compute_amax(*args, **kwargs, **extra)
        if value is None:
            continue
        q._store_calib_amax(value)
        took(name, q)
    # max calibrators: one concatenation and one conversion to the collected dtype per device and dtype; the
    # quantisers' buffers are slices of the result (two launches instead of two per quantiser)
    for (dev, dtype), group in running_max.items():
        accs = [q._calibrator._acc for _, q in group]
        flat = torch.cat(accs) if len(accs) > 1 else accs[0].clone()
        conv = flat.to(dtype)
        off = 0
        for (name, q), acc in zip(group, accs):
            n = acc.numel()
            q._store_calib_amax(conv[off:off + n].reshape(q._calibrator._shape), owned=True)
            off += n
            loaded.setdefault(dev, []).append((name, q))
        checks.setdefault(dev, []).append(flat)
    for (dev, pct), group in batched.items():
        values = ops.hist_percentile_batch(
            [(q._calibrator._calib_hist, q._calibrator._num_bins, q._calibrator._calib_bin_edges) for _, q in group], pct)
        for i, (name, q) in enumerate(group):
            q._store_calib_amax(values[i], owned=True)
            loaded.setdefault(dev, []).append((name, q))
        checks.setdefault(dev, []).append(values.reshape(-1).float())
    for dev, parts in checks.items():
        flat = torch.cat(parts) if len(parts) > 1 else parts[0]
        if bool((~torch.isfinite(flat) | (flat < 0)).any()):
            bad = [n for n, q in loaded[dev] if not q.validate_attr(attr_name="_amax")]
            raise ValueError(f"calibrated amax of {bad} contains nan, inf or negative values")
    return sum(len(g) for g in loaded.values())


def finish_stats_collection(model: nn.Module, method: str | None = None):
    items, done = [], []
    for name, m in model.named_modules():
        if not isinstance(m, TensorQuantizer) or m._disabled:
            continue
        cal = getattr(m, "_calibrator", None)
        if cal and not m._dynamic:
            if isinstance(cal, MseCalibrator) or method not in {"mse", "entropy"}:
                items.append((name, m, (), {}))
            else:
                items.append((name, m, (method,), {}))
        done.append(m)
    load_calib_amax_all(items)
    for m in done:
        if m.bias_calibrator is not None and m.bias_type == "static":
            m.load_calib_bias()
        m.enable_quant()
        m.disable_calib()


def weight_only_quantize(model: nn.Module):
    """Run every weight through its weight quantiser once (collects weight statistics)."""
    seen = set()
    for _, m in model.named_modules():
        if m in seen:
            continue
        if hasattr(m, "weight_quantizer") and getattr(m, "weight", None) is not None:
            m.weight_quantizer(m.weight)
        seen.add(m)


@torch.no_grad()
def max_calibrate(model: nn.Module, forward_loop=None, distributed_sync=True):
    """Max calibration: collect abs-max statistics while ``forward_loop(model)`` runs (or over the
    weights only when no loop is given), load them into the ``_amax`` buffers and take the MAX
    over the data-parallel group."""
    enable_stats_collection(model)
    if forward_loop is None:
        weight_only_quantize(model)
    else:
        forward_loop(model)
    finish_stats_collection(model)
    if distributed_sync and dist.is_available() and dist.is_initialized():
        qdist.sync_amax(model)


@torch.no_grad()
def histogram_calibrate(model: nn.Module, forward_loop, method: str = "percentile", first_batch_loop=None,
                        distributed_sync=True, share_inputs: bool = True, **compute_kwargs):
    """Histogram calibration (``"percentile"``, ``"entropy"`` or ``"mse"`` read-out) of every quantiser
    whose calibrator is a HistogramCalibrator; other calibrators are max-calibrated by the same loop.

    All histogram counters live in one arena (``attach_histogram_arena``): ranges stay on the device and
    quantisers fed the same tensor share a binning pass.  With a process group up the calibration is
    data-parallel — every rank runs ``forward_loop`` over its own batches — in the reference's contract
    (one calibrator over the union of the batches, the first batch of rank 0 fixing the bin width):
    ``first_batch_loop(model)`` (default: ``forward_loop``) runs once with the calibrators only observing
    ranges, rank 0's ranges are broadcast in place, ``forward_loop`` bins, one SUM all-reduce merges the
    counters, and every rank reads the same amax out (reference: calib/histogram.py:77-130,166-213 for the
    collection and read-out it reproduces; the reference has no data-parallel histogram merge)."""
    from .calib import HistogramCalibrator, attach_histogram_arena

    arenas = attach_histogram_arena(model, share_inputs)
    enable_stats_collection(model)
    dp = distributed_sync and dist.is_available() and dist.is_initialized()
    if dp:
        for a in arenas:
            a.observe_only = True
        (first_batch_loop or forward_loop)(model)
        for a in arenas:
            a.observe_only = False
        qdist.agree_histogram_ranges(model)
    forward_loop(model)
    if dp:
        qdist.sync_histograms(model)
    items, done = [], []
    for name, m in model.named_modules():
        if not isinstance(m, TensorQuantizer) or m._disabled:
            continue
        cal = getattr(m, "_calibrator", None)
        if cal is not None and not m._dynamic:
            if isinstance(cal, HistogramCalibrator):
                items.append((name, m, (method,), compute_kwargs))
            else:
                items.append((name, m, (), {}))
        done.append(m)
    load_calib_amax_all(items)
    for m in done:
        m.enable_quant()
        m.disable_calib()
    if dp:
        qdist.sync_amax(model)


@torch.no_grad()
def mse_calibrate(model: nn.Module, forward_loop=None, distributed_sync=True, num_steps: int = 10,
                  start_multiplier: float = 0.25, stop_multiplier: float = 4.0):
    """Max calibration first, then per quantiser an amax search over
    ``amax * linspace(start, stop, num_steps)`` minimising the fake-quantisation error
    (reference model_calib.py:188-269)."""
    max_calibrate(model, forward_loop, distributed_sync)
    for name, m in model.named_modules():
        if not isinstance(m, TensorQuantizer) or m._disabled:
            continue
        if m.is_static_block_quant:
            raise ValueError("MSE calibration does not support static block quantization. "
                             f"Found static block quantization at {name}.")
        if m._calibrator is not None and not m._dynamic and hasattr(m, "_amax"):
            def quant_func(x, amax, q=m):
                saved = q._amax
                if_quant, if_calib, fake = q._if_quant, q._if_calib, q._fake_quant
                q._amax = amax
                q._if_quant, q._if_calib, q._fake_quant = True, False, True
                try:
                    return q(x)
                finally:
                    q._amax = saved
                    q._if_quant, q._if_calib, q._fake_quant = if_quant, if_calib, fake

            # a plain integer / E4M3 fake quantiser: every candidate in one kernel pass over each batch
            fused = None
            plain = (m._fake_quant and m._block_sizes is None and m.pre_quant_scale is None
                     and getattr(m, "_bias", None) is None and not getattr(m, "_rotate", False))
            if plain and (isinstance(m._num_bits, int) or tuple(m._num_bits) == (4, 3)):
                fused = {"num_bits": m._num_bits, "unsigned": m._unsigned, "narrow_range": m._narrow_range}
            m._calibrator = MseCalibrator(amax=m._amax.clone().detach(), axis=m._calibrator._axis,
                                          num_steps=num_steps, start_multiplier=start_multiplier,
                                          stop_multiplier=stop_multiplier, quant_func=quant_func, fused=fused)
    enable_stats_collection(model)
    if forward_loop is None:
        weight_only_quantize(model)
    else:
        forward_loop(model)
    finish_stats_collection(model, method="mse")


# --------------------------------------------------------------------------------- AWQ lite ----

def _awq_block_size(weight, quantizer):
    bs = quantizer.block_sizes
    if bs is None:
        return None
    b = bs.get(-1) or bs.get(weight.dim() - 1)
    return b


def get_weight_scale(weight, block_size=None):
    """mean over rows of |W| / (block amax + tiny), reduced in the weight's dtype, then fp32
    (reference model_calib.py:588-603)."""
    org_shape = weight.shape
    sl = None
    if block_size:
        if org_shape[-1] % block_size:
            sl = slice(org_shape[-1])
            weight = F.pad(weight, (0, block_size - org_shape[-1] % block_size), "constant", 0)
            org_shape = weight.shape
        weight = weight.contiguous().view(-1, block_size)
    amax = weight.abs().amax(dim=1, keepdim=True)
    scale = (weight.abs() / (amax + torch.finfo(weight.dtype).tiny)).view(org_shape)
    if sl is not None:
        scale = scale[..., sl]
    return scale.mean(0).to(torch.float32)


def get_act_scale(x):
    return x.abs().contiguous().view(-1, x.shape[-1]).mean(0).to(torch.float32)


def get_scale(x_max, w_max, alpha):
    """s = clamp(a^alpha / (w^(1-alpha) + tiny), 1e-4, 1e4) / sqrt(max(s) * min(s))."""
    s = (x_max.pow(alpha) / (w_max.to(x_max.device).pow(1 - alpha) + torch.finfo(torch.float32).tiny)
         ).clamp(min=1e-4, max=1e4).view(-1)
    return (s / (s.max() * s.min()).sqrt()).view(-1)


def _fold_into_weight(linear, per_input_channel):
    """W <- (W * v[None, :]) in the weight's dtype, then the weight amax is calibrated afresh."""
    w = linear.weight
    w.data.copy_((w * per_input_channel.to(w.device).squeeze()[None, :]).to(w.dtype))
    linear.weight_quantizer.reset_amax()
    max_calibrate(linear, lambda lin: lin.weight_quantizer(lin.weight), distributed_sync=False)


@torch.no_grad()
def disable_pre_quant_scale_and_resmooth(linear, delete_pre_quant_scale: bool = False):
    """Undo the smoothing of one quantised linear layer: the input-side scale is folded back into the weight
    and switched off (kept as a buffer unless ``delete_pre_quant_scale``), the input amax returns to the
    largest per-channel value seen before smoothing (reference model_calib.py:308-339)."""
    assert is_quantized_linear(linear), "Only quantized linear modules are supported"
    iq = linear.input_quantizer
    assert iq._enable_pre_quant_scale, "pre_quant_scale should be enabled first!"
    assert hasattr(iq, "_pre_quant_scale"), "pre_quant_scale should be available"
    _fold_into_weight(linear, iq._pre_quant_scale.to(torch.float32))
    iq._enable_pre_quant_scale = False
    if iq.amax is not None:
        assert hasattr(iq, "_amax_for_smoothing")
        iq.amax = iq._amax_for_smoothing.amax().to(device=linear.weight.device, dtype=linear.weight.dtype)
    if delete_pre_quant_scale:
        delattr(iq, "_pre_quant_scale")


@torch.no_grad()
def apply_pre_quant_scale_and_smooth(linear, pre_quant_scale=None):
    """Set ``input_quantizer.pre_quant_scale`` and fold its inverse into the weight, then
    re-calibrate the weight amax (reference model_calib.py:344-408).  Without a scale the quantiser's
    stored (switched-off) one is applied again."""
    assert is_quantized_linear(linear), "Only quantized linear modules are supported"
    assert linear.input_quantizer.pre_quant_scale is None, "pre_quant_scale should be None first!"
    if pre_quant_scale is None:
        pre_quant_scale = getattr(linear.input_quantizer, "_pre_quant_scale", None)
    assert pre_quant_scale is not None, "pre_quant_scale should be provided or already set"
    assert torch.all(pre_quant_scale > 0), "pre_quant_scale should be positive"
    pqs = pre_quant_scale.to(torch.float32)
    linear.input_quantizer._enable_pre_quant_scale = True
    linear.input_quantizer.pre_quant_scale = pqs.to(linear.weight.dtype)
    _fold_into_weight(linear, 1.0 / pqs)
    if linear.input_quantizer.amax is not None:
        assert hasattr(linear.input_quantizer, "_amax_for_smoothing")
        dev, dt = linear.weight.device, linear.weight.dtype
        a = linear.input_quantizer._amax_for_smoothing.to(device=dev, dtype=dt)
        linear.input_quantizer.amax = (a * pqs.to(dev)).amax().to(dt)


# evaluate awq_lite candidates with the fused tcgen05 GEMM + loss kernel where its shape rules allow
USE_TENSOR_CORE_EVAL = True


class _AWQLiteState:
    def __init__(self, module, name, alpha_step):
        self.name = name
        self.module = module
        self.act_scale = 0.0
        self.num_cache_steps = 0
        self.num_search_steps = 0
        self.block_size = _awq_block_size(module.weight, module.weight_quantizer)
        self.weight_scale = get_weight_scale(module.weight, self.block_size)
        self.loss = {k.item(): torch.zeros((), device=module.weight.device, dtype=torch.float32)
                     for k in torch.arange(0, 1.0 + alpha_step, alpha_step)}
        self.best_scale = None
        self.best_alpha = None
        self.is_input_quantized = module.input_quantizer.is_enabled
        self.is_enabled = True
        # error bits of the evaluation kernel's bounded waits (checked once, after the search)
        self.gemm_status = (torch.zeros((), dtype=torch.int32, device=module.weight.device)
                            if module.weight.is_cuda else None)
        self.side_stream = None   # second stream and two weight-sized buffers of the pipelined search
        self.wfq_bufs = None
        self.cand_scales = None   # (weight-side, input-side) scales of every candidate, [n_alpha, cin] each


def _evaluate_alpha(module, st, x2d, out_actual, alpha):
    """loss contribution of one alpha for one batch: mean((x/s) @ fq(W*s)^T - x @ W^T)^2."""
    s = get_scale(st.act_scale, st.weight_scale, alpha)
    dt = module.weight.dtype
    w_s, x_s = s.to(dt), (1 / s).to(dt)
    wq = module.weight_quantizer
    fast = (wq._fake_quant and isinstance(wq._num_bits, int) and st.block_size
            and module.weight.shape[-1] % st.block_size == 0 and wq._block_sizes.get("type", "static") == "static")
    if fast:
        # (W * s) rounded to the weight dtype, per-block abs-max, integer fake quant: one kernel
        wfq = ops.awq_scale_fake_int(module.weight, w_s, st.block_size, wq._num_bits, wq._unsigned, wq._narrow_range)
    else:
        wq._enable_pre_quant_scale = True
        wq.pre_quant_scale = w_s
        wfq = wq(module.weight)
        delattr(wq, "_pre_quant_scale")
    xin = x2d * x_s
    if module.input_quantizer.is_enabled:
        xin = module.input_quantizer(xin)
    x2 = xin.reshape(-1, xin.shape[-1])
    ref2 = out_actual.reshape(-1, out_actual.shape[-1])
    if USE_TENSOR_CORE_EVAL and module.bias is None and ops.awq_gemm_supported(x2, wfq):
        # GEMM and squared-error reduction in one tcgen05 kernel: the product never reaches memory
        acc = torch.zeros((), dtype=torch.float64, device=x2.device)
        ops.awq_gemm_sqerr(x2, wfq, ref2, acc, st.gemm_status)
        return (acc / ref2.numel()).to(torch.float32)
    out = F.linear(xin, wfq, module.bias)
    return ops.mse_loss(out, out_actual)


# evaluate every candidate of a batch in one persistent launch that forms the scaled, fake-quantised
# weight in shared memory on the way into the tensor cores (``b200q_awq_search_fused``)
FUSED_AWQ_SEARCH = True
# bytes of scaled activations (candidates x tokens x channels) formed per launch of the fused search
FUSED_AWQ_SEARCH_BYTES = 1 << 30
# batches with more rows than this hand the kernel finished weights instead of the raw weight
FUSED_AWQ_SEARCH_MAX_ROWS = 2048


# one grow-only buffer per device and dtype for the finished weights of a group of candidates, shared by
# all layers of a model (their searches run one after the other on the stream); dropped when awq_lite ends
_SEARCH_SCRATCH: dict = {}


def _search_scratch(device, dtype, numel):
    buf = _SEARCH_SCRATCH.get((device, dtype))
    if buf is None or buf.numel() < numel:
        buf = _SEARCH_SCRATCH[(device, dtype)] = torch.empty(numel, dtype=dtype, device=device)
    return buf[:numel]


def _search_fused(module, st, x2d, out_actual) -> bool:
    """All candidates of one batch by the fused kernel: per launch, one elementwise multiply forms
    the scaled activations of a group of candidates, then one kernel evaluates the whole group.
    Same arithmetic as ``_evaluate_alpha`` (the weight side bit for bit, the product to the fp32
    summation order); returns False when the layer is outside what the kernel covers."""
    wq = module.weight_quantizer
    w = module.weight
    fast = (wq._fake_quant and isinstance(wq._num_bits, int) and st.block_size
            and wq._block_sizes.get("type", "static") == "static")
    x2 = x2d.reshape(-1, x2d.shape[-1])
    ref2 = out_actual.reshape(-1, out_actual.shape[-1])
    if not (FUSED_AWQ_SEARCH and USE_TENSOR_CORE_EVAL and fast and module.bias is None
            and not module.input_quantizer.is_enabled and ops.awq_search_fused_supported(x2, w, st.block_size)):
        return False
    alphas = list(st.loss.keys())
    if st.cand_scales is None:   # constants of the layer once the statistics are final
        scales = torch.stack([get_scale(st.act_scale, st.weight_scale, a) for a in alphas])
        st.cand_scales = (scales.to(w.dtype), (1 / scales).to(w.dtype))
    w_s, x_s = st.cand_scales
    m, k = x2.shape
    # The kernel forms a candidate's weight in shared memory on its way into the tensor cores, once per
    # 512-row slab of the batch.  That is free while the tensor cores wait for operands anyway (measured:
    # 512 to 2048 rows, the fused form is as fast or faster); beyond that the repeated transform starts to
    # cost, so each candidate's weight is written once by the stand-alone weight-side kernel and the same
    # kernel runs on the finished weights (8192 rows: 17 ms against 19 ms for the up_proj shape).
    prequant = m > FUSED_AWQ_SEARCH_MAX_ROWS
    per_alpha = m * k * 2 + (w.numel() * 2 if prequant else 0)
    group = max(1, min(len(alphas), FUSED_AWQ_SEARCH_BYTES // max(1, per_alpha)))
    accs = torch.zeros(len(alphas), dtype=torch.float64, device=w.device)
    wq_all = _search_scratch(w.device, w.dtype, group * w.numel()).view(group, *w.shape) if prequant else None
    for g0 in range(0, len(alphas), group):
        g1 = min(len(alphas), g0 + group)
        a_all = ops.awq_scale_acts(x2, x_s[g0:g1])
        if prequant:
            for i in range(g0, g1):
                ops.awq_scale_fake_int(w, w_s[i], st.block_size, wq._num_bits, wq._unsigned, wq._narrow_range,
                                       out=wq_all[i - g0])
            ops.awq_search_prequant(a_all, wq_all[: g1 - g0], ref2, accs[g0:g1], st.gemm_status)
        else:
            ops.awq_search_fused(a_all, w, w_s[g0:g1], ref2, accs[g0:g1], st.gemm_status, st.block_size,
                                 wq._num_bits, wq._unsigned, wq._narrow_range)
    losses = (accs / ref2.numel()).to(torch.float32)
    for i, a in enumerate(alphas):
        st.loss[a] += losses[i]
    return True


# run the weight-side kernel of candidate i+1 on a second stream while the GEMM of candidate i runs
PIPELINE_AWQ_SEARCH = True


def _search_pipelined(module, st, x2d, out_actual) -> bool:
    """All candidates of one batch with the two kernels of consecutive candidates overlapped: the
    scale + block-quantise kernel (HBM and ALU bound) of candidate i+1 runs on a side stream into
    the other of two weight-sized buffers while the tcgen05 GEMM (tensor pipe, operands from L2)
    of candidate i runs on the current stream.  Same kernels, inputs and results as
    ``_evaluate_alpha``; returns False when the layer is outside what the two kernels cover."""
    wq = module.weight_quantizer
    w = module.weight
    fast = (wq._fake_quant and isinstance(wq._num_bits, int) and st.block_size
            and w.shape[-1] % st.block_size == 0 and wq._block_sizes.get("type", "static") == "static")
    x2 = x2d.reshape(-1, x2d.shape[-1])
    ref2 = out_actual.reshape(-1, out_actual.shape[-1])
    if not (PIPELINE_AWQ_SEARCH and USE_TENSOR_CORE_EVAL and fast and module.bias is None and w.is_cuda
            and ops.awq_gemm_supported(x2, w)):
        return False
    alphas = list(st.loss.keys())
    dev, dt = w.device, w.dtype
    main = torch.cuda.current_stream(dev)
    if st.side_stream is None:
        st.side_stream = torch.cuda.Stream(dev)
        st.wfq_bufs = [torch.empty_like(w), torch.empty_like(w)]
    side, bufs = st.side_stream, st.wfq_bufs
    scales = [get_scale(st.act_scale, st.weight_scale, a) for a in alphas]
    w_s = [s.to(dt) for s in scales]
    x_s = [(1 / s).to(dt) for s in scales]
    accs = torch.zeros(len(alphas), dtype=torch.float64, device=dev)
    side.wait_stream(main)                      # weight, scales and buffers are ready
    done_q = [torch.cuda.Event() for _ in alphas]
    done_g = [torch.cuda.Event() for _ in alphas]
    for i in range(len(alphas)):
        with torch.cuda.stream(side):
            if i >= 2:
                side.wait_event(done_g[i - 2])  # the GEMM that read this buffer has finished
            ops.awq_scale_fake_int(w, w_s[i], st.block_size, wq._num_bits, wq._unsigned, wq._narrow_range,
                                   out=bufs[i % 2])
            done_q[i].record(side)
        xin = x2d * x_s[i]
        if module.input_quantizer.is_enabled:
            xin = module.input_quantizer(xin)
        main.wait_event(done_q[i])
        ops.awq_gemm_sqerr(xin.reshape(-1, xin.shape[-1]), bufs[i % 2], ref2, accs[i:i + 1], st.gemm_status)
        done_g[i].record(main)
    side.wait_stream(main)
    losses = (accs / ref2.numel()).to(torch.float32)
    for i, a in enumerate(alphas):
        st.loss[a] += losses[i]
    return True


def _awq_forward(self, input, *args, **kwargs):
    st = self.awq_lite
    for q in (self.input_quantizer, self.weight_quantizer):
        if hasattr(q, "_pre_quant_scale"):
            delattr(q, "_pre_quant_scale")
    out_actual = F.linear(input, self.weight, self.bias)
    if input.numel() == 0 or not st.is_enabled:
        return out_actual
    if st.cache_mode_ref[0]:
        st.act_scale = st.act_scale + get_act_scale(input)
        st.num_cache_steps += 1
        if st.is_input_quantized:
            self.input_quantizer._calibrator.collect(input)
        return out_actual
    if not _search_fused(self, st, input, out_actual) and not _search_pipelined(self, st, input, out_actual):
        for alpha in st.loss:
            st.loss[alpha] += _evaluate_alpha(self, st, input, out_actual, alpha)
    st.num_search_steps += 1
    return out_actual


@torch.no_grad()
def awq_lite(model: nn.Module, forward_loop, alpha_step: float = 0.1, debug: bool = False, **kwargs):
    """AWQ-lite: per linear layer, search the exponent alpha of the per-input-channel scale
    s = act_scale^alpha / weight_scale^(1-alpha) that minimises the output error of the
    block-quantised layer, then fold the best scale into the weight and the input quantiser."""
    if forward_loop is None:
        warnings.warn("forward_loop must be provided for awq_lite; skipping awq_lite")
        return
    cache_mode = [True]
    layers = []
    for name, m in model.named_modules():
        if is_quantized_linear(m) and m.weight_quantizer.is_enabled:
            st = _AWQLiteState(m, name, alpha_step)
            st.cache_mode_ref = cache_mode
            m.awq_lite = st
            if m.input_quantizer.is_enabled:
                m.input_quantizer.disable()
                if m.input_quantizer.axis not in (None, -1):
                    st.is_enabled = False
                else:
                    m.input_quantizer.axis = -1
            m.__dict__["_forward_no_awq"] = m.forward
            m.__dict__["forward"] = _awq_forward.__get__(m, type(m))
            layers.append((name, m))

    # pass 1: activation statistics
    forward_loop(model)
    for name, m in layers:
        st = m.awq_lite
        if st.is_input_quantized and st.num_cache_steps > 0:
            m.input_quantizer.load_calib_amax()
    if dist.is_available() and dist.is_initialized():
        qdist.sync_amax(model)
    cached = [m.awq_lite for _, m in layers if m.awq_lite.num_cache_steps > 0]
    for st in cached:
        st.act_scale = st.act_scale / st.num_cache_steps
    if cached:
        # one device->host copy for all layers' NaN flags, one collective for all layers' statistics
        nan = torch.stack([torch.isnan(st.act_scale).any() | torch.isnan(st.weight_scale).any().to(st.act_scale.device)
                           for st in cached]).tolist()
        for st, bad in zip(cached, qdist.sync_awq_statistics([st.act_scale for st in cached], nan)):
            if bad:
                st.is_enabled = False

    # pass 2: search
    cache_mode[0] = False
    try:
        forward_loop(model)
    finally:
        _SEARCH_SCRATCH.clear()

    for name, m in layers:
        st = m.awq_lite
        del m.__dict__["forward"]
        del m.__dict__["_forward_no_awq"]
        if st.num_cache_steps == 0:
            st.is_enabled = False
        elif st.num_search_steps == 0:
            st.is_enabled = False
            warnings.warn(f"awq_lite: the second forward_loop(model) did not reach {name}.")
        if st.gemm_status is not None and int(st.gemm_status) != 0:
            raise RuntimeError(f"awq_lite: the evaluation kernel timed out in {name} (status {int(st.gemm_status)})")
        st.wfq_bufs = None
        if st.is_enabled:
            st.loss = {k: float(v) for k, v in st.loss.items()}
            st.best_alpha = min(st.loss, key=st.loss.get)
            st.best_scale = get_scale(st.act_scale, st.weight_scale, st.best_alpha)
        for q in (m.weight_quantizer, m.input_quantizer):
            if hasattr(q, "_pre_quant_scale"):
                delattr(q, "_pre_quant_scale")
        if st.is_input_quantized and m.input_quantizer.amax is not None:
            act_amax = m.input_quantizer.amax
            m.input_quantizer._amax_for_smoothing = act_amax.cpu()
            m.input_quantizer.reset_amax()
            m.input_quantizer.axis = None
            m.input_quantizer.amax = act_amax.amax()
            m.input_quantizer.enable()
        if st.is_enabled:
            apply_pre_quant_scale_and_smooth(m, 1.0 / st.best_scale)
        else:
            warnings.warn(f"awq_lite: Disabling for {name}, quantizing with max calibration.")
            max_calibrate(m, lambda mod: mod.weight_quantizer(mod.weight), distributed_sync=False)
        if not debug:
            delattr(m, "awq_lite")


# --------------------------------------------------------------------------------- AWQ clip ----

class _AWQClipState:
    """Search state of one linear layer (reference model_calib.py:807-849)."""

    def __init__(self, module, min_clip_ratio, shrink_step):
        self.num_tokens = 0
        self.block_size = _awq_block_size(module.weight, module.weight_quantizer)
        wq = module.weight_quantizer
        wq.reset_amax()
        enable_stats_collection(wq)
        wq(module.weight)
        finish_stats_collection(wq)
        self.w_amax = wq.amax.clone()
        self.ratios = [round(float(k), 2) for k in torch.arange(min_clip_ratio, 1.0, shrink_step)] + [1.0]
        co, ci = module.weight.shape
        dev = module.weight.device
        self.per_tensor = self._is_per_tensor_clip(wq)
        if self.per_tensor:
            self.loss_t = torch.zeros(len(self.ratios), dtype=torch.float32, device=dev)
        else:
            # a ragged last block is zero-padded (weights and tokens), as the reference pads them
            self.pad = (-ci) % self.block_size
            self.loss_t = torch.zeros((len(self.ratios), co, (ci + self.pad) // self.block_size),
                                      dtype=torch.float32, device=dev)
            self.ratios_t = torch.tensor(self.ratios, dtype=torch.float32, device=dev)
        self.best_clip_val = None
        self.best_loss = None
        self.is_input_quantized = module.input_quantizer.is_enabled
        wq.disable()

    @staticmethod
    def _is_per_tensor_clip(q):
        bs = q.block_sizes
        dynamic_per_tensor = bs is not None and bs.get("type", None) == "dynamic" and q.axis is None
        return dynamic_per_tensor or (q.axis is None and bs is None)

    @property
    def loss(self):
        """{clip ratio: loss} like the reference's dictionary."""
        return {r: self.loss_t[i] for i, r in enumerate(self.ratios)}


def _clip_search(module, st, inputs, max_tokens):
    wq = module.weight_quantizer
    wq.enable()
    if st.per_tensor:
        # only the per-tensor amax is clipped (NVFP4): whole-layer output error per ratio
        x2 = inputs.reshape(-1, inputs.shape[-1])
        out_actual = F.linear(x2, module.weight)
        original = wq.amax.clone()
        st.num_tokens += inputs.shape[0]
        for i, shrink in enumerate(st.ratios):
            wq.amax = original * shrink
            out = F.linear(x2, wq(module.weight))
            st.loss_t[i] += ops.mse_loss(out, out_actual)
        wq.amax = original
        return
    x2 = inputs.reshape(-1, inputs.shape[-1])
    x2 = x2[0:: max(1, x2.shape[0] // max_tokens)].contiguous()
    st.num_tokens += x2.shape[0]
    w, x2 = module.weight, x2.to(module.weight.dtype)
    if st.pad:
        w, x2 = F.pad(w, (0, st.pad)), F.pad(x2, (0, st.pad))
    ops.awq_clip_loss(w, x2, st.w_amax, st.ratios_t, st.loss_t, st.block_size, wq._num_bits, wq._unsigned,
                      wq._narrow_range)


def _awq_clip_forward(self, input, *args, **kwargs):
    st = self.awq_clip
    if st.is_input_quantized:
        self.input_quantizer.enable()
        max_calibrate(self.input_quantizer, lambda q: q(input), distributed_sync=False)
        self.input_quantizer.disable()
    _clip_search(self, st, self.input_quantizer(input), st.max_tokens)
    self.weight_quantizer.disable()
    return self._forward_no_awq(input, *args, **kwargs)


@torch.no_grad()
def awq_clip(model: nn.Module, forward_loop, max_co_batch_size: int = 1024, max_tokens_per_batch: int = 64,
             min_clip_ratio: float = 0.5, shrink_step: float = 0.05, debug: bool = False, **kwargs):
    """AWQ-clip (reference model_calib.py:788-997): per weight block, pick the clip ratio of the
    block amax whose fake-quantised block changes the block's partial outputs least on a sample
    of the calibration tokens.  ``max_co_batch_size`` (the reference's memory knob) is accepted
    and unused: the search kernel never materialises the per-ratio products."""
    assert forward_loop is not None, "forward_loop must be provided for awq_clip"
    layers = []
    for name, m in model.named_modules():
        if is_quantized_linear(m) and m.weight_quantizer.is_enabled and m.weight_quantizer.block_sizes is not None:
            wq = m.weight_quantizer
            if not isinstance(wq._num_bits, int) and not _AWQClipState._is_per_tensor_clip(wq):
                raise NotImplementedError("awq_clip: block-wise search is built for integer weight formats")
            st = _AWQClipState(m, min_clip_ratio, shrink_step)
            st.max_tokens = max_tokens_per_batch
            m.awq_clip = st
            m.__dict__["_forward_no_awq"] = m.forward
            m.__dict__["forward"] = _awq_clip_forward.__get__(m, type(m))
            layers.append((name, m))
    enable_stats_collection(model)
    forward_loop(model)
    max_calibrate(model, lambda mod: None)
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    for name, m in layers:
        st = m.awq_clip
        del m.__dict__["forward"]
        del m.__dict__["_forward_no_awq"]
        if st.num_tokens > 0:
            if world > 1 and not st.per_tensor:   # the reference averages every block loss over the DP group
                dist.all_reduce(st.loss_t, op=dist.ReduceOp.SUM)
                st.loss_t /= world
            best_loss = torch.full_like(st.w_amax, float("inf"), dtype=torch.float32)
            best_clip = torch.zeros_like(st.w_amax)
            for i, shrink in enumerate(st.ratios):
                loss = st.loss_t[i].reshape(st.w_amax.shape)
                better = loss < best_loss
                best_loss = torch.where(better, loss, best_loss)
                best_clip = torch.where(better, st.w_amax * shrink, best_clip)
            st.best_loss, st.best_clip_val = best_loss, best_clip
            m.weight_quantizer.amax = best_clip
            m.weight_quantizer.enable()
            if st.is_input_quantized:
                m.input_quantizer.enable()
        if not debug:
            delattr(m, "awq_clip")


# --------------------------------------------------------------------------------- SmoothQuant --

@torch.no_grad()
def smoothquant(model: nn.Module, forward_loop=None, alpha: float = 1.0):
    """SmoothQuant for INT8 linears (reference model_calib.py:411-496): per-input-channel activation
    amax from a max calibration with ``axis=-1``, smoothing scale
    ``s = w_max^(1-alpha) / a_max^alpha`` folded into the weight (and its inverse into the input
    quantiser's pre-quant scale), then per-tensor activation quantisation."""
    assert forward_loop is not None, "forward_loop must be provided for smoothquant"
    from .utils import reduce_amax

    for _, m in model.named_modules():
        if is_quantized_linear(m) and m.input_quantizer.is_enabled and m.input_quantizer.axis is None:
            m.input_quantizer.axis = -1
    max_calibrate(model, forward_loop)
    smoothed = 0
    for name, m in model.named_modules():
        if not is_quantized_linear(m):
            continue
        iq, wq = m.input_quantizer, m.weight_quantizer
        if not hasattr(iq, "_amax"):
            warnings.warn(f"{name} is not calibrated, skip smoothing")
            continue
        if iq.num_bits != 8 or wq.num_bits != 8:
            warnings.warn(f"Only int8 smoothing is supported, skip {name}")
            continue
        if iq.axis != -1:
            warnings.warn(f"Only per-channel smoothing is supported, skip {name}")
            continue
        assert iq._amax.numel() > 1, f"Error: {name} has only one channel to smooth"
        act_amax = iq.amax.float()
        weight_scale = reduce_amax(m.weight, axis=0, keepdims=True)
        dev, dt = m.weight.device, m.weight.dtype
        scale_a = (weight_scale.pow(1 - alpha) / act_amax.pow(alpha)).squeeze()
        iq._amax_for_smoothing = act_amax.cpu()
        iq.reset_amax()
        iq.axis = None
        iq.amax = act_amax.amax().to(dtype=dt, device=dev)
        epsilon = 1.0 / (1 << 31)
        if scale_a.min() <= epsilon:   # channels that never fired
            scale_a[(act_amax <= epsilon).reshape(scale_a.shape)] = 1
        scale_a = scale_a.clamp(min=1e-4, max=1e4)
        apply_pre_quant_scale_and_smooth(m, scale_a)
        smoothed += 1
    return smoothed


def awq(model, forward_loop=None, algorithm="awq_lite", **kwargs):
    """AWQ entry point (reference model_calib.py:499-526): ``awq_lite``, ``awq_clip`` or
    ``awq_full`` (lite, then clip)."""
    if algorithm not in ("awq_lite", "awq_clip", "awq_full"):
        raise NotImplementedError(f"AWQ variant {algorithm!r} is outside the accelerated path")
    lite_kw = {k: v for k, v in kwargs.items() if k in ("alpha_step", "debug")}
    clip_kw = {k: v for k, v in kwargs.items()
               if k in ("max_co_batch_size", "max_tokens_per_batch", "min_clip_ratio", "shrink_step", "debug")}
    with SequentialQuantizer.convert_to_single_quantizer(model):
        if algorithm in ("awq_full", "awq_lite"):
            awq_lite(model, forward_loop, **lite_kw)
        if algorithm in ("awq_full", "awq_clip"):
            awq_clip(model, forward_loop, **clip_kw)
    for _, m in model.named_modules():
        if is_quantized_linear(m) and isinstance(m.weight_quantizer, SequentialQuantizer):
            max_calibrate(m, lambda lin: lin.weight_quantizer(lin.weight), distributed_sync=False)
