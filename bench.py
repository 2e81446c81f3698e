#!/usr/bin/env python
"""Benchmark of the NVFP4 weight quantisation path on the Llama-3-8B linear-weight shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = NVFP4 real quantisation + packing (global abs-max pass, then block-scale / E2M1 /
pack pass) of every linear weight of a random-init Llama-3-8B-shaped model: 32 layers of
q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096, down 4096x14336, bf16, Student-t(4) values
scaled to std 0.02.  With N GPUs the 32 layers are split across the ranks (strong scaling, no
data-path collective).  Prints one JSON line (rank 0) with, beside the contract's keys:

  roofline      the quantise kernel against the measured copy bandwidth (and the nominal 8 TB/s)
  e2e           mtq.compress on a host-resident (pinned) module tree, with the copy-only ceiling beside it
  calibration   data-parallel max and histogram calibration of the model's 224 input quantisers, every
                rank on its own batches, exchanges included (at every N)
  cpu_baseline  the reference's CPU torch path on the host cores (N = 1), also for the other formats
  formats       the other kernels of the path (N = 1): fake quant, calibration, INT4, MSE, dequantise, the
                awq_lite search, the real-quant GEMMs, and the reference's own GPU kernels timed beside ours

``--impl reference`` times the reference's CPU torch path (restated operation by operation in
oracle/torch_path.py) on the host cores for a bounded sample of the same workload, and reports a
fused multi-threaded C restatement (oracle/nvfp4_ref.c) beside it.  ``--workload calib70b`` runs the
calibration phases on Llama-3-70B shapes followed by that model's weight quantisation.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tensorrt-model-optimizer_b200"))

LAYER_SHAPES = [("q_proj", (4096, 4096)), ("k_proj", (1024, 4096)), ("v_proj", (1024, 4096)),
                ("o_proj", (4096, 4096)), ("gate_proj", (14336, 4096)), ("up_proj", (14336, 4096)),
                ("down_proj", (4096, 14336))]
N_LAYERS = 32
ELEMS_PER_LAYER = sum(a * b for _, (a, b) in LAYER_SHAPES)
# algorithmic bytes per element: abs-max pass reads 2 B; quantise pass reads 2 B, writes 0.5 B of
# codes and 1/16 B of block scale
BYTES_AMAX = 2.0
BYTES_QUANT = 2.0 + 0.5 + 1.0 / 16
BYTES_TOTAL = BYTES_AMAX + BYTES_QUANT
# DRAM bytes per element of the quantise kernel from the committed ncu capture
# (profiles/nvfp4_group_kernels_1layer_ncu_full.md: one layer's seven tensors, traffic in proportion to
# the elements processed)
NCU_QUANT_TRAFFIC_PER_ELEM = 2.477
NOMINAL_HBM_GBS = 8000.0      # B200 data-sheet HBM3e bandwidth, beside the measured copy bandwidth
LLAMA8B = {"hidden": 4096, "kv": 1024, "inter": 14336, "layers": 32}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_weight(shape, seed, device):
    """Student-t(4) scaled to std 0.02 (Var t4 = 2), bf16, from a per-tensor seed."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    z = torch.randn(shape, generator=g, device=device)
    chi = torch.zeros(shape, device=device)
    for _ in range(4):
        chi += torch.randn(shape, generator=g, device=device) ** 2
    w = z / (chi / 4).sqrt() * (0.02 / 2 ** 0.5)
    return w.to(torch.bfloat16)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for t, r in self.rows if (t0 is None or t >= t0 - 0.1) and (t1 is None or t <= t1 + 0.1)]
        if not rows:
            rows = [r for _, r in self.rows]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0])); smax.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------- CPU arm -------

def cpu_nvfp4_sample(seconds_target: float = 15.0, threads: int | None = None):
    """Time the oracle's NVFP4 quantisation (the reference's torch-path arithmetic, numpy) on host
    cores over row chunks of k_proj-shaped weights; returns (GB/s of algorithmic bytes, info)."""
    import numpy as np

    from oracle import cref
    from oracle import quant_oracle as qo

    threads = threads or os.cpu_count() or 1
    lib = cref.load()
    rng = np.random.default_rng(0)
    rows, cols = 14336, 4096
    w = rng.standard_t(4, size=(rows, cols)).astype(np.float32) * np.float32(0.02 / 2 ** 0.5)
    bits = (qo.round_bf16(w).view(np.uint32) >> 16).astype(np.uint16).reshape(-1)
    out = (np.empty(bits.size // 2, np.uint8), np.empty(bits.size // 16, np.uint8))

    def one_pass():
        # abs-max pass + quantise/pack pass, as the reference's NVFP4QTensor.quantize does
        cref.nvfp4_quantize_bf16(lib, bits, -1.0, threads, out)

    one_pass()
    t0 = time.perf_counter()
    one_pass()
    dt1 = time.perf_counter() - t0
    reps = max(1, min(50, int(seconds_target / max(dt1, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        one_pass()
    dt = (time.perf_counter() - t0) / reps
    gbs = rows * cols * BYTES_TOTAL / dt / 1e9
    return gbs, {"cores": threads, "kind": "port",
                 "sample": f"{reps} passes over one gate_proj-shaped weight [{rows},{cols}] bf16 "
                           f"({dt * 1e3:.1f} ms per pass), C restatement of the reference's torch path "
                           f"(oracle/nvfp4_ref.c), {threads} threads"}


def cpu_torch_path_sample(seconds_target: float = 15.0):
    """Time the reference's CPU torch path (oracle/torch_path.py: the same sequence of torch tensor
    operations as NVFP4QTensor.quantize on a CPU tensor, all intra-op threads) on one gate_proj-shaped
    bf16 weight; returns (GB/s of algorithmic bytes, info)."""
    import torch

    from oracle import torch_path

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows, cols = 14336, 4096
    g = torch.Generator().manual_seed(0)
    z = torch.randn(rows, cols, generator=g)
    chi = sum(torch.randn(rows, cols, generator=g) ** 2 for _ in range(4)) / 4
    w = (z / chi.sqrt() * (0.02 / 2 ** 0.5)).to(torch.bfloat16)
    del z, chi
    t0 = time.perf_counter()
    torch_path.nvfp4_quantize(w, 16)
    dt1 = time.perf_counter() - t0
    reps = max(1, min(20, int(seconds_target / max(dt1, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        torch_path.nvfp4_quantize(w, 16)
    dt = (time.perf_counter() - t0) / reps
    gbs = rows * cols * BYTES_TOTAL / dt / 1e9
    return gbs, {"cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"{reps} passes over one gate_proj-shaped weight [{rows},{cols}] bf16 "
                           f"({dt * 1e3:.0f} ms per pass): the reference's CPU torch path, restated operation by "
                           f"operation (oracle/torch_path.py), torch intra-op threads = {torch.get_num_threads()}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    per_step = max(2.0, min(20.0, 120.0 / (steps + warm)))
    vals = []
    info = None
    for i in range(steps + warm):
        gbs, info = cpu_torch_path_sample(per_step)
        if i >= warm:
            vals.append(gbs)
    v = statistics.mean(vals)
    c_gbs, c_info = cpu_nvfp4_sample(5.0)
    info["fused_c_port"] = {"value": c_gbs, "unit": "GB/s", **c_info}
    ms_full = N_LAYERS * ELEMS_PER_LAYER * BYTES_TOTAL / (v * 1e9) * 1e3
    line = {
        "impl": "reference", "metric": "nvfp4_weight_quantize_hbm_gbps", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms_full,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "llama3-8b-shape linear weights (224 tensors, 6.98e9 elements), NVFP4 "
                               "real quantize + pack: fp32 global scale, E4M3 scale per 16, E2M1 nibbles",
                   "layers": N_LAYERS, "bytes_per_element": BYTES_TOTAL,
                   "note": "each step is a bounded sample (one gate_proj-shaped tensor, repeated); value is its "
                           "throughput in the same algorithmic bytes, ms_per_step the extrapolation to the "
                           "full 32-layer model"},
        "cpu_baseline": {"value": v, "unit": "GB/s", **info},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))



# ------------------------------------------------------------ data-parallel calibration --------

def calibration_phases(dev, world, rank, dims, n_layers, tokens, batches):
    """Data-parallel activation calibration of every linear input of a Llama-shaped stack: each rank
    calibrates on its own batches, the statistics are merged over the ranks.

    The forward GEMMs that would produce the activations are not part of this path, so each kind of
    activation (attention input, o_proj input, MLP input, down_proj input) is one seeded synthetic
    [tokens, dim] bf16 buffer per rank, fed ``batches`` times per layer to that layer's input quantisers
    (q/k/v share the attention input, gate/up the MLP input, as they do in the model).
      max        the NVFP4 default: running abs-max per quantiser, one MAX all-reduce of all amax values;
      histogram  2048 bins, percentile 99.99: ranges observed on the device, rank 0's broadcast in place,
                 shared binning passes, one in-place SUM all-reduce of the counter arena, read-out.
    Returns seconds per phase (max over ranks), launches, bytes and whether all ranks ended with the same
    amax values."""
    import torch
    import torch.distributed as dist

    from b200q import dist as qdist
    from b200q import ops
    from b200q.calib import attach_histogram_arena
    from b200q.model_calib import load_calib_amax_all
    from b200q.nn import TensorQuantizer

    H, KV, I = dims["hidden"], dims["kv"], dims["inter"]
    kinds = [("attn_in", H, ("q_proj", "k_proj", "v_proj")), ("o_in", H, ("o_proj",)),
             ("mlp_in", H, ("gate_proj", "up_proj")), ("down_in", I, ("down_proj",))]
    acts = {}
    for k, (name, dim, _) in enumerate(kinds):
        g = torch.Generator(device=dev).manual_seed(50_000 + 16 * rank + k)
        ch = torch.exp(torch.randn(dim, generator=g, device=dev))          # lognormal(0,1) channel magnitudes
        acts[name] = (torch.randn(tokens, dim, generator=g, device=dev) * ch).bfloat16()

    def build(calibrator, layers):
        qcfg = {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)},
                "axis": None, "enable": True, "calibrator": calibrator}
        model = torch.nn.ModuleDict()
        for l in range(layers):
            for _, _, lins in kinds:
                for lin in lins:
                    q = TensorQuantizer(dict(qcfg))
                    q.disable_quant(); q.enable_calib()
                    model[f"l{l}_{lin}"] = q
        return model

    def feed(model, layers, n_batches, observe=False):
        for l in range(layers):
            for _ in range(n_batches):
                for name, _, lins in kinds:
                    for lin in lins:
                        if observe:
                            model[f"l{l}_{lin}"]._calibrator.observe_range(acts[name])
                        else:
                            model[f"l{l}_{lin}"](acts[name])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def phase(fn):
        barrier()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = t.item()
        return dt

    def same_everywhere(model):
        amaxes = torch.stack([q._amax.float().reshape(()) for q in model.values()])
        if world > 1:
            lo, hi = amaxes.clone(), amaxes.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            return bool(torch.equal(lo, hi)), amaxes
        return True, amaxes

    def run_max(layers, n_batches):
        model = build("max", layers)
        t_collect = phase(lambda: feed(model, layers, n_batches))
        t_readout = phase(lambda: load_calib_amax_all([(n, q, (), {}) for n, q in model.items()]))
        t_exchange = phase(lambda: qdist.sync_amax(model))
        return model, {"collect": t_collect, "readout": t_readout, "exchange": t_exchange}

    def run_hist(layers, n_batches):
        model = build("histogram", layers)
        attach_histogram_arena(model)
        t_observe = phase(lambda: feed(model, layers, 1, observe=True))       # first batch: abs-max into the range slots
        t_ranges = phase(lambda: qdist.agree_histogram_ranges(model))
        t_collect = phase(lambda: (feed(model, layers, n_batches), [a.flush() for a in {id(q._calibrator._arena): q._calibrator._arena for q in model.values()}.values()]))
        t_exchange = phase(lambda: qdist.sync_histograms(model))
        t_readout = phase(lambda: load_calib_amax_all(
            [(n, q, ("percentile",), {"percentile": 99.99}) for n, q in model.items()]))
        return model, {"observe": t_observe, "ranges": t_ranges, "collect": t_collect, "exchange": t_exchange, "readout": t_readout}

    # warm-up: kernels, allocator blocks of the sizes the timed pass uses, and the communicator's collectives
    run_max(n_layers, 1); run_hist(n_layers, 1)
    if world > 1:
        for op in (dist.ReduceOp.MAX, dist.ReduceOp.SUM):
            for _ in range(3):
                dist.all_reduce(torch.zeros(1 << 20, dtype=torch.int64, device=dev), op=op)
    m_max, t_max = run_max(n_layers, batches)
    same_max, _ = same_everywhere(m_max)
    del m_max
    m_hist, t_hist = run_hist(n_layers, batches)
    same_hist, amaxes = same_everywhere(m_hist)
    n_quant = len(m_hist)
    arena_bytes = sum(a.counts.numel() * 8 for a in {id(q._calibrator._arena): q._calibrator._arena for q in m_hist.values()}.values())
    del m_hist
    per_q_elems = n_layers * batches * tokens * (6 * H + I)          # every quantiser's own input, per rank
    distinct_elems = n_layers * batches * tokens * (3 * H + I)       # the four distinct tensors, per rank
    peak, which = peaks()
    return {
        "shapes": {"hidden": H, "kv": KV, "inter": I, "layers": n_layers}, "quantizers": n_quant,
        "tokens_per_batch_per_rank": tokens, "batches_per_rank_per_layer": batches,
        "max": {"seconds": t_max, "total_s": sum(t_max.values()), "launches_per_rank": n_layers * batches * 7,
                "bytes_read_per_rank": per_q_elems * 2,
                "collect_gbps_all_ranks": world * per_q_elems * 2 / t_max["collect"] / 1e9,
                "collect_frac_of_peak_per_gpu": per_q_elems * 2 / t_max["collect"] / 1e9 / peak,
                "collectives": {"all_reduce_max": 1}},
        "histogram": {"seconds": t_hist, "total_s": sum(t_hist.values()),
                      "binning_launches_per_rank": n_layers * batches * 4,
                      "bytes_read_per_rank": distinct_elems * 2,
                      "note": "q/k/v and gate/up bin their common input in one pass: bytes are the four distinct "
                              "tensors per layer and batch",
                      "collect_gbps_all_ranks": world * distinct_elems * 2 / t_hist["collect"] / 1e9,
                      "collect_frac_of_peak_per_gpu": distinct_elems * 2 / t_hist["collect"] / 1e9 / peak,
                      "collectives": {"broadcast": 1, "all_reduce_sum": 2, "arena_bytes": arena_bytes},
                      "amax_range": [float(amaxes.min()), float(amaxes.max())]},
        "amax_identical_on_all_ranks": bool(same_max and same_hist), "peak_source": f"of {which}",
    }

# ------------------------------------------------------------------------------- GPU arm -------

def split_layers(n_layers: int, world: int, rank: int):
    per = n_layers // world
    extra = n_layers % world
    lo = rank * per + min(rank, extra)
    return list(range(lo, lo + per + (1 if rank < extra else 0)))


def run_b200(args):
    import torch
    import torch.distributed as dist

    from b200q.ops import NvFp4Group
    from b200q.pipeline import HostNvFp4Packer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the kernels)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    layers = split_layers(args.layers, world, rank)

    # ---- resident inputs ---------------------------------------------------------------------
    weights = []
    for l in layers:
        for k, (_, shape) in enumerate(LAYER_SHAPES):
            weights.append(make_weight(shape, l * len(LAYER_SHAPES) + k, dev))
    group = NvFp4Group(weights) if weights else None
    my_elems = sum(w.numel() for w in weights)
    total_elems = args.layers * ELEMS_PER_LAYER
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if group is not None:
            group.run()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.25)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    from b200q._cabi import call
    from b200q.ops import _DT
    barrier()
    t_wall0 = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        if group is None:
            continue
        # same two launches as group.run(), with an event between them so that each kernel's
        # duration is known
        st = torch.cuda.current_stream().cuda_stream
        group.amax.zero_()
        ev[i][0].record()
        call("b200q_nvfp4_group_amax", group._descs.data_ptr(), group.n, group.total_tiles, _DT[group.dtype], st)
        ev[i][1].record()
        call("b200q_nvfp4_group_quantize", group._descs.data_ptr(), group.n, group.total_tiles, _DT[group.dtype], st)
        ev[i][2].record()
    end.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms = start.elapsed_time(end)
    clocks = sampler.stop(t_wall0, t_wall1)
    amax_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev) if group is not None else 0.0
    quant_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev) if group is not None else 0.0
    if world > 1:
        t = torch.tensor([ms, amax_ms, quant_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, amax_ms, quant_ms = t.tolist()
    ms_per_step = ms / args.steps
    value = total_elems * BYTES_TOTAL / (ms_per_step * 1e-3) / 1e9

    # ---- data-parallel activation calibration on the same model's shapes (every rank its own batches)
    calibration = None
    if not args.no_calibration:
        calibration = calibration_phases(dev, world, rank, LLAMA8B, args.layers, args.tokens, args.batches)
        calibration["ptq_seconds_weights_plus_max_calibration"] = ms_per_step * 1e-3 + calibration["max"]["total_s"]
        calibration["ptq_seconds_weights_plus_histogram_calibration"] = (
            ms_per_step * 1e-3 + calibration["histogram"]["total_s"])

    # ---- end to end: mtq.compress on a host-resident model (pinned weights in, packed weights out)
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, weights, layers, dev, world, total_elems, barrier)

    # ---- CPU baseline (rank 0, N=1 only) ---------------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu:
        gbs, info = cpu_torch_path_sample(12.0)
        cpu = {"value": gbs, "unit": "GB/s", **info}
        c_gbs, c_info = cpu_nvfp4_sample(6.0)
        cpu["fused_c_port"] = {"value": c_gbs, "unit": "GB/s", **c_info}
        cpu["other_configs"] = cpu_other_configs()

    formats = None
    if world == 1 and not args.no_formats:
        del group, weights
        torch.cuda.empty_cache()
        formats = run_formats(dev, peaks()[0])
        formats["reference_gpu_kernels"] = run_reference_gpu_kernels(dev, peaks()[0])

    if rank == 0:
        peak, which = peaks()
        per_rank_elems = my_elems  # rank 0's share; shares are equal when world divides the layers
        achieved = per_rank_elems * BYTES_QUANT / (quant_ms * 1e-3) / 1e9 if quant_ms else None
        achieved_amax = per_rank_elems * BYTES_AMAX / (amax_ms * 1e-3) / 1e9 if amax_ms else None
        line = {
            "metric": "nvfp4_weight_quantize_hbm_gbps", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "llama3-8b-shape linear weights (224 tensors, 6.98e9 elements), NVFP4 "
                                   "real quantize + pack: fp32 global scale, E4M3 scale per 16, E2M1 nibbles",
                       "layers": args.layers, "sharding": f"layers split over {world} rank(s)",
                       "l2": "inputs (>=1.7 GB per rank) are larger than L2; no flush needed",
                       "bytes_per_element": BYTES_TOTAL, "ptq_seconds": ms_per_step * 1e-3,
                       "tensors_per_second": args.layers * len(LAYER_SHAPES) / (ms_per_step * 1e-3)},
            "roofline": {"bound": "hbm", "kernel": "nvfp4_group_quantize_kernel", "achieved": achieved,
                         "peak": peak, "peak_source": f"of {which}", "unit": "GB/s",
                         "frac": achieved / peak if achieved else None,
                         "frac_of_nominal": achieved / NOMINAL_HBM_GBS if achieved else None,
                         "nominal_peak": NOMINAL_HBM_GBS,
                         "traffic": NCU_QUANT_TRAFFIC_PER_ELEM * per_rank_elems
                         if NCU_QUANT_TRAFFIC_PER_ELEM else None,
                         "algorithmic_bytes_per_launch": per_rank_elems * BYTES_QUANT,
                         "ms_per_launch": quant_ms,
                         "amax_kernel": {"achieved": achieved_amax, "frac": achieved_amax / peak
                                         if achieved_amax else None, "ms_per_launch": amax_ms}},
            "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "gpu_launches": 2 * args.steps,
            "calibration": calibration, "formats": formats,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_formats(dev, peak):
    """Achieved algorithmic GB/s of the other formats' kernels (BASELINE configs 1, 2, 4 and the
    histogram pass of config 5), each over inputs larger than L2 (several distinct tensors used
    in turn), timed with CUDA events after 3 warm-up passes."""
    import torch

    from b200q import ops

    def timed(fn, n_bytes, reps=5, groups=5):
        """median over `groups` of the mean time of `reps` back-to-back passes (CUDA events)"""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(groups):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / reps)
        ms = statistics.median(times)
        gbs = n_bytes / (ms * 1e-3) / 1e9
        return {"gbps": gbs, "frac_of_measured_peak": gbs / peak, "ms": ms, "algorithmic_bytes": n_bytes}

    out = {}
    g = torch.Generator(device=dev).manual_seed(0)
    # config 1: INT8 per-row (axis 0, narrow) fake quant of fp32 [4096,4096] fused with the row amax
    w32 = [torch.randn(4096, 4096, generator=g, device=dev) * 0.02 for _ in range(8)]
    out["int8_per_row_fused_amax_fp32_4096x4096"] = timed(
        lambda: [ops.fake_int_rows_dynamic(w, 8, False, True) for w in w32], 8 * 4096 * 4096 * 8)
    del w32
    # config 2: FP8 per-tensor, 16 batches of bf16 [8192,4096] with outlier channels
    idx = torch.randperm(4096, generator=torch.Generator().manual_seed(7))[:4].to(dev)
    xs = []
    for b in range(16):
        x = torch.randn(8192, 4096, generator=torch.Generator(device=dev).manual_seed(1000 + b), device=dev)
        x[:, idx] *= 50
        xs.append(x.bfloat16())
    amax = torch.zeros((), device=dev)
    n = 16 * 8192 * 4096
    out["fp8_max_calibration_bf16_16x8192x4096"] = timed(lambda: [ops.amax_tensor(x, out=amax) for x in xs], n * 2)
    out["fp8_per_tensor_fake_quant_bf16_16x8192x4096"] = timed(lambda: [ops.fake_e4m3(x, amax) for x in xs], n * 4)
    out["nvfp4_fake_quant_bf16_16x8192x4096"] = timed(lambda: [ops.nvfp4_fake(x, amax) for x in xs], n * 4)
    # histogram pass of config 5 (2048 bins) on the same activations
    counts = torch.zeros(2048, dtype=torch.int64, device=dev)
    rmax = float(amax)
    out["histogram_2048_bins_bf16_16x8192x4096"] = timed(lambda: [ops.hist_collect(x, counts, 2048, rmax) for x in xs], n * 2)
    # MSE calibration: 10 candidate amax values in one pass over each batch (instruction-issue bound)
    cands = (amax.reshape(1, 1) * torch.linspace(0.25, 4.0, 10, device=dev).reshape(-1, 1)).contiguous()
    mse_loss = torch.zeros(10, 1, dtype=torch.float64, device=dev)
    out["mse_10_candidates_int8_bf16_16x8192x4096"] = timed(
        lambda: [ops.mse_candidates(x, cands, mse_loss, None, 8, False, True) for x in xs], n * 2)
    out["mse_10_candidates_e4m3_bf16_16x8192x4096"] = timed(
        lambda: [ops.mse_candidates(x, cands, mse_loss, None, (4, 3), False, True) for x in xs], n * 2)
    # NVFP4 dequantise (the export format back to bf16): reads 0.5 B + 1/16 B per element, writes 2 B
    packed = [ops.nvfp4_quantize(x, amax=amax) for x in xs]
    out["nvfp4_dequantize_bf16_16x8192x4096"] = timed(
        lambda: [ops.nvfp4_dequantize(p, sc, s2, torch.bfloat16) for p, sc, s2 in packed], int(n * (0.5 + 1 / 16 + 2)))
    del xs, packed
    # config 4: INT4 block-128 amax + pack, and the per-alpha weight-side kernel of awq_lite
    ws = [(torch.randn(14336, 4096, generator=g, device=dev) * 0.02).bfloat16() for _ in range(3)]
    s = torch.exp(torch.randn(4096, generator=g, device=dev)).bfloat16()
    n = 3 * 14336 * 4096
    out["int4_block128_quantize_pack_bf16_14336x4096"] = timed(
        lambda: [ops.int4_quantize(w.reshape(-1), 128) for w in ws], int(n * (2 + 0.5 + 2 / 128)))
    out["awq_scale_fake_int4_bf16_14336x4096"] = timed(
        lambda: [ops.awq_scale_fake_int(w, s, 128, 4, False, False) for w in ws], n * 4)
    # config 4: the awq_lite search of one layer (up_proj shape): 21 candidates, each = fused
    # scale + INT4 block fake quant of W, then the tcgen05 GEMM with the squared-error epilogue
    x = (torch.randn(512, 4096, generator=g, device=dev) * torch.exp(torch.randn(4096, generator=g, device=dev))).bfloat16()
    w = ws[0]
    ref = torch.nn.functional.linear(x, w)
    acc = torch.zeros((), dtype=torch.float64, device=dev)
    status = torch.zeros((), dtype=torch.int32, device=dev)
    scales = [torch.exp(0.05 * i * torch.randn(4096, generator=g, device=dev)).bfloat16() for i in range(21)]

    def search_sequential():
        for sc in scales:
            wfq = ops.awq_scale_fake_int(w, sc, 128, 4, False, False)
            ops.awq_gemm_sqerr(x, wfq, ref, acc, status)

    # what awq_lite runs (b200q.model_calib._search_pipelined): the weight-side kernel of candidate
    # i+1 on a second stream while the GEMM of candidate i runs, two weight-sized buffers
    side = torch.cuda.Stream(dev)
    bufs = [torch.empty_like(w), torch.empty_like(w)]

    def search():
        main = torch.cuda.current_stream(dev)
        side.wait_stream(main)
        done_q = [torch.cuda.Event() for _ in scales]
        done_g = [torch.cuda.Event() for _ in scales]
        for i, sc in enumerate(scales):
            with torch.cuda.stream(side):
                if i >= 2:
                    side.wait_event(done_g[i - 2])
                ops.awq_scale_fake_int(w, sc, 128, 4, False, False, out=bufs[i % 2])
                done_q[i].record(side)
            main.wait_event(done_q[i])
            ops.awq_gemm_sqerr(x, bufs[i % 2], ref, acc, status)
            done_g[i].record(main)
        side.wait_stream(main)

    flops = 21 * 2.0 * 512 * 4096 * 14336
    r = timed(search, 21 * 14336 * 4096 * 4, reps=3, groups=3)
    out["awq_lite_search_21_alphas_up_proj_512tok"] = {
        "ms": r["ms"], "gemm_tflops_incl_quant_kernel": flops / (r["ms"] * 1e-3) / 1e12,
        "schedule": "scale+quantise kernel of candidate i+1 on a second stream under the GEMM of candidate i"}
    r = timed(search_sequential, 21 * 14336 * 4096 * 4, reps=3, groups=3)
    out["awq_lite_search_21_alphas_one_stream"] = {
        "ms": r["ms"], "gemm_tflops_incl_quant_kernel": flops / (r["ms"] * 1e-3) / 1e12}
    wfq = ops.awq_scale_fake_int(w, scales[1], 128, 4, False, False)
    r = timed(lambda: [ops.awq_gemm_sqerr(x, wfq, ref, acc, status) for _ in range(21)], 1, reps=3, groups=3)
    tf = flops / (r["ms"] * 1e-3) / 1e12
    out["awq_gemm_sqerr_tcgen05_512x14336x4096"] = {"ms_per_gemm": r["ms"] / 21, "tflops": tf,
                                                    "kernel_status": int(status)}
    r = timed(lambda: [torch.nn.functional.linear(x, wfq) for _ in range(21)], 1, reps=3, groups=3)
    out["cublas_linear_512x14336x4096_for_comparison"] = {"ms_per_gemm": r["ms"] / 21,
                                                          "tflops": flops / (r["ms"] * 1e-3) / 1e12}
    # the down projection of the same MLP (few tiles, long K): K split over two CTAs per tile
    xd = torch.randn(512, 14336, generator=g, device=dev).bfloat16()
    wd = (torch.randn(4096, 14336, generator=g, device=dev) * 0.02).bfloat16()
    refd = torch.nn.functional.linear(xd, wd)
    r = timed(lambda: [ops.awq_gemm_sqerr(xd, wd, refd, acc, status) for _ in range(21)], 1, reps=3, groups=3)
    out["awq_gemm_sqerr_tcgen05_512x4096x14336"] = {
        "ms_per_gemm": r["ms"] / 21, "tflops": flops / (r["ms"] * 1e-3) / 1e12,
        "k_splits": ops.awq_gemm_splits(512, 4096, 14336, dev), "kernel_status": int(status)}
    r = timed(lambda: [torch.nn.functional.linear(xd, wd) for _ in range(21)], 1, reps=3, groups=3)
    out["cublas_linear_512x4096x14336_for_comparison"] = {"ms_per_gemm": r["ms"] / 21,
                                                          "tflops": flops / (r["ms"] * 1e-3) / 1e12}
    # the search as awq_lite runs it now: one activation-scaling launch and ONE fused kernel for all 21
    # candidates (weight scale + INT4 block fake quant in shared memory, tcgen05 GEMM, squared-error epilogue)
    bf16_peak = peaks_tflops()

    def fused_entry(x_, w_, ref_, k_):
        s_all = torch.stack([torch.exp(0.05 * i * torch.randn(k_, generator=g, device=dev)) for i in range(21)])
        inv_all, s_all = (1 / s_all).bfloat16(), s_all.bfloat16()
        loss21 = torch.zeros(21, dtype=torch.float64, device=dev)

        def go():
            ops.awq_search_fused(ops.awq_scale_acts(x_, inv_all), w_, s_all, ref_, loss21, status)

        r_ = timed(go, 1, reps=3, groups=3)
        tf_ = flops / (r_["ms"] * 1e-3) / 1e12
        a_all = ops.awq_scale_acts(x_, inv_all)
        rk = timed(lambda: ops.awq_search_fused(a_all, w_, s_all, ref_, loss21, status), 1, reps=3, groups=3)
        tfk = flops / (rk["ms"] * 1e-3) / 1e12
        return {"ms": r_["ms"], "tflops_effective": tf_, "frac_of_measured_bf16_peak": tf_ / bf16_peak,
                "search_kernel_alone_ms": rk["ms"], "search_kernel_alone_tflops": tfk,
                "search_kernel_alone_frac_of_measured_bf16_peak": tfk / bf16_peak,
                "search_kernel_alone_frac_of_sustained_bf16_peak": tfk / peaks_tflops(sustained=True),
                "launches": 2, "kernel_status": int(status),
                "note": "ms / tflops_effective include the activation-scaling kernel; FLOPs are the 21 GEMMs only"}

    out["awq_lite_search_21_alphas_up_proj_512tok_fused_kernel"] = fused_entry(x, w, ref, 4096)
    out["awq_lite_search_21_alphas_down_proj_512tok_fused_kernel"] = fused_entry(xd, wd, refd, 14336)
    del xd, wd, refd
    del ws, wfq, bufs
    out["config4_int4_awq_mlp_through_mtq"] = run_config4(dev)
    # the real-quant GEMM consumers (a 70B-shape projection: 4096 tokens x 8192 -> 8192), beside
    # the library kernels torch._scaled_mm reaches for the same operands
    m_, n_, k_ = 4096, 8192, 8192
    flops = 2.0 * m_ * n_ * k_
    a16 = torch.randn(m_, k_, generator=g, device=dev).bfloat16()
    b16 = (torch.randn(n_, k_, generator=g, device=dev) * 0.02).bfloat16()
    one = torch.ones((), device=dev)

    def tflops(fn):
        r = timed(fn, 1, reps=5, groups=3)
        return {"ms": r["ms"], "tflops": flops / (r["ms"] * 1e-3) / 1e12}

    sa, sb = ops.amax_tensor(a16) / 448.0, ops.amax_tensor(b16) / 448.0
    a8, b8 = ops.fp8_gemm_operand(a16, sa), ops.fp8_gemm_operand(b16, sb)
    out["fp8_gemm_tcgen05_4096x8192x8192"] = tflops(lambda: ops.fp8_gemm(a8, b8, sa, sb))
    out["fp8_gemm_tcgen05_4096x8192x8192"]["with_activation_cast"] = tflops(
        lambda: ops.fp8_gemm(ops.fp8_gemm_operand(a16, sa), b8, sa, sb))
    out["library_scaled_mm_fp8_for_comparison"] = tflops(
        lambda: torch._scaled_mm(a8, b8.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16, use_fast_accum=True))
    a4, sfa, s2a = ops.nvfp4_quantize(a16)
    b4, sfb, s2b = ops.nvfp4_quantize(b16)
    sfa_t, sfb_t, alpha = ops.nvfp4_swizzle_scales(sfa), ops.nvfp4_swizzle_scales(sfb), s2a * s2b
    out["nvfp4_gemm_tcgen05_4096x8192x8192"] = tflops(lambda: ops.nvfp4_gemm(a4, sfa_t, b4, sfb_t, alpha))

    amax_a = ops.amax_tensor(a16)      # a calibrated input quantiser holds it

    def nvfp4_linear():
        q, sf, s2 = ops.nvfp4_quantize(a16, amax=amax_a)
        return ops.nvfp4_gemm(q, ops.nvfp4_swizzle_scales(sf), b4, sfb_t, s2 * s2b)

    out["nvfp4_gemm_tcgen05_4096x8192x8192"]["with_activation_quantise"] = tflops(nvfp4_linear)
    try:
        f4 = torch.float4_e2m1fn_x2
        lib = lambda: torch._scaled_mm(a4.view(f4), b4.view(f4).t(), scale_a=sfa_t.view(torch.float8_e4m3fn),  # noqa: E731
                                       scale_b=sfb_t.view(torch.float8_e4m3fn), out_dtype=torch.bfloat16)
        same = bool(torch.equal(lib(), ops.nvfp4_gemm(a4, sfa_t, b4, sfb_t, one)))
        out["library_scaled_mm_nvfp4_for_comparison"] = dict(tflops(lib), identical_to_ours=same)
    except Exception as e:  # the library path is a comparison only
        out["library_scaled_mm_nvfp4_for_comparison"] = {"unavailable": str(e)[:120]}
    out["bf16_cublas_4096x8192x8192_for_comparison"] = tflops(lambda: torch.nn.functional.linear(a16, b16))
    out["gemm_kernel_status"] = int(ops.qgemm_status(dev).item())
    return out


def peaks_tflops(sustained=False):
    """Measured dense bf16 rate of the library GEMM on this pool's GPUs: the burst figure (a kernel timed
    alone) or the one it sustains for seconds under the power cap."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["bf16_tflops_sustained" if sustained else "bf16_tflops"])
    return 1400.0 if sustained else 1590.0


def run_config4(dev):
    """BASELINE config 4 through the public API: mtq.quantize(INT4_AWQ_CFG, awq_lite, alpha grid 0..1 in
    0.05 steps) on one Llama-style MLP (up 4096 -> 14336, down 14336 -> 4096, bf16 N(0, 0.02)) with 512
    calibration tokens whose channel magnitudes are lognormal(0, 1), then mtq.compress (INT4 packing).
    Wall-clock seconds: the fastest of three runs after one warm-up run, all runs listed."""
    import copy

    import torch

    import b200q as mtq

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up_proj = torch.nn.Linear(4096, 14336, bias=False)
            self.down_proj = torch.nn.Linear(14336, 4096, bias=False)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.up_proj(x)))

    g = torch.Generator(device=dev).manual_seed(4)
    base = MLP().to(device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in base.parameters():
            p.copy_(torch.randn(p.shape, generator=g, device=dev) * 0.02)
    x = (torch.randn(512, 4096, generator=g, device=dev) * torch.exp(torch.randn(4096, generator=g, device=dev))).bfloat16()
    cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
    cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.05, "debug": True}
    secs, totals = {}, []
    for i in range(4):
        model = copy.deepcopy(base)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        mtq.quantize(model, cfg, lambda m: m(x))
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        mtq.compress(model)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        if i and (not totals or t2 - t0 < min(totals)):
            secs = {"quantize_awq_lite_s": t1 - t0, "compress_int4_pack_s": t2 - t1, "total_s": t2 - t0}
        if i:
            totals.append(t2 - t0)
        packed = model.up_proj.weight.dtype == torch.uint8
        alphas = {n: round(float(getattr(model, n).awq_lite.best_alpha), 4) for n in ("up_proj", "down_proj")}
        del model
    return {**secs, "total_s_all_runs": totals, "alphas_evaluated_per_linear": 21, "best_alpha": alphas, "weights_packed": bool(packed),
            "note": "two forward passes (statistics, search), 21 candidates per linear in one fused launch each, "
                    "scale folding, INT4 block-128 packing"}


def run_reference_gpu_kernels(dev, peak):
    """The reference's own GPU kernels (compiled unmodified into oracle/_ref by oracle/build_ref.py) timed
    beside ours on the same tensors: a reported baseline like the CPU one, not a product path."""
    import torch

    from b200q import ops
    from oracle import ref_ext

    ext, ext8, extmx, tri = ref_ext.cuda_ext(), ref_ext.cuda_ext_fp8(), ref_ext.cuda_ext_mx(), ref_ext.triton_fp4()
    if ext is None and tri is None:
        return {"unavailable": "oracle/_ref holds no build of the reference's extensions"}

    def ms(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    g = torch.Generator(device=dev).manual_seed(11)
    xs = [(torch.randn(8192, 4096, generator=g, device=dev)).bfloat16() for _ in range(8)]      # 0.5 GB > L2
    n = 8 * 8192 * 4096
    amax = ops.amax_tensor(xs[0])
    out = {"tensors": "8 x bf16 [8192, 4096] used in turn (larger than L2)"}

    def pair(name, ours, theirs, nbytes):
        if theirs is None:
            return
        try:
            t_ref = ms(theirs)
        except Exception as e:      # a baseline only
            out[name] = {"unavailable": str(e)[:120]}
            return
        t_our = ms(ours)
        out[name] = {"reference_ms": t_ref, "ours_ms": t_our, "speedup": t_ref / t_our,
                     "ours_gbps": nbytes / (t_our * 1e-3) / 1e9, "reference_gbps": nbytes / (t_ref * 1e-3) / 1e9,
                     "ours_frac_of_measured_peak": nbytes / (t_our * 1e-3) / 1e9 / peak}

    packed = [ops.nvfp4_quantize(x, amax=amax) for x in xs]
    if tri is not None:
        pair("nvfp4_dequantize_vs_triton_fp4_dequantize",
             lambda: [ops.nvfp4_dequantize(p, sc, s2, torch.bfloat16) for p, sc, s2 in packed],
             lambda: [tri.fp4_dequantize(p, sc, s2, 16, 128, torch.bfloat16) for p, sc, s2 in packed],
             int(n * (0.5 + 1 / 16 + 2)))
        pair("nvfp4_fake_quant_vs_triton_fp4_fake_quant_block",
             lambda: [ops.nvfp4_fake(x, amax) for x in xs], lambda: [tri.fp4_fake_quant_block(x, amax) for x in xs], n * 4)
    if extmx is not None:
        pair("nvfp4_fake_quant_vs_cuda_fused_amax_convert",
             lambda: [ops.nvfp4_fake(x, amax) for x in xs],
             lambda: [extmx.fused_amax_convert(x, 16, extmx.Types.E2M1, extmx.Types.E4M3, amax) for x in xs], n * 4)
    if ext8 is not None:
        pair("fp8_fake_quant_vs_cuda_fake_e4m3fy",
             lambda: [ops.fake_e4m3(x, amax) for x in xs], lambda: [ext8.fake_e4m3fy(x, amax) for x in xs], n * 4)
    if ext is not None:
        pair("int8_fake_quant_vs_cuda_fake_tensor_quant",
             lambda: [ops.fake_int(x, amax, 8, False, True) for x in xs],
             lambda: [ext.fake_tensor_quant(x, amax, 8, False, True) for x in xs], n * 4)
        flat = [x.view(-1) for x in xs]
        scales = [7 / x.view(-1, 128).abs().amax(-1, keepdim=True) for x in xs]
        pair("int4_block128_amax_and_pack_vs_cuda_INT4_quantize_pack_only",
             lambda: [ops.int4_quantize(f, 128) for f in flat],
             lambda: [ext.INT4_quantize(f, sc, 128) for f, sc in zip(flat, scales)], int(n * (2 + 0.5 + 2 / 128)))
    return out


def cpu_other_configs(seconds_each: float = 3.0):
    """The reference's CPU torch path for the other formats (oracle/torch_path.py), each on a bounded sample
    of its BASELINE configuration, all intra-op threads."""
    import torch

    from oracle import torch_path as tp

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)

    def rate(fn, nbytes, what):
        fn()
        t0 = time.perf_counter()
        fn()
        dt1 = time.perf_counter() - t0
        reps = max(1, min(20, int(seconds_each / max(dt1, 1e-3))))
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        dt = (time.perf_counter() - t0) / reps
        return {"gbps": nbytes / dt / 1e9, "seconds_per_pass": dt, "algorithmic_bytes": nbytes, "sample": what}

    out = {"cores": torch.get_num_threads(), "kind": "port"}
    w = torch.randn(4096, 4096, generator=g) * 0.02
    out["config1_int8_per_row_fake_quant_plus_max_calibration_fp32_4096x4096"] = rate(
        lambda: tp.fake_int(w, tp.max_calibrate_collect(w, None, axis=0), 8, False, True), 4096 * 4096 * 8,
        "the whole configuration (one fp32 [4096, 4096] weight)")
    x = torch.randn(8192, 4096, generator=g)
    x[:, :4] *= 50
    x = x.bfloat16()
    amax = tp.max_calibrate_collect(x, None)
    out["config2_fp8_max_calibration_bf16_8192x4096"] = rate(
        lambda: tp.max_calibrate_collect(x, None), 8192 * 4096 * 2, "one of the 16 batches")
    out["config2_fp8_per_tensor_fake_quant_bf16_8192x4096"] = rate(
        lambda: tp.fp8_eager(x, amax), 8192 * 4096 * 4, "one of the 16 batches")
    hp = tp.HistogramPath(2048)
    hp.collect(x)
    out["config5_histogram_2048_bins_bf16_8192x4096"] = rate(
        lambda: hp.collect(x), 8192 * 4096 * 2, "one [8192, 4096] activation batch (70B shapes have 8192 and 28672 columns)")
    rows = 1792
    w4 = (torch.randn(rows, 4096, generator=g) * 0.02).bfloat16()
    x4 = (torch.randn(512, 4096, generator=g) * torch.exp(torch.randn(4096, generator=g))).bfloat16()
    ref = torch.nn.functional.linear(x4, w4)
    a_s, w_s = x4.abs().float().mean(0), (w4.abs().float() / w4.abs().float().amax(1, keepdim=True)).mean(0)
    t0 = time.perf_counter()
    tp.awq_lite_candidate(w4, x4, ref, a_s, w_s, 0.5)
    t0 = time.perf_counter()
    tp.awq_lite_candidate(w4, x4, ref, a_s, w_s, 0.5)
    dt = time.perf_counter() - t0
    out["config4_awq_lite_one_candidate"] = {
        "seconds_sample": dt, "sample": f"one alpha on {rows} of the 14336 rows of up_proj, 512 tokens",
        "seconds_full_search_extrapolated": dt * (14336 / rows) * 21 * 2,
        "note": "x 8 row slabs x 21 alphas x 2 linears; statistics pass and packing not included"}
    return out



def run_profile_kernels():
    """A few launches of each secondary kernel on small inputs (larger than L2, < 1 GB on the
    device) — the program the committed ncu summaries of these kernels were captured from."""
    import torch

    from b200q import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    m, n, k = 512, 14336, 4096
    a = torch.randn(m, k, generator=g, device=dev).bfloat16()
    w = (torch.randn(n, k, generator=g, device=dev) * 0.02).bfloat16()
    s = torch.exp(torch.randn(k, generator=g, device=dev)).bfloat16()
    ref = torch.nn.functional.linear(a, w)
    acc = torch.zeros((), dtype=torch.float64, device=dev)
    status = torch.zeros((), dtype=torch.int32, device=dev)
    x = torch.randn(2, 8192, 4096, generator=g, device=dev).bfloat16()
    x[:, :, :4] *= 50
    w32 = torch.randn(2, 4096, 4096, generator=g, device=dev) * 0.02
    counts = torch.zeros(2048, dtype=torch.int64, device=dev)
    amax = ops.amax_tensor(x)
    rmax = float(amax)
    counts_open = torch.zeros(2048 * 16, dtype=torch.int64, device=dev)
    overflow = torch.zeros(1, dtype=torch.int64, device=dev)
    xs = a[:64].contiguous()                                    # awq_clip: 64 sampled tokens
    w_amax = w.reshape(n, k // 128, 128).abs().amax(-1).reshape(-1, 1)
    ratios = torch.tensor([0.5 + 0.05 * i for i in range(10)] + [1.0], device=dev)
    clip_loss = torch.zeros(11, n, k // 128, device=dev)
    amax_slot = torch.zeros((), device=dev)
    mse_cands = (amax.reshape(1, 1) * torch.linspace(0.25, 4.0, 10, device=dev).reshape(-1, 1)).contiguous()
    mse_loss = torch.zeros(10, 1, dtype=torch.float64, device=dev)
    mse_cands_rows = (w.abs().amax(dim=1).float().reshape(1, -1) * torch.linspace(0.25, 4.0, 10, device=dev).reshape(-1, 1)).contiguous()
    mse_loss_rows = torch.zeros(10, n, dtype=torch.float64, device=dev)
    for i in range(4):
        wfq = ops.awq_scale_fake_int(w, s, 128, 4, False, False)
        ops.awq_gemm_sqerr(a, wfq, ref, acc, status)
        ops.hist_collect(x[i % 2], counts, 2048, rmax)
        ops.hist_collect_open(x[i % 2], counts_open, 2048, rmax / 4, overflow)
        ops.fake_e4m3(x[i % 2], amax)
        ops.nvfp4_fake(x[i % 2], amax)
        ops.fake_int_rows_dynamic(w32[i % 2], 8, False, True)
        ops.int4_quantize(w.reshape(-1), 128)
        ops.mx_fake(x[i % 2], 32, (4, 3))
        ops.mxfp4_quantize(x[i % 2], 32)
        ops.awq_clip_loss(w, xs, w_amax, ratios, clip_loss, 128, 4, False, False)
        ops.amax_tensor(x[i % 2], out=amax_slot)
        ops.mse_candidates(x[i % 2], mse_cands, mse_loss, None, 8, False, True)
        ops.mse_candidates(w, mse_cands_rows, mse_loss_rows, 0, 8, False, True)
    # real-quant GEMM consumers on a 2048 x 4096 x 4096 problem
    a16, b16 = a.new_empty(2048, k).normal_(generator=g), w[:4096]
    one = torch.ones((), device=dev)
    a8, b8 = ops.fp8_gemm_operand(a16, one), ops.fp8_gemm_operand(b16, one * 0.001)
    a4, sfa, _ = ops.nvfp4_quantize(a16)
    b4, sfb, _ = ops.nvfp4_quantize(b16)
    sfa_t, sfb_t = ops.nvfp4_swizzle_scales(sfa), ops.nvfp4_swizzle_scales(sfb)
    for i in range(3):
        ops.fp8_gemm(a8, b8, one, one)
        ops.nvfp4_gemm(a4, sfa_t, b4, sfb_t, one)
    ops.check_qgemm_status(dev)
    torch.cuda.synchronize()
    print(json.dumps({"profile_kernels": "done", "gemm_status": int(status)}))


def run_profile_awq_fused(n_alpha: int = 2):
    """Three launches of the fused awq_lite search kernel on the BASELINE config-4 up_proj shape with
    ``n_alpha`` candidates (about 0.3 GB on the device) — the program its ncu summary was captured from."""
    import torch

    from b200q import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    m, n, k = 512, 14336, 4096
    x = (torch.randn(m, k, generator=g, device=dev) * torch.exp(torch.randn(k, generator=g, device=dev))).bfloat16()
    w = (torch.randn(n, k, generator=g, device=dev) * 0.02).bfloat16()
    s = torch.exp(0.5 * torch.randn(n_alpha, k, generator=g, device=dev))
    a_all = x.unsqueeze(0) * (1 / s).bfloat16().unsqueeze(1)
    ref = torch.nn.functional.linear(x, w)
    loss = torch.zeros(n_alpha, dtype=torch.float64, device=dev)
    status = torch.zeros((), dtype=torch.int32, device=dev)
    for _ in range(3):
        ops.awq_search_fused(a_all, w, s.bfloat16(), ref, loss, status)
    torch.cuda.synchronize()
    print(json.dumps({"profile_awq_fused": "done", "status": int(status), "loss0": float(loss[0])}))


def run_e2e(args, weights, layers, dev, world, total_elems, barrier):
    """End to end through the public API: ``mtq.compress`` on a Llama-shaped module tree that lives in
    pinned HOST memory (this rank's layers).  Every step builds a fresh tree over the same pinned weight
    buffers and inserts the NVFP4 weight quantisers (outside the timed region: a few hundred small host
    objects), then times compress(): host -> device copies, the two grouped kernels per streamed group,
    device -> host copies of the packed weights and scales, and the swap of the module's parameters."""
    import torch
    import torch.distributed as dist

    import b200q as mtq

    names = [n for n, _ in LAYER_SHAPES]
    shapes = [s for _, s in LAYER_SHAPES]
    try:
        host_in = []
        for li in range(len(layers)):
            host_in.append([torch.empty(s, dtype=torch.bfloat16).pin_memory() for s in shapes])
            for k in range(len(shapes)):
                host_in[li][k].copy_(weights[li * len(shapes) + k])
    except RuntimeError as e:  # pinned allocation refused
        return {"value": None, "unit": "GB/s", "error": str(e)[:200]}
    torch.cuda.synchronize()
    wcfg = {"*weight_quantizer": {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)},
                                  "axis": None, "enable": True},
            "*input_quantizer": {"enable": False}, "default": {"enable": False}}

    def build_tree():
        tree = torch.nn.ModuleList()
        for li in range(len(layers)):
            layer = torch.nn.ModuleDict()
            for k, (n, (rows, cols)) in enumerate(LAYER_SHAPES):
                lin = torch.nn.Linear(1, 1, bias=False)
                lin.in_features, lin.out_features = cols, rows
                lin.weight = torch.nn.Parameter(host_in[li][k], requires_grad=False)   # aliases the pinned buffer
                layer[n] = lin
            tree.append(layer)
        model = torch.nn.ModuleDict({"layers": tree})
        mtq.replace_quant_module(model)
        mtq.set_quantizer_by_cfg(model, wcfg)
        return model

    steps = max(1, min(args.steps, args.e2e_steps))
    times = []
    out_bytes = 0
    for i in range(steps + 1):          # the first pass warms the pinned-memory pool and the streams
        model = build_tree()
        barrier()
        t0 = time.perf_counter()
        mtq.compress(model)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if i:
            times.append(dt)
        if layers:
            lin = model["layers"][0][names[0]]
            assert lin.weight.dtype == torch.uint8 and lin.weight.device.type == "cpu"
        out_bytes = sum(m.weight.numel() + m.weight_quantizer._scale.numel() + 4
                        for m in model.modules() if hasattr(m, "weight_quantizer"))
        del model
    dt = statistics.mean(times)
    if world > 1:
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = t.item()
    h2d = sum(w.numel() * 2 for w in weights)
    # the same bytes over the same links with no kernel between them: what the host side allows
    copy_only = None
    if layers:
        dbuf = [torch.empty_like(weights[k]) for k in range(len(shapes))]
        obuf = [torch.empty(int(w.numel() * (0.5 + 1 / 16)), dtype=torch.uint8, device=dev) for w in dbuf]
        hout = [torch.empty(o.numel(), dtype=torch.uint8).pin_memory() for o in obuf]
        up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        barrier()
        t0 = time.perf_counter()
        for li in range(len(layers)):
            with torch.cuda.stream(up):
                for k in range(len(shapes)):
                    dbuf[k].copy_(host_in[li][k], non_blocking=True)
            with torch.cuda.stream(down):
                for k in range(len(shapes)):
                    hout[k].copy_(obuf[k], non_blocking=True)
        torch.cuda.synchronize()
        ct = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([ct], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ct = t.item()
        copy_only = {"seconds": ct, "h2d_gbps_per_rank": h2d / ct / 1e9,
                     "note": "this rank's weights host->device and the packed bytes device->host on two streams, "
                             "no kernels: the ceiling the host memory and PCIe paths set for e2e at this N"}
    return {"value": total_elems * BYTES_TOTAL / dt / 1e9, "unit": "GB/s", "seconds_per_step": dt,
            "steps": steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": out_bytes,
            "api": "mtq.compress(model) on a host-resident (pinned) Llama-shaped module tree with NVFP4 weight "
                   "quantisers: weights streamed through the GPU, packed weights and scales back on the host",
            "copy_only": copy_only}


# ---------------------------------------------------------------- 70B-shape calibration --------
L70 = {"hidden": 8192, "kv": 1024, "inter": 28672, "layers": 80}


def model_flow_70b(dev, world, rank, n_layers, sequences_per_rank, seq_len=1024, micro_batch=8):
    """The calibration of BASELINE config 5 as a user runs it, on a reduced depth: a random-init decoder of
    Llama-3-70B layer shapes (hidden 8192, 64 query / 8 key-value heads of 128, intermediate 28672, bf16;
    embedding over the 128256-token vocabulary, ``n_layers`` layers, final norm; plain torch modules whose
    names end in q_proj .. down_proj), seeded random token IDs batch-sharded over the ranks, NVFP4 quantisers
    on every linear with 2048-bin histogram calibrators on the inputs, ``mtq.histogram_calibrate`` with the
    percentile-99.99 read-out.  The forward GEMMs and attention are torch's (not part of the hand-written
    path); reported are the calibration's wall time, the same forward passes without any quantiser, and
    whether every rank ended with identical amax values."""
    import copy

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch import nn

    import b200q as mtq

    H, HEADS, KVH, HD, I, VOCAB = 8192, 64, 8, 128, 28672, 128256

    class RMSNorm(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.ones(H))

        def forward(self, x):
            v = x.float()
            return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * self.weight

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(H, HEADS * HD, bias=False)
            self.k_proj = nn.Linear(H, KVH * HD, bias=False)
            self.v_proj = nn.Linear(H, KVH * HD, bias=False)
            self.o_proj = nn.Linear(HEADS * HD, H, bias=False)

        def forward(self, x):
            b, s, _ = x.shape
            q = self.q_proj(x).view(b, s, HEADS, HD).transpose(1, 2)
            k = self.k_proj(x).view(b, s, KVH, HD).transpose(1, 2)
            v = self.v_proj(x).view(b, s, KVH, HD).transpose(1, 2)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            return self.o_proj(o.transpose(1, 2).reshape(b, s, HEADS * HD))

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = nn.Linear(H, I, bias=False)
            self.up_proj = nn.Linear(H, I, bias=False)
            self.down_proj = nn.Linear(I, H, bias=False)

        def forward(self, x):
            return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.input_layernorm, self.self_attn = RMSNorm(), Attention()
            self.post_attention_layernorm, self.mlp = RMSNorm(), MLP()

        def forward(self, x):
            x = x + self.self_attn(self.input_layernorm(x))
            return x + self.mlp(self.post_attention_layernorm(x))

    class Decoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(VOCAB, H)
            self.layers = nn.ModuleList(Layer() for _ in range(n_layers))
            self.norm = RMSNorm()

        def forward(self, ids):
            x = self.embed_tokens(ids)
            for layer in self.layers:
                x = layer(x)
            return self.norm(x)

    torch.manual_seed(1234)                                # the same replica on every rank
    with torch.device(dev):
        model = Decoder().to(torch.bfloat16)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.02)
    model.eval()
    g = torch.Generator(device=dev).manual_seed(0)
    ids_all = torch.randint(0, VOCAB, (world * sequences_per_rank, seq_len), generator=g, device=dev)
    mine = ids_all[rank * sequences_per_rank:(rank + 1) * sequences_per_rank]
    batches = list(mine.split(micro_batch))

    def forward_loop(m):
        with torch.no_grad():
            for ids in batches:
                m(ids)

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = t.item()
        return dt

    forward_loop(model)                                    # warm-up: GEMM plans, allocator
    t_forward = timed(lambda: forward_loop(model))
    cfg = copy.deepcopy(mtq.NVFP4_DEFAULT_CFG)
    cfg["quant_cfg"]["*input_quantizer"]["calibrator"] = "histogram"
    mtq.replace_quant_module(model)
    mtq.set_quantizer_by_cfg(model, cfg["quant_cfg"])
    first = batches[:1]
    t_calib = timed(lambda: mtq.histogram_calibrate(
        model, forward_loop, method="percentile", percentile=99.99,
        first_batch_loop=lambda m: [m(ids) for ids in first]))
    qs = [(n, m) for n, m in model.named_modules() if isinstance(m, mtq.nn.TensorQuantizer) and m.amax is not None]
    amaxes = torch.cat([m.amax.float().reshape(-1) for _, m in qs])
    same = True
    if world > 1:
        lo, hi = amaxes.clone(), amaxes.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(torch.equal(lo, hi))
    with torch.no_grad():
        out = model(batches[0])                            # the calibrated, fake-quantised model runs
    inputs_q = [m for n, m in qs if n.endswith("input_quantizer")]
    return {
        "model": "llama3-70b layer shapes, %d layers, random init, bf16; token IDs randint(0, 128256), seed 0" % n_layers,
        "sequences_per_rank": sequences_per_rank, "seq_len": seq_len, "micro_batch_sequences": micro_batch,
        "tokens_per_rank": sequences_per_rank * seq_len, "quantizers_with_amax": len(qs),
        "histogram_input_quantizers": len(inputs_q),
        "seconds": {"forward_only": t_forward, "histogram_calibrate": t_calib,
                    "note": "histogram_calibrate = range pass over the first micro-batch + the forward passes with "
                            "collection + exchanges + read-out; forward_only = the same forward passes before "
                            "conversion"},
        "input_amax_range": [float(min(m.amax.float().min() for m in inputs_q)),
                             float(max(m.amax.float().max() for m in inputs_q))],
        "amax_identical_on_all_ranks": same, "output_finite": bool(torch.isfinite(out.float()).all()),
    }


def run_calib70b(args):
    """Data-parallel NVFP4 activation calibration on Llama-3-70B shapes (``calibration_phases``: 560 input
    quantisers, max and 2048-bin histogram calibration), then the NVFP4 weight quantisation of this rank's
    layers.  Activation work per rank is fixed (weak scaling in the batch dimension), weight work is split
    by layer."""
    import torch
    import torch.distributed as dist

    from b200q.ops import NvFp4Group

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the kernels)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_layers = args.layers if args.layers != N_LAYERS else L70["layers"]
    H, KV, I = L70["hidden"], L70["kv"], L70["inter"]
    sampler = ClockSampler(local)
    sampler.start()
    t_wall0 = time.perf_counter()
    calibration = calibration_phases(dev, world, rank, L70, n_layers, args.tokens, args.batches)

    # weights of one layer, reused for every layer of this rank's share
    shapes = [(H, H), (KV, H), (KV, H), (H, H), (I, H), (I, H), (H, I)]
    my_layers = split_layers(n_layers, world, rank)
    weights = [make_weight(sh, 7000 + k, dev) for k, sh in enumerate(shapes)]
    group = NvFp4Group(weights)
    group.run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in my_layers:
        group.run()
    torch.cuda.synchronize()
    t_weights = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([t_weights], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_weights = t.item()
    clocks = sampler.stop(t_wall0, time.perf_counter())
    model_flow = None
    if args.model_layers > 0:
        del group, weights
        torch.cuda.empty_cache()
        model_flow = model_flow_70b(dev, world, rank, args.model_layers, args.model_sequences)
    if rank == 0:
        w_elems = n_layers * sum(a * b for a, b in shapes)
        total = calibration["histogram"]["total_s"] + t_weights
        print(json.dumps({
            "metric": "nvfp4_calibration_70b_shape_seconds", "value": total, "unit": "s", "n_gpus": world,
            "higher_is_better": False, "scaling": "weak (activation batches per rank fixed); weights split by layer",
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3-70b-shape NVFP4 calibration: 2048-bin histogram of every linear input, "
                                   "percentile 99.99 amax, then NVFP4 weight quantisation",
                       "layers": n_layers, "tokens_per_batch": args.tokens, "batches_per_rank_per_layer": args.batches,
                       "full_size_note": "the named configuration is 4096x1024 tokens over 8 GPUs = 64 batches of "
                                         "8192 tokens per rank per layer"},
            "calibration": calibration, "weights_seconds": t_weights,
            "weights_gbps_all_ranks": w_elems * BYTES_TOTAL / t_weights / 1e9, "clocks": clocks,
            "model_flow": model_flow,
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-formats", action="store_true")
    ap.add_argument("--no-calibration", action="store_true")
    ap.add_argument("--workload", default="ptq8b", choices=["ptq8b", "calib70b"],
                    help="ptq8b: NVFP4 weight quantisation on 8B shapes (the headline line); "
                         "calib70b: data-parallel histogram calibration on 70B shapes")
    ap.add_argument("--tokens", type=int, default=8192, help="calibration: tokens per batch (per rank)")
    ap.add_argument("--batches", type=int, default=2, help="calibration: batches per rank per layer")
    ap.add_argument("--model-layers", type=int, default=2,
                    help="calib70b: depth of the 70B-shape decoder that is calibrated through mtq.histogram_calibrate "
                         "on token IDs (0 = skip)")
    ap.add_argument("--model-sequences", type=int, default=32,
                    help="calib70b: sequences of 1024 tokens per rank for that model (the named configuration has 512)")
    ap.add_argument("--profile-kernels", action="store_true",
                    help="run a few launches of the secondary kernels and exit (for ncu captures)")
    ap.add_argument("--profile-awq-fused", type=int, default=0, metavar="N_ALPHA",
                    help="run three launches of the fused awq_lite search kernel with N_ALPHA candidates and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.profile_awq_fused:
        run_profile_awq_fused(args.profile_awq_fused)
    elif args.profile_kernels:
        run_profile_kernels()
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "calib70b":
        run_calib70b(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
