"""Host-side logic that needs no GPU: configuration matching, module conversion, state-dict
names, quantiser bookkeeping and the batched data-parallel exchanges over gloo (2 CPU ranks)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

import b200q as mtq
from b200q.calib import HistogramCalibrator
from b200q.nn import QuantLinear, SequentialQuantizer, TensorQuantizer


class MLP(nn.Module):
    def __init__(self, hidden=32, inter=64):
        super().__init__()
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)
        self.lm_head = nn.Linear(hidden, 10, bias=False)

    def forward(self, x):
        return self.lm_head(self.down_proj(torch.relu(self.up_proj(x))))


def test_convert_and_configure_by_wildcards():
    m = MLP()
    keys_before = list(m.state_dict().keys())
    mtq.replace_quant_module(m)
    assert isinstance(m.up_proj, QuantLinear) and isinstance(m.lm_head, QuantLinear)
    assert list(m.state_dict().keys()) == keys_before  # no buffers until calibrated
    mtq.set_quantizer_by_cfg(m, mtq.NVFP4_DEFAULT_CFG["quant_cfg"])
    q = m.up_proj.weight_quantizer
    assert q.is_enabled and q.num_bits == (2, 1) and q.block_sizes[-1] == 16
    assert q.block_sizes["scale_bits"] == (4, 3) and q.maxbound == 6.0
    assert m.up_proj.input_quantizer.is_enabled
    assert not m.up_proj.output_quantizer.is_enabled          # "default": disabled
    assert not m.lm_head.weight_quantizer.is_enabled          # "*lm_head*": disabled
    assert not m.lm_head.input_quantizer.is_enabled


def test_int4_awq_config_and_sequential():
    m = MLP()
    mtq.replace_quant_module(m)
    mtq.set_quantizer_by_cfg(m, mtq.INT4_AWQ_CFG["quant_cfg"])
    q = m.down_proj.weight_quantizer
    assert q.num_bits == 4 and q.block_sizes == {-1: 128, "type": "static"} and q.is_static_block_quant
    assert not m.down_proj.input_quantizer.is_enabled
    assert q.maxbound == 7 and not q.narrow_range
    # a list of attribute dicts makes a SequentialQuantizer
    mtq.set_quantizer_attribute(m, "*up_proj.weight_quantizer",
                                [{"num_bits": 4, "block_sizes": {-1: 128}}, {"num_bits": (4, 3)}])
    assert isinstance(m.up_proj.weight_quantizer, SequentialQuantizer) and len(m.up_proj.weight_quantizer) == 2
    with SequentialQuantizer.convert_to_single_quantizer(m):
        assert isinstance(m.up_proj.weight_quantizer, TensorQuantizer)
    assert isinstance(m.up_proj.weight_quantizer, SequentialQuantizer)


def test_enable_disable_keeps_attributes():
    m = MLP()
    mtq.replace_quant_module(m)
    mtq.set_quantizer_by_cfg(m, mtq.INT8_DEFAULT_CFG["quant_cfg"])
    mtq.disable_quantizer(m, "*up_proj*")
    assert not m.up_proj.weight_quantizer.is_enabled and m.up_proj.weight_quantizer.axis == 0
    mtq.enable_quantizer(m, "*up_proj.weight_quantizer")
    assert m.up_proj.weight_quantizer.is_enabled and not m.up_proj.input_quantizer.is_enabled


def test_quantizer_attribute_validation_and_amax_rules():
    with pytest.raises(ValueError):
        mtq.QuantizerAttributeConfig(num_bits=0)
    with pytest.raises(ValueError):
        mtq.QuantizerAttributeConfig(axis=0, block_sizes={-1: 16})
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, axis=0))
    q.amax = torch.ones(4, 1)
    with pytest.raises(RuntimeError):
        q.amax = torch.ones(5, 1)          # shape change is refused, as in the reference
    assert "_amax" in q.state_dict()
    q.reset_amax()
    assert q.amax is None
    with pytest.raises(ValueError):         # negative amax is rejected where it is produced
        q.validate_attr(attr_value=torch.tensor([-1.0]), raise_error=True)
    e = q.export_amax()
    assert e is None


def test_export_amax_shapes():
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8))
    q.amax = torch.tensor(0.0)
    assert q.export_amax().shape == (1,) and q.export_amax().item() == 127   # 0 -> maxbound
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, axis=0))
    q.amax = torch.rand(6, 1) + 0.1
    assert q.export_amax().shape == (6,)


def test_kernels_refuse_cpu_tensors():
    from b200q import ops

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.amax_tensor(torch.randn(64))
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8))
    q.amax = torch.tensor(1.0)
    with pytest.raises(RuntimeError, match="CUDA"):
        q(torch.randn(4, 16))


def test_awq_scale_formula_matches_reference_definition():
    from b200q.model_calib import get_scale

    a = torch.tensor([1.0, 4.0, 0.25, 9.0])
    w = torch.tensor([0.5, 0.5, 1.0, 0.1])
    s = get_scale(a, w, 0.5)
    raw = (a.pow(0.5) / (w.pow(0.5) + torch.finfo(torch.float32).tiny)).clamp(1e-4, 1e4)
    assert torch.allclose(s, raw / (raw.max() * raw.min()).sqrt())
    assert torch.allclose(s.max() * s.min(), torch.tensor(1.0))


# ------------------------------------------------------------------------------- gloo ranks ----

def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(fn, world=2):
    port = _free_port()
    mp.spawn(_entry, args=(world, port, fn), nprocs=world, join=True)


def _entry(rank, world, port, fn):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world)
    finally:
        dist.destroy_process_group()


def _amax_job(rank, world):
    torch.manual_seed(0)
    m = MLP()
    mtq.replace_quant_module(m)
    mtq.set_quantizer_by_cfg(m, mtq.INT8_DEFAULT_CFG["quant_cfg"])
    g = torch.Generator().manual_seed(100 + rank)      # different data per data-parallel rank
    local = {}
    for name, q in m.named_modules():
        if isinstance(q, TensorQuantizer) and q.is_enabled:
            shape = (64, 1) if name == "up_proj.weight_quantizer" else (32, 1) if "weight" in name else ()
            q.amax = torch.rand(shape, generator=g) + rank
            local[name] = q.amax.clone()
    n = mtq.dist.sync_amax(m)
    assert n == 1, "all amaxes must travel in one collective"
    for name, q in m.named_modules():
        if name in local:
            gathered = [torch.zeros_like(local[name]) for _ in range(world)]
            dist.all_gather(gathered, local[name])
            assert torch.equal(q.amax, torch.stack(gathered).amax(0)), name
    # a second sync changes nothing (MAX is idempotent) — the reference's own DP invariant
    before = {n_: q.amax.clone() for n_, q in m.named_modules() if n_ in local}
    mtq.dist.sync_amax(m)
    assert all(torch.equal(before[n_], q.amax) for n_, q in m.named_modules() if n_ in local)


def test_sync_amax_two_gloo_ranks():
    _spawn(_amax_job)


def _hist_job(rank, world):
    m = MLP()
    mtq.replace_quant_module(m)
    cfg = {"*input_quantizer": {"num_bits": 8, "axis": None, "calibrator": "histogram"},
           "*weight_quantizer": {"enable": False}, "default": {"enable": False}}
    mtq.set_quantizer_by_cfg(m, cfg)
    cals = [(n, q._calibrator) for n, q in m.named_modules()
            if isinstance(q, TensorQuantizer) and q.is_enabled]
    assert len(cals) == 3 and all(isinstance(c, HistogramCalibrator) for _, c in cals)
    # rank 0's first-batch maxima define the common bin width
    first_max = {n: 1.0 + i + 10.0 * rank for i, (n, _) in enumerate(cals)}
    mtq.dist.agree_histogram_ranges(m, first_max, torch.device("cpu"))
    rng = np.random.default_rng(5 + rank)
    mine = []
    for i, (n, c) in enumerate(cals):
        assert abs(float(c._calib_bin_edges[-1]) - (1.0 + i)) < 1e-6     # rank 0's value everywhere
        nb = 2048 + (300 * rank if i == 1 else 0)                          # rank 1 grew one histogram
        h = torch.from_numpy(rng.integers(0, 1000, nb))
        c._load_counts(h.clone())
        mine.append(h)
    assert mtq.dist.sync_histograms(m) == 2
    for i, (n, c) in enumerate(cals):
        nb = 2048 + (300 if i == 1 else 0)
        assert c._num_bins == nb and c.hist.numel() == nb and c._calib_bin_edges.numel() == nb + 1
        pad = torch.zeros(nb, dtype=torch.int64)
        pad[: mine[i].numel()] = mine[i]
        gathered = [torch.zeros_like(pad) for _ in range(world)]
        dist.all_gather(gathered, pad)
        assert torch.equal(c.hist, sum(gathered)), n


def test_sync_histograms_two_gloo_ranks():
    _spawn(_hist_job)


def _arena_job(rank, world):
    """Arena calibrators: ranges broadcast in place, counters summed in place (no packing), one
    collective each; the result is the element-wise sum of what the ranks held."""
    from b200q.calib import attach_histogram_arena

    m = MLP()
    mtq.replace_quant_module(m)
    cfg = {"*input_quantizer": {"num_bits": 8, "axis": None, "calibrator": "histogram"},
           "*weight_quantizer": {"enable": False}, "default": {"enable": False}}
    mtq.set_quantizer_by_cfg(m, cfg)
    (arena,) = attach_histogram_arena(m)
    assert len(arena.cals) == 3
    arena._allocate(torch.device("cpu"))
    rng = np.random.default_rng(9 + rank)
    arena.ranges.copy_(torch.tensor([1.0, 2.0, 3.0]) + 10.0 * rank)
    for c in arena.cals:
        c._ranged = True
    mtq.dist.agree_histogram_ranges(m)
    assert torch.equal(arena.ranges, torch.tensor([1.0, 2.0, 3.0]))        # rank 0's everywhere
    live = 2048 + 500 * rank                                                 # rank 1 reached further bins
    mine = torch.zeros_like(arena.counts)
    mine[:, :live] = torch.from_numpy(rng.integers(0, 1000, (3, live)))
    arena.counts.copy_(mine)
    ptr = arena.counts.data_ptr()
    assert mtq.dist.sync_histograms(m) == 2
    assert arena.counts.data_ptr() == ptr                                    # reduced where it was
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    assert torch.equal(arena.counts, sum(gathered))
    arena.resolve()
    for i, c in enumerate(arena.cals):
        assert c._num_bins == 2048 + 500 and c.hist.numel() == 2548
        assert abs(float(c._calib_bin_edges[2048]) - (1.0 + i)) < 1e-6


def test_sync_histogram_arena_two_gloo_ranks():
    _spawn(_arena_job)


def _awq_stats_job(rank, world):
    """awq_lite's exchange between its passes: act_scale becomes the mean over the ranks, and a layer
    with a NaN on ANY rank is flagged on ALL ranks and left alone; one collective for all layers."""
    a = [torch.full((8,), 1.0 + rank), torch.full((4,), 10.0 * (rank + 1)), torch.arange(6, dtype=torch.float32) + rank]
    if rank == 1:
        a[1][2] = float("nan")
    before = [t.clone() for t in a]
    nan = [bool(torch.isnan(t).any()) for t in a]
    flags = mtq.dist.sync_awq_statistics(a, nan)
    assert flags == [False, True, False]
    assert torch.equal(a[0], torch.full((8,), 1.5))
    assert torch.equal(a[2], torch.arange(6, dtype=torch.float32) + 0.5)
    assert torch.equal(torch.nan_to_num(a[1]), torch.nan_to_num(before[1]))   # the flagged layer keeps its own


def test_awq_statistics_exchange_two_gloo_ranks():
    _spawn(_awq_stats_job)


def _failing_rank_job(rank, world):
    """A rank that never joins the exchange: the others get an error from the collective's
    timeout instead of hanging (host-side failure, no GPU involved)."""
    import datetime

    pg = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=2))
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8))
    q.amax = torch.tensor(float(rank + 1))
    if rank == 1:
        return                              # leaves between steps, nothing in flight
    with pytest.raises(RuntimeError):
        mtq.dist.flat_all_reduce([q._amax], dist.ReduceOp.MAX, group=pg)


def test_missing_rank_surfaces_as_error():
    _spawn(_failing_rank_job)


def test_export_format_detection_and_state_dict_postprocess():
    """Host-only parts of the checkpoint export: format names from quantiser attributes, state-dict
    key filtering and renaming (no kernels involved)."""
    from b200q import export
    from b200q.nn import QuantLinear, SequentialQuantizer

    def lin(wcfg, icfg):
        m = torch.nn.Sequential(torch.nn.Linear(32, 16, bias=False))
        mtq.replace_quant_module(m)
        mtq.set_quantizer_by_cfg(m, {"*weight_quantizer": wcfg, "*input_quantizer": icfg, "default": {"enable": False}})
        assert isinstance(m[0], QuantLinear)
        return m[0]

    nv = {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, "enable": True}
    cases = [
        ({"num_bits": (4, 3), "axis": None}, {"num_bits": (4, 3), "axis": None}, "fp8"),
        ({"num_bits": (4, 3), "axis": 0}, {"enable": False}, "fp8_pc_pt"),
        ({"num_bits": (4, 3), "block_sizes": {-1: 128, -2: 128}}, {"enable": False}, "fp8_pb_wo"),
        ({"num_bits": 8, "axis": 0}, {"num_bits": 8, "axis": None}, "int8_sq"),
        ({"num_bits": 8, "axis": 0}, {"enable": False}, "int8_wo"),
        ({"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}}, {"enable": False}, "int4_awq"),
        (nv, nv, "nvfp4"),
        ({"enable": False}, {"enable": False}, None),
    ]
    for wcfg, icfg, want in cases:
        m = lin(wcfg, icfg)
        assert export.get_quantization_format(m) == want, (wcfg, want)
    m = lin({"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}}, {"enable": False})
    assert export.get_weight_block_size(m) == 128
    m = lin(nv, nv)
    m.input_quantizer.register_buffer("_pre_quant_scale", torch.ones(32))
    assert export.get_quantization_format(m) == "nvfp4_awq"
    w4a8 = lin([{"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                {"num_bits": (4, 3), "axis": None, "enable": True}], {"num_bits": (4, 3), "axis": None})
    assert isinstance(w4a8.weight_quantizer, SequentialQuantizer)
    assert export.get_quantization_format(w4a8) == "w4a8_awq" and export.get_weight_block_size(w4a8) == 128

    t = torch.arange(4.0)
    sd = {"a.weight": t.clone(), "a.weight_scale": torch.ones(1, 2, 3), "a.input_quantizer._amax": t.clone(),
          "a.input_quantizer._pre_quant_scale": t.clone() + 1, "a.weight_quantizer._amax": t.clone(),
          "a.weight_quantizer._scale": t.clone(), "a.output_quantizer._amax": t.clone(), "b.weight": t.clone() + 2}
    sd["b.tied"] = sd["b.weight"]
    out = export.postprocess_state_dict(sd)
    assert sorted(out) == ["a.pre_quant_scale", "a.weight", "a.weight_scale", "b.weight"]
    assert out["a.weight_scale"].shape == (2, 3) and torch.equal(out["a.pre_quant_scale"], t + 1)


def test_every_config_converts_a_model_on_cpu():
    """Conversion (module replacement and quantiser attributes) is host logic: every named
    configuration applies to a small model without a GPU."""
    for name in sorted(mtq.config.choices):
        m = MLP()
        mtq.replace_quant_module(m)
        cfg = getattr(mtq, name)
        mtq.set_quantizer_by_cfg(m, cfg["quant_cfg"])
        qs = [q for _, q in m.named_modules() if isinstance(q, TensorQuantizer)]
        assert qs, name
        algo = cfg["algorithm"]
        assert algo is None or isinstance(algo, (str, dict)), name


def test_bias_calibrator_matches_reference_values():
    """Running-mean and running-mid-range bias over two batches against the reference's values
    (tests/golden/bias.npz); the calibrator is plain tensor arithmetic, so this runs on CPU."""
    from b200q.calib import BiasCalibrator

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "bias.npz"))
    xs = [torch.from_numpy(g["x0"]), torch.from_numpy(g["x1"])]
    mean = BiasCalibrator("mean", (-2, -4))
    mid = BiasCalibrator("max_min", (-1,))
    for x in xs:
        mean.collect(x)
        mid.collect(x)
    assert mean.compute_bias().shape == (1, 3, 1, 16) and mid.compute_bias().shape == (2, 3, 8, 1)
    assert torch.allclose(mean.compute_bias(), torch.from_numpy(g["fp8_mean_bias"]), rtol=1e-6, atol=1e-7)
    assert torch.equal(mid.compute_bias(), torch.from_numpy(g["int8_maxmin_bias"]))
    assert torch.equal(mid.compute_dynamic_bias(xs[0]), (xs[0].amax(-1, keepdim=True) + xs[0].amin(-1, keepdim=True)) / 2)
    mean.reset()
    assert mean.compute_bias() is None
    with pytest.raises(ValueError):
        BiasCalibrator("median")


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "W4A8_AWQ_BETA_CFG", "INT8_DEFAULT_CFG"])
def test_modelopt_state_restores_structure_on_cpu(name):
    """Checkpoint / resume without compute: the recorded modes, the quantiser properties and the
    buffer shapes are enough for ``load_state_dict(strict=True)`` on a fresh model."""
    import copy
    import io

    torch.manual_seed(0)
    m = MLP()
    from b200q.conversion import convert_to_quantized_model
    from b200q.model_quant import _record_mode
    cfg = copy.deepcopy(getattr(mtq, name))
    convert_to_quantized_model(m, cfg)
    _record_mode(m, "quantize", cfg)
    # stand-in for calibration: amax buffers of the shapes calibration would leave
    for n, q in m.named_modules():
        if isinstance(q, TensorQuantizer) and q.is_enabled \
                and not (q.block_sizes and q.block_sizes.get("type") == "dynamic"):
            q.amax = torch.rand(()) + 0.5
    m.up_proj.input_quantizer.pre_quant_scale = torch.rand(32) + 0.5
    buf = io.BytesIO()
    torch.save({"model": m.state_dict(), "modelopt": mtq.modelopt_state(m)}, buf)
    buf.seek(0)
    ckpt = torch.load(buf, weights_only=False)

    fresh = MLP()
    mtq.restore_from_modelopt_state(fresh, ckpt["modelopt"])
    fresh.load_state_dict(ckpt["model"], strict=True)
    for (na, a), (nb, b) in zip(m.named_modules(), fresh.named_modules()):
        assert na == nb and type(a) is type(b)
        if isinstance(a, TensorQuantizer):
            assert a.get_modelopt_state() == b.get_modelopt_state(), na
    assert torch.equal(fresh.up_proj.input_quantizer.pre_quant_scale, m.up_proj.input_quantizer.pre_quant_scale)
    with pytest.raises(KeyError):
        bad = dict(ckpt["modelopt"], quantizer_state={"no.such.quantizer": {}})
        mtq.restore_from_modelopt_state(MLP(), bad)


def test_gemm_registry_and_real_quant_switches_on_cpu():
    """Host logic of the GEMM back ends: registration order, enable / disable marks, and the
    availability checks refusing what they cannot run (CPU tensors, other formats)."""
    from b200q import backends
    from b200q.backends.gemm_registry import GEMMRegistry
    from b200q.backends.fp8_per_tensor_gemm import _fp8_availability_check
    from b200q.backends.nvfp4_gemm import _nvfp4_availability_check

    assert backends.Fp8PerTensorLinear.apply in backends.gemm_registry
    assert backends.Nvfp4Linear.apply in backends.gemm_registry
    reg = GEMMRegistry()
    f = lambda *a, **k: "f"  # noqa: E731
    g = lambda *a, **k: "g"  # noqa: E731
    reg.register(f, lambda module, input, args, kwargs: input.shape[-1] == 8)
    reg.register(g)                                        # no predicate: always available
    assert reg.find_match(None, torch.zeros(2, 8)) is f and reg.find_match(None, torch.zeros(2, 4)) is g
    reg.unregister(f)
    assert f not in reg and reg.find_match(None, torch.zeros(2, 8)) is g

    m = MLP()
    mtq.replace_quant_module(m)
    mtq.set_quantizer_by_cfg(m, mtq.FP8_DEFAULT_CFG["quant_cfg"])
    assert not backends.is_real_quant_gemm_enabled(m)
    backends.enable_real_quant_gemm(m)
    assert m.up_proj._use_real_quant_gemm and not hasattr(m.lm_head, "_use_real_quant_gemm")   # lm_head quantisers are off
    assert backends.is_real_quant_gemm_enabled(m)
    backends.disable_real_quant_gemm(m)
    assert not backends.is_real_quant_gemm_enabled(m)
    x = torch.zeros(4, 32)
    assert not _fp8_availability_check(m.up_proj, x, (), {})       # CPU input, not a RealQuantLinear
    assert not _nvfp4_availability_check(m.up_proj, x, (), {})
    # a QuantLinear ignores the mark: its forward is the fake-quant path (disabled here -> plain linear)
    mtq.disable_quantizer(m, "*")
    backends.enable_real_quant_gemm(m)
    assert torch.equal(m.up_proj(x), torch.nn.functional.linear(x, m.up_proj.weight))


def test_host_packer_group_plan():
    """Groups for the host-to-host NVFP4 packer: whole layers of a repeated stack (one signature, so one
    pipeline that never drains), a large layer cut at the same places every time, shape buckets for
    anything irregular; every tensor in exactly one group."""
    import torch

    from b200q.pipeline import _plan_groups, _repeating_unit

    bf = torch.bfloat16
    layer = [((4096, 4096), bf), ((1024, 4096), bf), ((1024, 4096), bf), ((4096, 4096), bf),
             ((14336, 4096), bf), ((14336, 4096), bf), ((4096, 14336), bf)]
    keys = layer * 32
    sizes = [a * b * 2 for (a, b), _ in keys]
    assert _repeating_unit(keys) == 7
    groups = _plan_groups(keys, sizes, 512 << 20)
    assert groups == [list(range(i, i + 7)) for i in range(0, 224, 7)]
    assert len({tuple(keys[i] for i in g) for g in groups}) == 1
    cut = _plan_groups(keys, sizes, 200 << 20)               # a layer is 436 MB: cut into three pieces
    assert len(cut) == 96 and len({tuple(keys[i] for i in g) for g in cut}) == 3
    assert all(sum(sizes[i] for i in g) <= 200 << 20 for g in cut)
    irregular = keys + [((128256, 4096), bf)]
    flat = sorted(i for g in _plan_groups(irregular, sizes + [128256 * 4096 * 2], 512 << 20) for i in g)
    assert flat == list(range(225))
    small = _plan_groups(layer[:2] * 3, [1, 1] * 3, 512 << 20)
    assert small == [[0, 1, 2, 3, 4, 5]]


def test_register_a_custom_quantized_module():
    """Reference tests/unit/torch/quantization/test_module_registry.py: a user class replaces every module
    of exactly the registered type, its quantisers answer to the wildcard configuration, and it can be
    unregistered again."""
    from b200q.nn import TensorQuantizer

    class QuantReLU(nn.ReLU):
        def _setup(self):
            self.input_quantizer = TensorQuantizer(mtq.QuantizerAttributeConfig())
            self.output_quantizer = TensorQuantizer(mtq.QuantizerAttributeConfig(enable=False))

        def forward(self, x):
            return self.output_quantizer(super().forward(self.input_quantizer(x)))

    model = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.LeakyReLU())
    mtq.register(original_cls=nn.ReLU, quantized_cls=QuantReLU)
    try:
        assert mtq.QuantModuleRegistry.get(nn.ReLU) is QuantReLU and nn.ReLU in mtq.QuantModuleRegistry
        mtq.replace_quant_module(model)
        assert sum(isinstance(m, QuantReLU) for m in model.modules()) == 2
        assert type(model[4]) is nn.LeakyReLU
        mtq.set_quantizer_by_cfg(model, {"*input_quantizer": {"num_bits": 4, "enable": False}})
        assert model[1].input_quantizer.num_bits == 4 and not model[1].input_quantizer.is_enabled
        x = torch.randn(2, 8)
        mtq.disable_quantizer(model, "*")
        assert torch.equal(model[1](x), torch.relu(x))
    finally:
        mtq.unregister(nn.ReLU)
    assert mtq.QuantModuleRegistry.get(nn.ReLU) is None
    with pytest.raises(KeyError):
        mtq.unregister(nn.ReLU)
    with pytest.raises(AssertionError, match="_setup"):
        mtq.register(nn.ReLU, nn.ReLU)


def test_quantizer_attribute_config_like_the_reference_tests():
    """Reference tests/unit/torch/quantization/test_tensor_quant_cpu.py:33-87."""
    C = mtq.QuantizerAttributeConfig
    assert C(num_bits=5).num_bits == 5 and C(num_bits=5).axis is None
    assert C(axis=(0, 1, 3)).num_bits == 8 and C(axis=(0, 1, 3)).axis == (0, 1, 3)
    for cfg in (C(num_bits=2, fake_quant=True, axis=(1, 2)), C(num_bits=2, unsigned=True)):
        assert C(**cfg.dict()) == cfg
    with pytest.raises(ValueError, match="Cannot specify only {'enable': True}"):
        C(enable=True)
    C(enable=False)
    C()
    for bits in (0, -1, (0, 3), (-1, 2)):
        with pytest.raises(ValueError, match="num_bits must be a positive integer or a tuple of positive integers."):
            C(enable=True, num_bits=bits)
    m = MLP()
    mtq.replace_quant_module(m)
    mtq.set_quantizer_by_cfg(m, mtq.INT8_DEFAULT_CFG["quant_cfg"])
    mtq.disable_quantizer(m, "*up_proj*")
    mtq.enable_quantizer(m, "*up_proj*")          # a bare enable through the wildcard API keeps the attributes
    assert m.up_proj.weight_quantizer.is_enabled and m.up_proj.weight_quantizer.num_bits == 8


def test_need_calibration_like_the_reference_test():
    """Reference tests/unit/torch/quantization/test_config_validation.py:28-35.  NVFP4 needs data although its
    block scales are dynamic: the second-level scale comes from a calibrated per-tensor amax."""
    from b200q.config import need_calibration

    assert need_calibration(mtq.FP8_DEFAULT_CFG)
    assert not need_calibration(mtq.FP8_PER_CHANNEL_PER_TOKEN_CFG)
    assert not need_calibration(mtq.FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG)
    assert need_calibration(mtq.INT4_AWQ_CFG)
    assert need_calibration(mtq.W4A8_AWQ_BETA_CFG)
    assert need_calibration(mtq.NVFP4_DEFAULT_CFG)


@pytest.mark.parametrize(("shape", "quant_axis", "expected"), [
    ((2, 3, 4), None, None), ((2, 3, 4), 0, [1, 2]), ((2, 3, 4), -2, [0, 2]),
    ((2, 3, 4, 5), [0, -1], [1, 2]), ((2, 3, 4), (0, 2), [1])])
def test_quantization_axis_to_reduce_axis_like_the_reference_test(shape, quant_axis, expected):
    """Reference tests/unit/torch/quantization/test_utils.py:62-103."""
    from b200q.utils import convert_quantization_axis_to_reduce_axis

    assert convert_quantization_axis_to_reduce_axis(torch.empty(shape), quant_axis) == expected


def test_replaced_modules_with_quantisers_off_compute_what_the_originals_do():
    """Reference tests/unit/torch/quantization/test_quantize_replace.py:35-58, the linear model: conversion
    keeps the parameters, and with every quantiser switched off nothing of the forward changes (no kernel
    runs, so this holds on the CPU too)."""
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))
    quantised = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))
    quantised.load_state_dict(ref.state_dict())
    mtq.replace_quant_module(quantised)
    for m in quantised.modules():
        assert not isinstance(m, nn.Linear) or (hasattr(m, "weight_quantizer") and hasattr(m, "input_quantizer"))
    mtq.set_quantizer_attribute(quantised, "*", {"enable": False})
    x = torch.randn(2, 16)
    assert torch.equal(ref(x), quantised(x))


@pytest.mark.parametrize(("state_dict", "quantization", "expected"), [
    ({"layer1.k_bmm_quantizer._amax": torch.tensor([0.128]), "layer1.v_bmm_quantizer._amax": torch.tensor([256.0]),
      "layer1.input_quantizer._pre_quant_scale": torch.tensor([0.128])}, "FP8",
     {"layer1.k_proj.k_scale": torch.tensor([1.0]), "layer1.v_proj.v_scale": torch.tensor([2.0]),
      "layer1.pre_quant_scale": torch.tensor([0.128])}),
    ({"layer1.q_bmm_quantizer._amax": torch.tensor([0.128]), "layer1.k_bmm_quantizer._amax": torch.tensor([0.128]),
      "layer1.v_bmm_quantizer._amax": torch.tensor([256])}, "FP8",
     {"layer1.k_proj.k_scale": torch.tensor([1.0]), "layer1.v_proj.v_scale": torch.tensor([2.0])}),
    ({"layer1.input_quantizer._pre_quant_scale": torch.tensor([0.128])}, None,
     {"layer1.pre_quant_scale": torch.tensor([0.128])})])
def test_postprocess_state_dict_like_the_reference_test(state_dict, quantization, expected):
    """Reference tests/gpu/torch/export/test_export.py:199-253: KV-cache amax becomes k_scale / v_scale =
    amax / maxbound, at least 1 for an FP8 cache; other amax entries are dropped."""
    from b200q import export

    got = export.postprocess_state_dict(state_dict, 128.0, quantization)
    assert got.keys() == expected.keys()
    for k, v in expected.items():
        assert torch.equal(got[k], v), k
    with pytest.raises(AssertionError, match="Invalid KV cache"):
        export.postprocess_state_dict({"l.k_bmm_quantizer._amax": torch.tensor([1.0])}, 128.0, None)


def test_process_layer_quant_config_like_the_reference_test():
    """Reference tests/gpu/torch/export/test_export.py:84-142: several formats give MIXED_PRECISION with the
    settings layer by layer; one format gives that format with the excluded modules."""
    from b200q import export

    mixed = export.process_layer_quant_config({
        "layer1.quantization": "nvfp4", "layer1.awq_block_size": 16, "layer3.quantization": "int4_awq",
        "layer3.awq_block_size": 8, "layer4.quantization": "w4a8_awq", "layer4.awq_block_size": 64,
        "layer5.quantization": "int8_sq", "layer6.quantization": "fp8", "layer7.quantization": "xyz",
        "layer8.quantization": None})
    assert mixed == {
        "quant_algo": "MIXED_PRECISION", "kv_cache_quant_algo": None,
        "quantized_layers": {
            "layer1": {"quant_algo": "NVFP4", "group_size": 16},
            "layer3": {"quant_algo": "W4A16_AWQ", "group_size": 8, "has_zero_point": False, "pre_quant_scale": True},
            "layer4": {"quant_algo": "W4A8_AWQ", "group_size": 64, "has_zero_point": False, "pre_quant_scale": True},
            "layer5": {"quant_algo": "W8A8_SQ_PER_CHANNEL"}, "layer6": {"quant_algo": "FP8"},
            "layer7": {"quant_algo": "xyz"}}}
    single = export.process_layer_quant_config({
        "layer1.quantization": "nvfp4", "layer1.awq_block_size": 16, "layer2.quantization": "nvfp4",
        "layer2.awq_block_size": 16, "layer8.quantization": None})
    assert single == {"quant_algo": "NVFP4", "kv_cache_quant_algo": None, "group_size": 16,
                      "exclude_modules": ["layer8"]}
    # excluded modules are summarised by prefixes cut at dots that match no quantised layer
    summary = export.process_layer_quant_config({
        **{f"model.layers.{i}.mlp.up.quantization": "fp8" for i in range(2)},
        **{f"model.layers.{i}.mlp.gate.quantization": None for i in range(2)},
        "vision.a.quantization": None, "vision.b.quantization": None, "lm_head.quantization": None})
    assert summary["exclude_modules"] == ["lm_head", "model.layers.0.mlp.gate", "model.layers.1.mlp.gate", "vision*"]
    for items, same in ((["a", "a", "a"], True), (["b", "a", "a"], False), ([True, False, True], False), ([False], True)):
        assert export.all_items_same(items) == same


def test_quantization_record_in_the_hugging_face_shape():
    """Reference modelopt/torch/export/convert_hf_config.py:21-117 (its docstring's FP8 example)."""
    from b200q import export

    got = export.convert_hf_quant_config_format({
        "producer": {"name": "modelopt", "version": "0.19.0"},
        "quantization": {"quant_algo": "FP8", "kv_cache_quant_algo": "FP8", "exclude_modules": ["lm_head"]}})
    eight = {"dynamic": False, "num_bits": 8, "type": "float"}
    assert got == {"config_groups": {"group_0": {"input_activations": eight, "weights": eight, "targets": ["Linear"]}},
                   "ignore": ["lm_head"], "quant_algo": "FP8", "kv_cache_scheme": eight,
                   "producer": {"name": "modelopt", "version": "0.19.0"}, "quant_method": "modelopt"}
    nvfp4 = export.convert_hf_quant_config_format({"quantization": {"quant_algo": "NVFP4", "group_size": 16}})
    assert nvfp4["config_groups"]["group_0"]["weights"] == {"dynamic": False, "num_bits": 4, "type": "float", "group_size": 16}
    assert nvfp4["ignore"] == [] and "kv_cache_scheme" not in nvfp4
