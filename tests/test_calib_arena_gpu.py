"""Histogram calibrators whose counters live in one arena: device-resident ranges, shared binning passes,
the in-place data-parallel merge, and that merge against its oracle — the sequential single-process
calibrator over all shards in rank order (the reference has no histogram exchange at all,
modelopt/torch/quantization/calib/histogram.py:158-163, so the sequential run is what a merge must equal;
tolerance 1e-3 on the percentile amax, counts identical)."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from _util import load, tensor_from_f32, to_f32

pytestmark = pytest.mark.gpu


def _quantizers(mtq, n):
    m = torch.nn.ModuleDict()
    for i in range(n):
        q = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, calibrator="histogram")).cuda()
        q.enable_calib()
        q.disable_quant()
        m[f"q{i}"] = q
    return m


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


def _batches(seed, n, shape=(512, 1024), grow=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for i in range(n):
        x = torch.randn(shape, generator=g, device="cuda") * (1.0 + grow * i)
        x[:, :3] *= 20
        out.append(x.bfloat16())
    return out


def test_arena_calibrators_equal_standalone_ones(mtq):
    """Same batches through an arena calibrator (range on the device, binning held back one call) and a
    stand-alone one (range through the host): identical counters, live lengths, edges and amax — also
    when later batches exceed the first batch's range."""
    from b200q.calib import HistogramCalibrator, attach_histogram_arena

    model = _quantizers(mtq, 2)
    (arena,) = attach_histogram_arena(model)
    ref = [HistogramCalibrator(8, None, False, num_bins=2048) for _ in range(2)]
    data = [_batches(1, 3), _batches(2, 3, grow=3.0)]
    for b in range(3):
        for i in range(2):
            model[f"q{i}"](data[i][b])
            ref[i].collect(data[i][b])
    for i in range(2):
        cal = model[f"q{i}"]._calibrator
        assert cal._arena is arena
        assert torch.equal(cal.hist, ref[i].hist)
        assert cal._num_bins == ref[i]._num_bins and cal._num_bins >= 2048
        assert torch.equal(cal._calib_bin_edges, ref[i]._calib_bin_edges)
        for method in ("percentile", "entropy"):
            assert cal.compute_amax(method).item() == ref[i].compute_amax(method).item()
    assert ref[1]._num_bins > 2048          # the growing sequence did outgrow the first range


def test_calibrators_fed_the_same_tensor_share_one_pass(mtq, monkeypatch):
    """q/k/v-style: three calibrators see tensor A, one sees B, two see C, per batch.  One launch per
    distinct tensor, and every calibrator ends with exactly the counters it gets on its own."""
    from b200q import ops
    from b200q.calib import HistogramCalibrator, attach_histogram_arena

    model = _quantizers(mtq, 6)
    attach_histogram_arena(model)
    launches = []
    real = ops.hist_collect_shared
    monkeypatch.setattr(ops, "hist_collect_shared", lambda x, counts, *a, **k: (launches.append(len(counts)), real(x, counts, *a, **k))[1])
    groups = [(0, 1, 2), (3,), (4, 5)]
    data = [_batches(10 + j, 3, grow=0.7 * j) for j in range(3)]
    ref = [HistogramCalibrator(8, None, False, num_bins=2048) for _ in range(6)]
    for b in range(3):
        for j, members in enumerate(groups):
            for i in members:
                model[f"q{i}"](data[j][b])
                ref[i].collect(data[j][b])
    for i in range(6):
        assert torch.equal(model[f"q{i}"]._calibrator.hist, ref[i].hist), i
    assert launches == [3, 1, 2] * 3


def test_tensor_modified_before_its_held_back_pass_is_reported(mtq):
    from b200q.calib import attach_histogram_arena

    model = _quantizers(mtq, 1)
    (arena,) = attach_histogram_arena(model)
    x = _batches(3, 1)[0]
    model["q0"](x)
    x.mul_(2)
    with pytest.raises(RuntimeError, match="modified in place"):
        arena.flush()


@pytest.mark.parametrize("world", [2, 4])
def test_data_parallel_merge_equals_the_sequential_calibrator(mtq, world):
    """`world` virtual ranks on one GPU, each with its own model and arena and its own shard of the
    batches; ranges and counters are exchanged by the code the real ranks run (`agree_histogram_ranges`,
    `sync_histograms`), with the collective replaced by its definition over the virtual ranks.  Every
    rank must end with the counters and the percentile amax of ONE calibrator that saw all shards in rank
    order; that calibrator is checked against the numpy oracle, and the reference's own batches
    (`hist.npz`) are pushed through the same merge."""
    from b200q import dist as qdist
    from b200q.calib import HistogramCalibrator, attach_histogram_arena

    n_q, per_rank = 3, 2
    shards = [[_batches(100 * r + q, per_rank, grow=0.5 * (r + 1)) for q in range(n_q)] for r in range(world)]
    g = load("hist")
    golden = [tensor_from_f32(to_f32(g[f"x{b}"], "bf16"), "bf16") for b in range(3)]
    if world == 2:               # quantiser 0 of the two virtual ranks shares out the reference's own batches
        for r in range(world):
            shards[r][0] = golden[r::world]
    models = [_quantizers(mtq, n_q) for _ in range(world)]
    arenas = [attach_histogram_arena(m)[0] for m in models]
    # first batch of every rank fixes a (rank-local) range on the device ...
    for r in range(world):
        for q in range(n_q):
            models[r][f"q{q}"]._calibrator.observe_range(shards[r][q][0])
    # ... and rank 0's is broadcast
    for r in range(world):
        qdist.agree_histogram_ranges(models[r], broadcast=lambda t, r=r: t.copy_(arenas[0].ranges) if r else None)
    for r in range(world):
        for q in range(n_q):
            for x in shards[r][q]:
                models[r][f"q{q}"](x)
    for a in arenas:
        a.flush()
    total = {"counts": sum(a.counts for a in arenas), "overflow": sum(a.overflow for a in arenas)}

    def all_reduce_for(rank):
        def fn(t, op):
            which = "counts" if t.dim() == 2 else "overflow"
            assert op == torch.distributed.ReduceOp.SUM and t.data_ptr() == getattr(arenas[rank], which).data_ptr()
            t.copy_(total[which])
        return fn

    for r in range(world):
        assert qdist.sync_histograms(models[r], all_reduce=all_reduce_for(r)) == 2
    for q in range(n_q):
        seq = HistogramCalibrator(8, None, False, num_bins=2048)
        everything = [x for r in range(world) for x in shards[r][q]]
        for x in everything:
            seq.collect(x)
        want = seq.compute_amax("percentile", percentile=99.99).item()
        for r in range(world):
            cal = models[r][f"q{q}"]._calibrator
            assert torch.equal(cal.hist, seq.hist), (q, r)
            got = cal.compute_amax("percentile", percentile=99.99).item()
            assert abs(got - want) <= 1e-3 * want, (q, r, got, want)
        # the sequential calibrator itself against the oracle (same binning arithmetic, numpy)
        orc = qo.HistogramOracle(2048)
        for x in everything:
            orc.collect(x.float().cpu().numpy())
        o = float(qo.percentile_amax(orc.hist, orc.edges, 99.99)[0])
        assert abs(want - o) <= 1e-3 * o, (q, want, o)
    if world == 2:
        # quantiser 0 held the reference's batches: its merged amax against what the reference got sequentially
        got = models[0]["q0"]._calibrator.compute_amax("percentile", percentile=99.99).item()
        assert abs(got - g["pct_99.99"]) <= 1e-3 * g["pct_99.99"]


def test_histogram_calibrate_equals_the_stand_alone_calibrators(mtq):
    """mtq.histogram_calibrate (arena, shared passes, percentile read-out into ``_amax``) against
    stand-alone calibrators fed the same batches; with no process group it is the sequential contract."""
    from b200q.calib import HistogramCalibrator

    model = torch.nn.ModuleDict()
    for i in range(3):
        model[f"q{i}"] = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, calibrator="histogram")).cuda()
    data = _batches(21, 3, grow=1.5)

    def loop(m):
        for x in data:
            for q in m.values():
                q(x)

    mtq.histogram_calibrate(model, loop, method="percentile", percentile=99.9)
    ref = HistogramCalibrator(8, None, False, num_bins=2048)
    for x in data:
        ref.collect(x)
    want = ref.compute_amax("percentile", percentile=99.9)
    for q in model.values():
        assert q._if_quant and not q._if_calib
        assert q._amax.item() == want.item()
        assert torch.equal(q._calibrator.hist, ref.hist)
    y = model["q0"](data[0])
    assert y.shape == data[0].shape and not torch.equal(y, data[0])


def test_batched_amax_load_reports_every_invalid_quantiser(mtq):
    """finish_stats_collection loads all calibrated amax values with one validity read; a NaN or inf
    input is reported with the names of the quantisers it reached (the reference raises at the first)."""
    from b200q.model_calib import enable_stats_collection, finish_stats_collection

    model = torch.nn.ModuleDict({f"q{i}": mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8)).cuda()
                                 for i in range(4)})
    good = torch.randn(64, 64, device="cuda")
    enable_stats_collection(model)
    for q in model.values():
        q(good)
    finish_stats_collection(model)
    for q in model.values():
        assert q._amax.item() == good.abs().max().item() and q._if_quant and not q._if_calib
    bad = good.clone()
    bad[3, 3] = float("inf")
    enable_stats_collection(model)
    for name, q in model.items():
        q._calibrator.reset()
        q(bad if name in ("q1", "q3") else good)
    with pytest.raises(ValueError, match=r"q1.*q3"):
        finish_stats_collection(model)


def test_batched_percentile_read_out_equals_the_single_one(mtq):
    """load_calib_amax_all reads the percentile amax of all histogram calibrators with one launch; every
    value equals the single-histogram kernel's (bit for bit: the same code per CTA), for arena and
    stand-alone calibrators, grown and not grown histograms."""
    from b200q.calib import attach_histogram_arena
    from b200q.model_calib import load_calib_amax_all

    model = _quantizers(mtq, 5)
    loose = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, calibrator="histogram")).cuda()
    loose.enable_calib(); loose.disable_quant()
    attach_histogram_arena(model)
    model["loose"] = loose
    for i, q in enumerate(model.values()):
        for x in _batches(40 + i, 3, grow=1.0 * i):
            q(x)
    want = {n: q._calibrator.compute_amax("percentile", percentile=99.9).item() for n, q in model.items()}
    assert model["q4"]._calibrator._num_bins > 2048          # grown histograms are part of the batch
    n = load_calib_amax_all([(name, q, ("percentile",), {"percentile": 99.9}) for name, q in model.items()])
    assert n == 6
    for name, q in model.items():
        assert q._amax.item() == want[name], name


def test_batched_bin_edges_equal_torch_linspace_and_the_grown_form():
    """The arena builds all calibrators' bin edges in two batched computations; each row must be what the
    single calibrator builds: ``torch.linspace(0, range, bins + 1)`` to the bit (torch's kernel rounds the
    second half once, through a fused multiply-add), and ``arange(n + 1) * width`` once the histogram grew."""
    from b200q.calib.histogram import _batched_linspace

    g = torch.Generator(device="cuda").manual_seed(0)
    ends = torch.cat([torch.rand(500, generator=g, device="cuda") * 100 + 0.01,
                      torch.tensor([33.72509765625, 85.3857421875, 1.0, 3.0, 7.123456], device="cuda")])
    for steps in (2049, 33, 1001):
        want = torch.stack([torch.linspace(0, float(e), steps, device="cuda") for e in ends])
        assert torch.equal(_batched_linspace(ends, steps), want), steps


def test_arena_read_back_gives_the_single_calibrators_edges_after_growth():
    from b200q.calib import HistogramCalibrator, attach_histogram_arena
    from b200q.nn import TensorQuantizer

    g = torch.Generator(device="cuda").manual_seed(1)
    batches = [torch.randn(256, 512, generator=g, device="cuda").bfloat16() * s for s in (1.0, 1.0, 3.0)]   # the third grows the range
    model = torch.nn.ModuleDict({f"q{i}": TensorQuantizer({"num_bits": 8, "calibrator": "histogram"}) for i in range(3)}).cuda()
    for q in model.values():
        q.disable_quant(); q.enable_calib()
    attach_histogram_arena(model)
    alone = [HistogramCalibrator(8, None, False) for _ in range(3)]
    for i, (q, cal) in enumerate(zip(model.values(), alone)):
        for b in batches[: 2 + (i > 0)]:        # the first calibrator never grows
            q(b * (i + 1))
            cal.collect(b * (i + 1))
    for q, cal in zip(model.values(), alone):
        a = q._calibrator
        a._resolve(); cal._resolve()
        assert a._num_bins == cal._num_bins
        assert torch.equal(a._calib_bin_edges, cal._calib_bin_edges)
        assert torch.equal(a._calib_hist[: a._num_bins], cal._calib_hist[: cal._num_bins])
        assert torch.equal(a.compute_amax("percentile", percentile=99.9), cal.compute_amax("percentile", percentile=99.9))
