"""The modelopt-style API (quantize / calibrate / compress, TensorQuantizer, calibrators, QTensors)
on the GPU against golden results of the reference run on CPU and against the oracle."""
import copy

import numpy as np
import pytest
import torch
from torch import nn

from oracle import quant_oracle as qo
from _util import f32_from_tensor, load, same_bits, tensor_from_f32, to_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


class MLP(nn.Module):
    def __init__(self, hidden=128, inter=256):
        super().__init__()
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.up_proj(x)))


def build(g, prefix, T, dtype):
    m = MLP().to(dtype).cuda()
    with torch.no_grad():
        m.up_proj.weight.copy_(tensor_from_f32(to_f32(g[prefix + "w_up"], T), T))
        m.down_proj.weight.copy_(tensor_from_f32(to_f32(g[prefix + "w_down"], T), T))
    return m


def bits_of(t):
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


@pytest.mark.parametrize("fmt", ["int8", "fp8", "nvfp4"])
def test_quantize_max_calibration_matches_reference(mtq, fmt):
    g = load("flows")
    model = build(g, "", "bf16", torch.bfloat16)
    batches = [tensor_from_f32(to_f32(g[f"x{i}"], "bf16"), "bf16") for i in range(3)]
    cfg = {"int8": mtq.INT8_DEFAULT_CFG, "fp8": mtq.FP8_DEFAULT_CFG, "nvfp4": mtq.NVFP4_DEFAULT_CFG}[fmt]

    def loop(m):
        for b in batches:
            m(b)

    mtq.quantize(model, copy.deepcopy(cfg), loop)
    for name in ("up_proj", "down_proj"):
        lin = getattr(model, name)
        assert lin.input_quantizer._amax.dtype == torch.bfloat16
        assert same_bits(lin.input_quantizer._amax.float().reshape(-1).cpu().numpy(), g[f"{fmt}_{name}_in_amax"])
        assert same_bits(lin.weight_quantizer._amax.float().reshape(-1).cpu().numpy(), g[f"{fmt}_{name}_w_amax"])
    y = model(batches[0])
    assert torch.isfinite(y).all()
    if fmt != "nvfp4":
        ref = to_f32(g[f"{fmt}_y"], "bf16")
        # GEMMs accumulate in a different order on the two devices: outputs agree to bf16 noise
        assert np.allclose(f32_from_tensor(y), ref, rtol=5e-2, atol=5e-3 * np.abs(ref).max())
    else:
        mtq.compress(model, config={"quant_gemm": False})
        assert np.array_equal(np.array(sorted(model.state_dict().keys())), g["nvfp4_state_keys"])
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            assert type(lin).__name__ == "RealQuantLinear"
            assert np.array_equal(bits_of(lin.weight.data), g[f"nvfp4_{name}_packed"]), name
            assert np.array_equal(bits_of(lin.weight_quantizer._scale), g[f"nvfp4_{name}_scale"]), name
            assert same_bits(lin.weight_quantizer._double_scale.reshape(1).cpu().numpy(),
                             g[f"nvfp4_{name}_double_scale"]), name
        y2 = model(batches[0])  # forward through dequantised packed weights
        assert torch.isfinite(y2).all()
        assert np.allclose(f32_from_tensor(y2), f32_from_tensor(y), rtol=5e-2, atol=1e-2 * float(y.abs().max()))


def _bf16_ulp(v):
    """Spacing of bfloat16 at |v| (normal range)."""
    return 2.0 ** (np.floor(np.log2(np.maximum(np.abs(v), 1e-30))) - 7)


def _equal_up_to_rounding_flips(got, ref, T, max_fraction, what):
    """Statistics the reference reduces in the tensor dtype: for bf16 every channel is either equal or
    ONE bf16 ulp away (a mean whose fp32 value sits near a bf16 tie rounds the other way under another
    summation order), and only a small fraction may be; for fp32 only the summation order of the fp32
    mean differs (1e-5)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    if T != "bf16":
        assert np.allclose(got, ref, rtol=1e-5), what
        return np.zeros(got.shape, bool)
    diff = got != ref
    assert np.all(np.abs(got - ref)[diff] <= 1.0000001 * _bf16_ulp(np.maximum(np.abs(got), np.abs(ref)))[diff]), what
    assert diff.mean() <= max_fraction, (what, int(diff.sum()), diff.size)
    return diff


@pytest.mark.parametrize("fixture,shape", [("awq", (128, 256)), ("awq128", (256, 512))])
@pytest.mark.parametrize("T,dtype", [("bf16", torch.bfloat16), ("f32", torch.float32)])
def test_awq_lite_matches_reference(mtq, T, dtype, fixture, shape, monkeypatch):
    """mtq.quantize(INT4_AWQ_CFG, alpha_step 0.05) against what the reference produced on the CPU for the
    same model and batches: the alpha grid exactly, the statistics up to single-ulp rounding flips, the
    scale function to 1e-5, the selected scale to 1e-3, the loss curve to 2 %; ``awq128`` (256 -> 512 ->
    256, 128 tokens per batch) and ``awq`` (128 -> 256 -> 128, 48 tokens) both run the fused tcgen05
    search kernel in bf16 (asserted)."""
    from b200q import model_calib, ops

    g = load(fixture)
    p = T + "_"
    model = MLP(*shape).to(dtype).cuda()
    with torch.no_grad():
        model.up_proj.weight.copy_(tensor_from_f32(to_f32(g[p + "w_up"], T), T))
        model.down_proj.weight.copy_(tensor_from_f32(to_f32(g[p + "w_down"], T), T))
    batches = [tensor_from_f32(to_f32(g[f"{p}x{i}"], T), T) for i in range(2)]
    cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
    cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.05, "debug": True}
    fused_calls = []
    real = ops.awq_search_fused
    monkeypatch.setattr(ops, "awq_search_fused", lambda *a, **k: (fused_calls.append(1), real(*a, **k))[1])

    def loop(m):
        for b in batches:
            m(b)

    mtq.quantize(model, cfg, loop)
    assert bool(fused_calls) == (T == "bf16"), "bf16 layers of these shapes go through the fused search kernel"
    for name in ("up_proj", "down_proj"):
        lin = getattr(model, name)
        st = lin.awq_lite
        k = f"{p}{name}_"
        alphas = list(st.loss.keys())
        assert np.array_equal(np.array(alphas, dtype=np.float64), g[k + "alphas"])  # 21 fp32 keys
        ours_w, ours_a = st.weight_scale.cpu().numpy(), st.act_scale.cpu().numpy()
        flips = _equal_up_to_rounding_flips(ours_w, g[k + "weight_scale"], T, 0.05, name + " weight_scale")
        flips |= _equal_up_to_rounding_flips(ours_a, g[k + "act_scale"], T, 0.05, name + " act_scale")
        losses = np.array([float(v) for v in st.loss.values()])
        ref = g[k + "losses"]
        curves = f"{name}: ours {losses.tolist()} reference {ref.tolist()}"
        assert np.allclose(losses, ref, rtol=2e-2), curves
        # the scale function itself: the reference's formula on OUR statistics, for every alpha of the grid
        for a in (alphas[0], alphas[7], st.best_alpha, alphas[-1]):
            want = qo.awq_get_scale(ours_a, ours_w, a)
            assert np.allclose(model_calib.get_scale(st.act_scale, st.weight_scale, a).cpu().numpy(), want, rtol=1e-5), a
        ref_alpha = float(g[k + "best_alpha"])
        if st.best_alpha != ref_alpha:
            # a different grid point may only win where the reference's own curve is flat to 2 %
            i = alphas.index(st.best_alpha)
            assert ref[i] <= ref.min() * 1.02, (st.best_alpha, ref_alpha, curves)
            continue
        ours_s, ref_s = st.best_scale.cpu().numpy().astype(np.float64), g[k + "best_scale"].astype(np.float64)
        same = ~flips
        ratio = ours_s[same] / ref_s[same]
        # channels with identical statistics differ from the reference by one common factor (the
        # normalisation sqrt(max * min), which a flipped extreme channel moves by half a bf16 ulp at most)
        assert ratio.max() / ratio.min() - 1 <= 1e-5, name
        raw = qo.awq_get_scale(g[k + "act_scale"], g[k + "weight_scale"], ref_alpha)
        extremes_flipped = bool(flips[int(np.argmax(raw))] or flips[int(np.argmin(raw))])
        assert abs(np.median(ratio) - 1) <= (2.5e-3 if extremes_flipped else 1e-3), (name, float(np.median(ratio)))
        assert np.allclose(ours_s[same], ref_s[same], rtol=2.5e-3 if extremes_flipped else 1e-3)
        # what is folded into the layer: pre_quant_scale = T(1 / scale), weight = T(W * scale)
        pqs = lin.input_quantizer._pre_quant_scale.float().cpu().numpy()
        assert np.array_equal(pqs, qo.round_to((1.0 / st.best_scale.cpu().numpy()).astype(np.float32), T))
        ref_pqs = to_f32(g[k + "pqs"], T)
        if T == "bf16":
            assert np.all(np.abs(pqs - ref_pqs) <= 1.0000001 * _bf16_ulp(np.maximum(pqs, ref_pqs))), name
        else:
            assert np.allclose(pqs, ref_pqs, rtol=1e-3)
        wf, ref_w = f32_from_tensor(lin.weight), to_f32(g[k + "w_folded"], T)
        if T == "bf16":   # T(W * T(scale)): equal, or a bf16 ulp or two apart where the scale's bf16 value differs
            assert np.all(np.abs(wf - ref_w) <= 2.0000001 * _bf16_ulp(np.maximum(np.abs(wf), np.abs(ref_w))))
            assert np.mean(wf != ref_w) <= max(0.05, 2.0 * np.mean(pqs != ref_pqs)), name
        else:
            assert np.allclose(wf, ref_w, rtol=1e-3, atol=1e-7)
        assert lin.weight_quantizer._amax.shape == g[k + "w_amax"].shape
    assert torch.isfinite(model(batches[0])).all()
    mtq.compress(model)
    assert model.up_proj.weight.dtype == torch.uint8
    assert model.up_proj.weight.shape == (shape[1], shape[0] // 2)
    assert torch.isfinite(model(batches[0])).all()


@pytest.mark.parametrize("name,n,k", [("up_proj", 14336, 4096), ("down_proj", 4096, 14336)])
def test_awq_lite_at_the_benchmark_shapes_against_the_oracle(mtq, name, n, k):
    """The awq_lite search of one Llama-3-8B MLP projection (512 tokens, lognormal channel magnitudes,
    alpha step 0.05) through mtq.quantize against the oracle's restatement of the reference's search on
    five candidates of the grid: statistics up to single-ulp flips, scales to 1e-3, losses to 1e-3."""
    g = torch.Generator(device="cuda").manual_seed(7)
    lin = nn.Linear(k, n, bias=False, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        lin.weight.copy_((torch.randn(n, k, generator=g, device="cuda") * 0.02).bfloat16())
    x = (torch.randn(512, k, generator=g, device="cuda") * torch.exp(torch.randn(k, generator=g, device="cuda"))).bfloat16()
    model = nn.Sequential()
    model.add_module(name, lin)
    cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
    cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.05, "debug": True}
    w_np, x_np = lin.weight.detach().float().cpu().numpy(), x.float().cpu().numpy()
    mtq.quantize(model, cfg, lambda m: m(x))
    st = getattr(model, name).awq_lite
    alphas = list(st.loss.keys())
    assert len(alphas) == 21
    subset = [alphas[i] for i in (0, 5, 10, 15, 20)]
    wsc, asc, losses, _, _ = qo.awq_lite_search(w_np, [x_np], 128, subset, "bf16")
    flips = _equal_up_to_rounding_flips(st.weight_scale.cpu().numpy(), wsc, "bf16", 0.05, "weight_scale")
    flips |= _equal_up_to_rounding_flips(st.act_scale.cpu().numpy(), asc, "bf16", 0.05, "act_scale")
    ours = np.array([st.loss[a] for a in subset])
    want = np.array([losses[a] for a in subset])
    # a flipped statistic moves a few channels' scales by a bf16 ulp: second order in the loss
    assert np.allclose(ours, want, rtol=1e-3 if not flips.any() else 5e-3), (ours.tolist(), want.tolist())
    assert st.loss[st.best_alpha] == min(st.loss.values())
    s_ours = st.best_scale.cpu().numpy()
    s_want = qo.awq_get_scale(st.act_scale.cpu().numpy(), st.weight_scale.cpu().numpy(), st.best_alpha)
    assert np.allclose(s_ours, s_want, rtol=1e-5)


def test_awq_scale_fake_int_kernel_vs_oracle(mtq):
    from b200q import ops

    rng = np.random.default_rng(3)
    for T in ("bf16", "f16", "f32"):
        w = qo.round_to(rng.standard_normal((96, 512)).astype(np.float32) * 0.02, T)
        s = qo.round_to(np.exp(rng.standard_normal(512)).astype(np.float32), T)
        y = ops.awq_scale_fake_int(tensor_from_f32(w, T), tensor_from_f32(s, T), 128, 4, False, False)
        v = qo.round_to((w * s[None, :]).astype(np.float32), T).reshape(-1, 128)
        amax = np.abs(v).max(-1, keepdims=True)
        want = qo.fake_int(v, amax, 4, False, False, T).reshape(w.shape)
        assert same_bits(f32_from_tensor(y), want), T
        a = tensor_from_f32(w, T)
        b = tensor_from_f32(want, T)
        d = qo.round_to((w - want).astype(np.float32), T).astype(np.float64)
        got = ops.mse_loss(a, b).item()
        assert abs(got - (d ** 2).mean()) <= 1e-6 * (d ** 2).mean()


def test_tensor_quantizer_block_quant_with_padding_matches_oracle(mtq):
    from b200q.nn import TensorQuantizer

    x = qo.round_bf16(np.random.default_rng(0).standard_normal((24, 200)).astype(np.float32))
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=4, block_sizes={-1: 128})).cuda()
    xt = tensor_from_f32(x, "bf16")
    y = q(xt)                                   # dynamic block amax (fused kernel), padded to 256
    xp = qo.pad_last(x, 128).reshape(-1, 128)
    want = qo.fake_int(xp, np.abs(xp).max(-1, keepdims=True), 4, False, False, "bf16").reshape(24, 256)[:, :200]
    assert y.shape == xt.shape and same_bits(f32_from_tensor(y), want)
    # calibrated: amax buffer per block, same result; export shape follows the reference
    mtq.max_calibrate(q, lambda m: m(xt), distributed_sync=False)
    assert q._amax.shape == (48, 1)
    assert same_bits(f32_from_tensor(q(xt)), want)
    assert q.export_amax().shape == (24, 2)


def test_tensor_quantizer_pre_quant_scale_and_per_channel(mtq):
    from b200q.nn import TensorQuantizer

    x = qo.round_bf16(np.random.default_rng(1).standard_normal((64, 256)).astype(np.float32))
    xt = tensor_from_f32(x, "bf16")
    q = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, axis=0, narrow_range=True)).cuda()
    mtq.max_calibrate(q, lambda m: m(xt), distributed_sync=False)
    amax = np.abs(x).max(-1, keepdims=True)
    assert same_bits(q._amax.float().cpu().numpy(), amax)
    assert same_bits(f32_from_tensor(q(xt)), qo.fake_int(x, amax, 8, False, True, "bf16"))
    pqs = qo.round_bf16(np.linspace(0.5, 2, 256).astype(np.float32))
    q2 = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=(4, 3))).cuda()
    q2.pre_quant_scale = tensor_from_f32(pqs, "bf16")
    xs = qo.round_bf16(x * pqs[None, :])
    q2.amax = torch.tensor(float(np.abs(xs).max()), device="cuda")
    assert same_bits(f32_from_tensor(q2(xt)), qo.fake_e4m3(xs, np.float32(np.abs(xs).max()), "bf16"))


def test_histogram_calibrator_matches_reference_sequence(mtq):
    g = load("hist")
    cal = mtq.calib.HistogramCalibrator(8, None, False, num_bins=2048)
    for b in range(3):
        cal.collect(tensor_from_f32(to_f32(g[f"x{b}"], "bf16"), "bf16"))
        ref = g[f"hist{b}"]
        got = cal.hist.cpu().numpy()
        assert got.size == ref.size and got.sum() == ref.sum(), b
        assert np.abs(got - ref).sum() <= 2e-3 * ref.sum(), b
        assert np.allclose(cal._calib_bin_edges.cpu().numpy(), g[f"edges{b}"], rtol=1e-5)
    for p in (99.0, 99.9, 99.99, 100.0):
        a = cal.compute_amax("percentile", percentile=p).item()
        assert abs(a - g[f"pct_{p}"]) <= 1e-3 * g[f"pct_{p}"], p
    e = cal.compute_amax("entropy").item()
    assert abs(e - g["entropy"]) <= 1e-3 * g["entropy"] + 2 * float(cal._calib_bin_edges[1])
    q = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=8, calibrator="histogram")).cuda()
    q.enable_calib(); q.disable_quant()
    for b in range(3):
        q(tensor_from_f32(to_f32(g[f"x{b}"], "bf16"), "bf16"))
    q.load_calib_amax("percentile", percentile=99.99)
    assert abs(q.amax.item() - g["pct_99.99"]) <= 1e-3 * g["pct_99.99"]


def test_qtensor_classes_roundtrip(mtq):
    from b200q.qtensor import FP8QTensor, INT4QTensor, INT8QTensor, NVFP4QTensor

    x = qo.round_bf16(np.random.default_rng(2).standard_normal((32, 200)).astype(np.float32) * 0.05)
    xt = tensor_from_f32(x, "bf16")
    q, s, s2 = NVFP4QTensor.quantize(xt, 16)                       # pads 200 -> 208
    wp, ws, ws2 = qo.nvfp4_quantize(x, 16)
    assert np.array_equal(q._quantized_data.cpu().numpy(), wp) and s2.item() == ws2
    d = q.dequantize(scale=s, double_scale=s2, block_sizes={-1: 16})
    assert d.shape == xt.shape
    assert same_bits(f32_from_tensor(d), qo.nvfp4_dequantize(wp, ws, ws2, 16, "bf16")[:, :200])
    qi, si = INT4QTensor.quantize(xt, 128)
    pk, sc = qo.int4_quantize(x, 128, "bf16")
    assert np.array_equal(qi._quantized_data.cpu().numpy().reshape(-1), pk)
    di = qi.dequantize(scale=si, block_sizes={-1: 128})
    assert same_bits(f32_from_tensor(di).reshape(-1), qo.int4_dequantize(pk, sc, 128, "bf16")[: x.size])
    for cls, fn, div in ((FP8QTensor, qo.fp8_quantize, 448.0), (INT8QTensor, qo.int8_quantize, 127.0)):
        for kw, view in (({}, None), ({"axis": 0}, (-1, 1)), ({"block_sizes": {-1: 40}}, None)):
            qq, ss = cls.quantize(xt, **kw)
            sf = ss.float().cpu().numpy()
            if "block_sizes" in kw:
                want = fn(x.reshape(32, 5, 40), sf.reshape(32, 5, 1), "bf16").reshape(32, 200)
            else:
                want = fn(x, sf.reshape(view) if view else sf.reshape(()), "bf16")
            assert np.array_equal(qq._quantized_data.view(torch.uint8).cpu().numpy(), want.view(np.uint8)), (cls, kw)
            dd = qq.dequantize(scale=ss, **({"block_sizes": kw["block_sizes"]} if "block_sizes" in kw else {}))
            assert dd.shape == xt.shape and torch.isfinite(dd).all()


def test_mse_calibration_matches_reference_int8(mtq):
    """INT8 amax search (algorithm "mse"): the selected candidates equal the reference's.  (The
    reference's FP8 result on CPU is an artefact of its non-saturating eager cast — every candidate
    below the data maximum yields NaN losses — and is not a parity target.)"""
    g = load("flows")
    model = build(g, "", "bf16", torch.bfloat16)
    batches = [tensor_from_f32(to_f32(g[f"x{i}"], "bf16"), "bf16") for i in range(3)]
    cfg = copy.deepcopy(mtq.INT8_DEFAULT_CFG)
    cfg["algorithm"] = "mse"
    mtq.quantize(model, cfg, lambda m: [m(b) for b in batches])
    for name in ("up_proj", "down_proj"):
        lin = getattr(model, name)
        got_in = lin.input_quantizer._amax.float().reshape(-1).cpu().numpy()
        got_w = lin.weight_quantizer._amax.float().reshape(-1).cpu().numpy()
        assert same_bits(got_in, g[f"int8_mse_{name}_in_amax"]), name
        ref_w = g[f"int8_mse_{name}_w_amax"]
        assert np.mean(got_w != ref_w) <= 0.02, name      # a near-tie between two candidates may flip
    from b200q.calib import MseCalibrator
    assert isinstance(model.up_proj.weight_quantizer._calibrator, MseCalibrator)


def test_reference_op_names_resolve_to_these_kernels(mtq):
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    amax = x.abs().amax().float()
    a = torch.ops.tensorrt.quantize_op(x, amax, 8, 4, False, False)
    b = torch.ops.b200q.quantize_op(x, amax, 8, 4, False, False)
    assert torch.equal(a, b)
    c = torch.ops.tensorrt.dynamic_block_quantize_op(x, 16, amax, 4, 2, 8, 4)
    assert torch.equal(c, mtq.ops.nvfp4_fake(x, amax))
    assert torch.ops.tensorrt.quantize_op(x.to("meta"), amax.to("meta"), 8, 0, False, True).shape == x.shape
    # the overload without a global amax: NVFP4 takes the tensor's own abs-max, the MX formats need none
    d = torch.ops.tensorrt.dynamic_block_quantize_op.overload(x, 16, None, 4, 2, 8, 4)
    assert torch.equal(d, c)
    e = torch.ops.tensorrt.dynamic_block_quantize_op.overload(x, 32, None, 8, 4, 9, 8)
    assert torch.equal(e, mtq.ops.mx_fake(x, 32, (4, 3)))


def test_batched_exchanges_over_nccl_single_rank(mtq):
    """The flat amax / histogram exchanges on GPU tensors through NCCL (world of one rank: the
    collectives run, the values must come back unchanged)."""
    import torch.distributed as dist

    if dist.is_initialized():
        pytest.skip("a process group already exists")
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29631", rank=0, world_size=1,
                            device_id=torch.device("cuda", 0))
    try:
        m = MLP().cuda().bfloat16()
        mtq.replace_quant_module(m)
        cfg = {"*input_quantizer": {"num_bits": 8, "axis": None, "calibrator": "histogram"},
               "*weight_quantizer": {"num_bits": 8, "axis": 0}, "default": {"enable": False}}
        mtq.set_quantizer_by_cfg(m, cfg)
        x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
        for q in (m.up_proj.input_quantizer, m.down_proj.input_quantizer):
            q._calibrator.collect(x)
        m.up_proj.weight_quantizer.amax = m.up_proj.weight.abs().amax(1, keepdim=True)
        m.down_proj.weight_quantizer.amax = m.down_proj.weight.abs().amax(1, keepdim=True)
        before = m.up_proj.weight_quantizer.amax.clone()
        assert mtq.dist.sync_amax(m) == 1
        assert torch.equal(before, m.up_proj.weight_quantizer.amax)
        h = m.up_proj.input_quantizer._calibrator.hist.clone()
        assert mtq.dist.sync_histograms(m) == 2
        assert torch.equal(h, m.up_proj.input_quantizer._calibrator.hist)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", ["f32", "f16", "bf16"])
def test_export_packers_match_reference(mtq, T):
    from b200q import export

    g = load("export")
    w = to_f32(g[f"{T}_w"], T)
    wt = tensor_from_f32(w, T)
    s4 = export.get_scaling_factor_from_weight(wt, 128)
    assert same_bits(s4.cpu().numpy(), g[f"{T}_int4_scale"])
    assert np.array_equal(export.to_quantized_weight(wt, s4, "int4_awq").cpu().numpy(), g[f"{T}_int4_packed"])
    # scales given in the weight's own type: the quotient is rounded to that type first
    s4t = tensor_from_f32(qo.round_to(s4.cpu().numpy(), T), T)
    got = export.pack_int4_in_uint8(wt, s4t).cpu().numpy()
    assert np.array_equal(got, qo.pack_int4_export(w, qo.round_to(s4.cpu().numpy(), T), T, scales_in_T=True))
    s8 = export.get_scaling_factor_from_weight(wt, 0)
    assert same_bits(s8.cpu().numpy(), g[f"{T}_int8_scale"])
    assert np.array_equal(export.to_quantized_weight(wt, s8, "int8_sq").cpu().numpy(), g[f"{T}_int8_q"])
    sf = torch.from_numpy(g[f"{T}_fp8_scale"]).cuda().reshape(())
    q = export.to_quantized_weight(wt, sf, "fp8")
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g[f"{T}_fp8_q"])
    wsf = torch.from_numpy(g[f"{T}_nvfp4_wsf"]).cuda().view(torch.float8_e4m3fn)
    wsf2 = torch.from_numpy(g[f"{T}_nvfp4_wsf2"]).cuda().reshape(())
    p = export.to_quantized_weight(wt, wsf, "nvfp4", wsf2, 16)
    assert np.array_equal(p.cpu().numpy(), g[f"{T}_nvfp4_packed"])


def test_histogram_calibrator_small_sequence_of_the_reference_test(mtq):
    """The 19-bin, 15-sample sequence of the reference's test_torch_hist (growth on every other
    batch), plus its integer-input and outlier property tests."""
    g = load("hist")
    x1, x2 = torch.from_numpy(g["small_x1"]).cuda(), torch.from_numpy(g["small_x2"]).cuda()
    cal = mtq.calib.HistogramCalibrator(8, None, False, num_bins=19)
    cal.collect(x1)
    assert np.array_equal(cal.hist.cpu().numpy(), g["small_hist0"])
    for r in range(3):
        cal.collect(x2)
        cal.collect(x1)
        got, ref = cal.hist.cpu().numpy(), g[f"small_hist{r + 1}"]
        assert got.sum() == ref.sum() and got.size == ref.size
        # x1's maximum IS the first range's right edge: the reference puts it in bin 18 while the range is
        # [0, max] and in bin 19 once the range has grown; here it stays in bin 18.  Everything else is equal.
        merged = lambda h: np.concatenate([h[:18], [h[18] + h[19]], h[20:]])  # noqa: E731
        assert np.array_equal(merged(got), merged(ref)), (got, ref)
        assert cal.hist.numel() == cal._calib_bin_edges.numel() - 1
        assert np.allclose(cal._calib_bin_edges.cpu().numpy(), g[f"small_edges{r + 1}"], rtol=1e-5)
        a = cal.compute_amax("percentile", percentile=99.99).item()
        assert abs(a - g[f"small_pct{r + 1}"]) <= float(cal._calib_bin_edges[1]) + 1e-6
    # integer inputs, a second batch one past the range (reference test_grow)
    cal = mtq.calib.HistogramCalibrator(8, None, False, num_bins=2048)
    cal.collect(torch.tensor([0, 255, 255, 255, 255, 255]).cuda())
    cal.collect(torch.tensor([0, 255, 255, 255, 255, 256]).cuda())
    assert abs(cal.compute_amax("mse", start_bin=128).item() - 255.0) < 0.5
    # one outlier among uniform samples is discarded by the entropy method (reference TestEntropyCalibrator)
    torch.manual_seed(1)
    for unsigned in (False, True):
        cal = mtq.calib.HistogramCalibrator(8, None, unsigned, num_bins=2048)
        x = torch.rand(11, 7, 3, 3).cuda()
        x[1, 1, 1, 1] = 10.0
        cal.collect(x)
        cal.collect(torch.rand(11, 7, 3, 3).cuda())
        assert cal.compute_amax("entropy", start_bin=128).item() < 1.1


def test_scales_from_quantizer_amax_like_the_reference_test(mtq):
    """reference test_amax_from_tensor_quantizer: with amax preset to 1.1 the NVFP4 per-tensor scale
    is amax/448/6 and the FP8 scale amax/448."""
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for num_bits, blocks, attr, want in (
                ((2, 1), {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, "_double_scale", 1.1 / 448.0 / 6.0),
                ((4, 3), None, "_scale", 1.1 / 448.0)):
            q = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=num_bits, block_sizes=blocks,
                                                                    fake_quant=False)).cuda()
            q.amax = torch.tensor(1.1, device="cuda")
            q(torch.rand(32, 32, device="cuda").to(dtype))
            assert torch.allclose(getattr(q, attr).float().reshape(()), torch.tensor(want, device="cuda"))


@pytest.mark.parametrize("T", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("block", [8, 32, 64])
def test_nvfp4_other_block_sizes_vs_oracle(mtq, T, block):
    """NVFP4 with the reference's other block sizes (8 in its tests, 32 in its W4A8 / MLP-only
    configs): packed bytes, scales, dequantised and fake-quantised values against the oracle."""
    from b200q import ops
    from test_kernels_gpu import rnd

    x = rnd((48, 256), T, 900 + block, 0.3, heavy=True)
    xt = tensor_from_f32(x, T)
    packed, scales, s2 = ops.nvfp4_quantize(xt, block=block)
    wp, ws, w2 = qo.nvfp4_quantize(x, block)
    assert np.array_equal(packed.cpu().numpy(), wp) and np.array_equal(scales.view(torch.uint8).cpu().numpy(), ws)
    assert float(s2) == float(w2)
    deq = ops.nvfp4_dequantize(packed, scales, s2, xt.dtype, block=block)
    assert same_bits(f32_from_tensor(deq), qo.nvfp4_dequantize(wp, ws, w2, block, T))
    fq = ops.nvfp4_fake(xt, block=block)
    assert same_bits(f32_from_tensor(fq), qo.nvfp4_fake(x, np.abs(x).max(), block, T))


@pytest.mark.parametrize("name", ["FP8_PER_CHANNEL_PER_TOKEN_CFG", "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG",
                                  "W4A8_AWQ_BETA_CFG", "W4A8_NVFP4_FP8_CFG", "W4A8_MXFP4_FP8_CFG",
                                  "INT4_BLOCKWISE_WEIGHT_ONLY_CFG", "INT8_WEIGHT_ONLY_CFG"])
def test_more_reference_configs_quantize_and_run(mtq, name):
    """Every further configuration of the reference that is made of the built formats converts,
    calibrates and runs; the quantised output stays close to the unquantised one."""
    torch.manual_seed(5)
    model = MLP().to(torch.bfloat16).cuda()
    with torch.no_grad():
        for p in model.parameters():
            p.mul_(0.5)
    x = [torch.randn(32, 128, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    ref = model(x[0]).float()

    def loop(m):
        for b in x:
            m(b)

    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), loop)
    y = model(x[0]).float()
    assert torch.isfinite(y).all()
    rel = (y - ref).abs().mean() / ref.abs().mean()
    assert rel < (0.35 if "W4" in name or "INT4" in name else 0.1), float(rel)


def test_affine_bias_quantization_matches_reference(mtq):
    """Static mean / static mid-range / dynamic bias through TensorQuantizer (calibrate on two
    batches, then quantise) against the reference's CPU results."""
    g = load("bias")
    xs = [torch.from_numpy(g[f"x{i}"]).cuda() for i in range(2)]
    cfgs = {"fp8_mean": dict(num_bits=(4, 3), axis=None, bias={-2: None, -4: None, "type": "static"}),
            "int8_maxmin": dict(num_bits=8, axis=None, bias={-1: None, "type": "static", "method": "max_min"}),
            "int8_dynamic": dict(num_bits=8, axis=None, bias={-2: None, "type": "dynamic"})}
    for tag, kw in cfgs.items():
        q = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(**kw)).cuda()
        q.enable_calib(); q.disable_quant()
        for x in xs:
            q(x)
        q.load_calib_amax()
        if q.bias_type == "static":
            q.load_calib_bias()
            assert np.allclose(q._bias_value.cpu().numpy(), g[f"{tag}_bias"], rtol=1e-6, atol=1e-7), tag
        q.enable_quant(); q.disable_calib()
        assert np.allclose(q._amax.float().cpu().numpy().reshape(-1), g[f"{tag}_amax"], rtol=1e-6), tag
        y = q(xs[1]).cpu().numpy()
        ref = g[f"{tag}_y"]
        # the bias is a mean formed in another summation order: a last-bit difference of the bias can move
        # single elements across a rounding boundary of the quantiser
        assert np.mean(np.abs(y - ref) > 1e-5) < 2e-3 and np.abs(y - ref).max() < 0.1, tag


def test_scaled_e4m3_on_a_non_contiguous_input(mtq):
    """Mirror of TestScaledE4M3.test_e4m3_incontiguous
    (tests/gpu/torch/quantization/test_tensor_quant_cuda.py:129-134 of the reference): a transposed
    view goes in, the result has its logical layout and equals the eager cast element by element."""
    from b200q import tensor_quant

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(4, 4, device="cuda", generator=g).transpose(1, 0)
    assert not x.is_contiguous()
    want = x.to(torch.float8_e4m3fn).to(x.dtype)          # fp8_eager with amax 448: scale 1
    got = tensor_quant.scaled_e4m3(x, None, None, 4, 3)
    assert got.shape == x.shape
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    big = torch.randn(96, 200, device="cuda", generator=g)[:, ::2].t()   # strided and transposed
    amax = big.abs().amax()
    ref = qo.fake_e4m3(big.contiguous().cpu().numpy(), np.float32(amax.item()), "f32")
    assert np.array_equal(tensor_quant.scaled_e4m3(big, amax, None, 4, 3).cpu().numpy(), ref)


def test_fake_quant_backward_is_the_straight_through_estimator(mtq):
    """Mirror of TestScaledE4M3.test_backward (same file, :136-146): without an amax the gradient
    passes through unchanged; with one (and pass_through_bwd=False) it is zeroed where |x| > amax
    (FakeTensorQuantFunction / ScaledE4M3Function backward, tensor_quant.py:293-301)."""
    from b200q import tensor_quant

    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(3, 7, device="cuda", generator=g).requires_grad_()
    labels = torch.randint(6, (3,), device="cuda", generator=g)
    qx = tensor_quant.scaled_e4m3(x, None, None, 4, 3)
    qx.retain_grad()
    torch.nn.CrossEntropyLoss()(qx, labels).backward()
    assert torch.allclose(qx.grad, x.grad)

    amax = torch.tensor(0.7, device="cuda")
    for fn, args in ((tensor_quant.scaled_e4m3, (amax, None, 4, 3)),
                     (tensor_quant.fake_tensor_quant, (amax, None, 8, False, True))):
        y = x.detach().clone().requires_grad_()
        out = fn(y, *args)
        w = torch.arange(1, 22, device="cuda", dtype=torch.float32).reshape(3, 7)
        (out * w).sum().backward()
        inside = (y.detach().abs() <= amax)
        assert bool(inside.any()) and bool((~inside).any())
        assert torch.equal(y.grad, torch.where(inside, w, torch.zeros_like(w)))
