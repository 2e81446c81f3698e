"""Calibration algorithms on the reference's toy MLP, after the reference's own test file
(tests/unit/torch/quantization/test_calib.py: awq_lite against a direct grid search, the same scales from
one large batch and from several small ones, layer widths that need block padding, smoothquant switched
off and on again, postprocess_amax), with the model and the data on the GPU."""
import copy

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


class SimpleMLP(nn.Module):
    def __init__(self, fi=16, f1=32, f2=16, fo=16):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(fi, f1, bias=False), nn.ReLU(), nn.Linear(f1, f2, bias=False), nn.ReLU(),
                                 nn.Linear(f2, fo, bias=False))

    def forward(self, x):
        return self.net(x)


def _awq_config(mtq, method, block=8):
    cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
    cfg["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: block}
    cfg["algorithm"]["method"] = method
    cfg["algorithm"]["debug"] = True
    if method == "awq_clip":
        cfg["algorithm"].pop("alpha_step", None)
    return cfg


def _data(n, *shape, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn(*shape, generator=g, device="cuda") for _ in range(n)]


def _pair(seed=0, **kw):
    torch.manual_seed(seed)
    a = SimpleMLP(**kw).cuda()
    b = SimpleMLP(**kw).cuda()
    b.load_state_dict(a.state_dict())
    return a, b


def _grid_search(mtq, linear, x, alphas, block):
    """The search written out directly: per candidate, scale the weight's input channels, fake-quantise in
    blocks, divide the scale back out, and compare the layer's output with the unquantised one."""
    w = linear.weight.detach()
    quantizer = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=4, block_sizes={-1: block})).cuda()
    blocks = w.reshape(-1, block)
    w_mean = (blocks.abs() / blocks.abs().amax(dim=1, keepdim=True)).reshape(w.shape).mean(0)
    x_mean = x.abs().reshape(-1, x.shape[-1]).mean(0)
    want = x @ w.t()
    best = (float("inf"), None)
    for alpha in alphas:
        s = (x_mean.pow(alpha) / w_mean.pow(1 - alpha)).clamp(min=1e-4, max=1e4)
        s = s / (s.max() * s.min()).sqrt()
        wq = quantizer(w * s[None, :]) / s[None, :]
        loss = ((x @ wq.t()) - want).float().pow(2).mean().item()
        if loss < best[0]:
            best = (loss, s)
    return best[1]


def test_awq_lite_equals_a_direct_grid_search(mtq):
    model, plain = _pair()
    data = _data(1, 2, 64, 16)
    mtq.quantize(model, _awq_config(mtq, "awq_lite"), lambda m: [m(b) for b in data])
    x = data[0].clone()
    for i, layer in enumerate(plain.net):
        if isinstance(layer, nn.Linear):
            alphas = [float(k) for k in model.net[i].awq_lite.loss]
            assert len(alphas) == 11
            want = _grid_search(mtq, layer, x, alphas, 8)
            assert torch.allclose(model.net[i].awq_lite.best_scale, want, rtol=1e-5, atol=1e-7), i
        x = layer(x)
    with torch.no_grad():
        assert torch.isfinite(model(data[0])).all()


def test_awq_full_one_large_batch_or_several_small_ones(mtq):
    small = _data(4, 2, 16, 16, seed=1)
    large = [torch.cat(small, dim=0)]
    model_s, model_m = _pair(seed=1)
    mtq.quantize(model_s, _awq_config(mtq, "awq_full"), lambda m: [m(b) for b in large])
    mtq.quantize(model_m, _awq_config(mtq, "awq_full"), lambda m: [m(b) for b in small])
    for i in (0, 2, 4):
        assert torch.allclose(model_s.net[i].awq_lite.best_scale, model_m.net[i].awq_lite.best_scale), i


def test_awq_full_with_widths_that_need_padding(mtq):
    torch.manual_seed(2)
    model = SimpleMLP(f1=13, f2=19).cuda()
    data = _data(2, 2, 16, 16, seed=2)
    mtq.quantize(model, _awq_config(mtq, "awq_full"), lambda m: m(data[0]))
    assert torch.isfinite(model(data[1])).all()


def test_smoothquant_switched_off_and_on_again(mtq):
    from b200q.model_calib import apply_pre_quant_scale_and_smooth, disable_pre_quant_scale_and_resmooth

    model, model_no_sq = _pair(seed=1234)
    cal, (x,) = _data(1, 2, 16, 16, seed=3), _data(1, 2, 16, 16, seed=4)
    mtq.quantize(model, copy.deepcopy(mtq.INT8_SMOOTHQUANT_CFG), lambda m: [m(b) for b in cal])
    mtq.quantize(model_no_sq, copy.deepcopy(mtq.INT8_DEFAULT_CFG), lambda m: [m(b) for b in cal])
    with torch.no_grad():
        out_sq = model(x)
        for m in model.modules():
            if isinstance(m, nn.Linear):
                disable_pre_quant_scale_and_resmooth(m)
                assert m.input_quantizer.pre_quant_scale is None
        assert torch.allclose(model(x), model_no_sq(x), rtol=1e-4, atol=1e-5)
        for m in model.modules():
            if isinstance(m, nn.Linear):
                apply_pre_quant_scale_and_smooth(m)
                assert m.input_quantizer.pre_quant_scale is not None
        assert torch.allclose(model(x), out_sq, rtol=1e-4, atol=1e-5)


def test_postprocess_amax(mtq):
    torch.manual_seed(5)
    model = SimpleMLP().cuda()
    data = _data(1, 2, 16, 16, seed=5)
    mtq.quantize(model, copy.deepcopy(mtq.INT8_DEFAULT_CFG), lambda m: m(data[0]))
    before = {n: m.amax.clone() for n, m in model.named_modules()
              if isinstance(m, mtq.nn.TensorQuantizer) and m.amax is not None}
    mtq.postprocess_amax(model, "*input_quantizer", lambda amax: torch.clamp(amax, max=0.5))
    touched = 0
    for n, m in model.named_modules():
        if isinstance(m, mtq.nn.TensorQuantizer) and m.amax is not None:
            if n.endswith("input_quantizer"):
                assert m.amax.amax() <= 0.5
                touched += 1
            else:
                assert torch.equal(m.amax, before[n])
    assert touched == 3
