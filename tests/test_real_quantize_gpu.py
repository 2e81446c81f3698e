"""quantize -> compress on the reference's small linear test model, after the reference's own test file
(tests/gpu/torch/quantization/test_real_quantize_cuda.py: real quantisation shrinks the parameters and the
model still runs; save / restore of a compressed model; ``compress`` with a per-layer pattern config).
The reference's convolution models are absent: only linear layers are on this library's path."""
import copy
import fnmatch

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu

CONFIGS = ["INT4_AWQ_CFG", "INT8_DEFAULT_CFG", "FP8_DEFAULT_CFG", "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG",
           "FP8_PER_CHANNEL_PER_TOKEN_CFG"]


class SimpleLinear(nn.Module):
    """16 -> 32 -> 64 -> 16 with ReLUs, as in the reference's tests/_test_utils/torch/quantization/models.py:44."""

    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))

    def forward(self, x):
        return self.net(x)

    @staticmethod
    def get_input():
        return torch.randn(2, 16)


def _config(name):
    import b200q as mtq

    cfg = copy.deepcopy(getattr(mtq, name))
    if name == "INT4_AWQ_CFG":                      # blocks that fit the 16-wide first layer
        cfg["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 16, "scale_bits": 8}
    return cfg


def _quantized(name, seed=0, batches=8):
    import b200q as mtq

    torch.manual_seed(seed)
    model = SimpleLinear().cuda()
    data = [model.get_input().cuda() for _ in range(batches)]
    mtq.quantize(model, _config(name), lambda m: [m(b) for b in data])
    return model, data


def _size(model):
    return sum(p.element_size() * p.nelement() for p in model.parameters())


@pytest.mark.parametrize("name", CONFIGS)
def test_real_quantize_shrinks_the_model_and_it_still_runs(name):
    import b200q as mtq
    from b200q.qtensor import QTensorWrapper

    model, data = _quantized(name)
    with torch.no_grad():
        fake_out = model(data[0])
    before = _size(model)
    mtq.compress(model)
    assert all(isinstance(m.weight, QTensorWrapper) for m in model.net if isinstance(m, nn.Linear))
    if name != "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG":          # 128 x 128 blocks pad these small weights
        assert _size(model) < before
    with torch.no_grad():
        real_out = model(data[0])
    assert real_out.shape == fake_out.shape and torch.isfinite(real_out).all()
    assert torch.allclose(real_out, fake_out, rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize("name", CONFIGS)
def test_save_restore_of_a_compressed_model(name):
    """Reference _test_utils/torch/quantization/quantize_common.py:78-119: the state restores a fresh
    model to the same outputs, and refuses a model that already carries quantisation state."""
    import b200q as mtq

    model, data = _quantized(name, batches=2)
    mtq.compress(model)
    state = mtq.modelopt_state(model)
    torch.manual_seed(1)
    fresh = SimpleLinear().cuda()
    mtq.restore_from_modelopt_state(fresh, state)
    fresh.load_state_dict(model.state_dict())
    with torch.no_grad():
        assert torch.allclose(model(data[0]), fresh(data[0]))
    other, _ = _quantized("FP8_DEFAULT_CFG" if name != "FP8_DEFAULT_CFG" else "INT8_DEFAULT_CFG", batches=2)
    with pytest.raises(AssertionError, match="Model already has modelopt state!"):
        mtq.restore_from_modelopt_state(other, state)


@pytest.mark.parametrize("name", CONFIGS)
def test_compress_config_selects_layers_by_pattern(name):
    import b200q as mtq
    from b200q.qtensor import QTensorWrapper

    patterns = {"*net.0*": False, "*.conv1*": False, "*.fc1*": False, "default": True}
    model, data = _quantized(name)
    mtq.compress(model, config={"compress": patterns})
    seen = {True: 0, False: 0}
    for mod_name, m in model.named_modules():
        if not hasattr(m, "weight_quantizer") or not hasattr(m, "weight"):
            continue
        chosen = patterns["default"]
        for p, v in patterns.items():
            if p != "default" and fnmatch.fnmatch(mod_name, p):
                chosen = v
        assert isinstance(m.weight, QTensorWrapper) == chosen, mod_name
        seen[chosen] += 1
    assert seen == {True: 2, False: 1}
    x = SimpleLinear.get_input().cuda()
    assert model(x).shape[0] == x.shape[0]


# ---- every configuration of the reference's sweep on the small model --------------------------------------
# (tests/gpu/torch/quantization/test_quantize_cuda.py:30-84; the SVDQuant entry is outside this library)

SWEEP = ["INT8_DEFAULT_CFG", "FP8_DEFAULT_CFG", "W4A8_AWQ_BETA_CFG", "INT8_SMOOTHQUANT_CFG",
         "INT4_BLOCKWISE_WEIGHT_ONLY_CFG", "INT4_AWQ_CFG", "INT4_AWQ_CLIP", "INT4_AWQ_FULL", "NVFP4_DEFAULT_CFG",
         "NVFP4_AWQ_LITE_CFG", "NVFP4_AWQ_CLIP_CFG", "NVFP4_AWQ_FULL_CFG", "MXFP8_DEFAULT_CFG", "MXFP6_DEFAULT_CFG",
         "MXFP4_DEFAULT_CFG", "MXINT8_DEFAULT_CFG", "NVFP4_KV_ROTATE_CFG", "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG"]


@pytest.mark.parametrize("name", SWEEP)
def test_quantize_runs_for_every_configuration(name):
    import b200q as mtq

    if name in ("INT4_AWQ_CLIP", "INT4_AWQ_FULL"):          # the reference's test-local variants of INT4_AWQ_CFG
        cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
        cfg["algorithm"] = {"INT4_AWQ_CLIP": "awq_clip", "INT4_AWQ_FULL": "awq_full"}[name]
    else:
        cfg = copy.deepcopy(getattr(mtq, name))
    if name == "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG":
        cfg["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 8, -2: 8}
    torch.manual_seed(3)
    model = SimpleLinear().cuda()
    data = [model.get_input().cuda() for _ in range(8)]
    with torch.no_grad():
        plain = model(data[0])
    mtq.quantize(model, cfg, lambda m: [m(b) for b in data])
    assert all(hasattr(m, "weight_quantizer") for m in model.net if isinstance(m, nn.Linear))
    with torch.no_grad():
        out = model(data[0])
    assert out.shape == plain.shape and torch.isfinite(out).all()
    assert (out - plain).abs().mean() <= 0.5 * plain.abs().mean() + 0.05


@pytest.mark.parametrize("name", ["INT8_SMOOTHQUANT_CFG", "W4A8_AWQ_BETA_CFG"])
def test_save_restore_of_a_fake_quantised_model(name):
    """Reference test_quantize_cuda.py:86-95 (the linear-model rows): also restores into a model built on
    the CPU and moved afterwards."""
    import b200q as mtq

    model, data = _quantized(name, batches=2)
    state = mtq.modelopt_state(model)
    torch.manual_seed(1)
    fresh = SimpleLinear().cuda()
    mtq.restore_from_modelopt_state(fresh, state)
    fresh.load_state_dict(model.state_dict())
    with torch.no_grad():
        want = model(data[0])
        assert torch.allclose(want, fresh(data[0]))
    late = SimpleLinear()
    mtq.restore_from_modelopt_state(late, state)
    late.load_state_dict(model.state_dict())
    late.cuda()
    with torch.no_grad():
        assert torch.allclose(want, late(data[0]))
    if name == "INT8_SMOOTHQUANT_CFG":
        assert all(m.input_quantizer.axis is None for m in fresh.net if isinstance(m, nn.Linear))
