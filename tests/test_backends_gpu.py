"""The real-quantisation GEMM backends, after the reference's own test file
(tests/gpu/torch/quantization/backends/test_gemm_common.py): ``Nvfp4Linear.apply`` and
``Fp8PerTensorLinear.apply`` on 2-D and 3-D inputs with the bias absent, given by keyword and given by
position; gradients to the input and the bias through a compressed model; and dynamic against calibrated
scales, fake-quantised against compressed models.  fp16 models, as in the reference."""
import copy

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu

CASES = {"nvfp4": ("NVFP4_DEFAULT_CFG", "Nvfp4Linear"), "fp8": ("FP8_DEFAULT_CFG", "Fp8PerTensorLinear")}


class OneLayerLinear(nn.Module):
    def __init__(self, in_features=64, out_features=32):
        super().__init__()
        self.in_features = in_features
        self.net = nn.Sequential(nn.Linear(in_features, out_features))

    def forward(self, x):
        return self.net(x)

    def get_input(self, batch_size=2):
        return torch.randn(batch_size, self.in_features)


class SimpleLinear(nn.Module):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))

    def forward(self, x):
        return self.net(x)

    def get_input(self):
        return torch.randn(2, 16)


def _case(which):
    import importlib

    import b200q as mtq

    cfg_name, fn = CASES[which]
    module = importlib.import_module("b200q.backends." + ("nvfp4_gemm" if which == "nvfp4" else "fp8_per_tensor_gemm"))
    return mtq, copy.deepcopy(getattr(mtq, cfg_name)), getattr(module, fn).apply


@pytest.mark.parametrize(("which", "atol", "rtol"), [("nvfp4", 0.5, 0.1), ("fp8", 0.05, 0.1)])
@pytest.mark.parametrize("input_dim", [2, 3])
def test_gemm_with_and_without_bias(which, atol, rtol, input_dim):
    mtq, cfg, gemm = _case(which)
    torch.manual_seed(42)              # the reference's seed: weights and inputs come from the CPU generator
    model = OneLayerLinear().half().cuda()
    data = [model.get_input().half().cuda() for _ in range(8)]
    mtq.quantize(model, cfg, lambda m: [m(b) for b in data])
    module = model.net[0]
    x = data[0].clone() if input_dim == 2 else data[0].reshape(1, *data[0].shape)
    want = nn.functional.linear(x, module.weight)
    got = gemm(module, x, module.weight)
    assert got.shape == want.shape and torch.allclose(got, want, atol=atol, rtol=rtol), (got - want).abs().max()
    bias = torch.randn(module.weight.shape[0], device="cuda", dtype=torch.float16)
    want = nn.functional.linear(x, module.weight, bias)
    by_keyword = gemm(module, x, module.weight, bias=bias)
    by_position = gemm(module, x, module.weight, bias)
    assert torch.allclose(by_keyword, want, atol=atol, rtol=rtol)
    assert torch.equal(by_keyword, by_position)


def _grads(model, x):
    out = model(x).sum()
    model.zero_grad()
    out.backward()
    layers = [m for m in model.net if isinstance(m, nn.Linear)]
    return [m.weight.grad for m in layers], [m.bias.grad for m in layers]


@pytest.mark.parametrize(("which", "atol_bias", "atol_input"), [("nvfp4", 0.5, 0.2), ("fp8", 0.02, 0.02)])
def test_gradients_through_a_compressed_model(which, atol_bias, atol_input):
    mtq, cfg, _ = _case(which)
    # the reference's weights and inputs (CPU generator, seed 42): its two models are built one after the
    # other when the test module loads, the input and the calibration batches after a re-seed
    torch.manual_seed(42)
    model = [SimpleLinear(), SimpleLinear()][("nvfp4", "fp8").index(which)].half().cuda()
    torch.manual_seed(42)
    x = model.get_input().half().cuda().requires_grad_(True)
    data = [model.get_input().half().cuda() for _ in range(8)]
    mtq.quantize(model, cfg, lambda m: [m(b) for b in data])
    _, bias_grads = _grads(model, x)
    input_grad, x.grad = x.grad, None
    mtq.compress(model)
    weight_grads_q, bias_grads_q = _grads(model, x)
    assert all(g is None for g in weight_grads_q)                  # packed weights take no gradient
    for a, b in zip(bias_grads, bias_grads_q):
        assert torch.allclose(a, b, atol=atol_bias)
    assert torch.allclose(input_grad, x.grad, atol=atol_input)


@pytest.mark.parametrize(("which", "atol", "rtol"), [("nvfp4", 0.3, 0.1), ("fp8", 0.1, 0.1)])
def test_dynamic_and_calibrated_scales_fake_and_compressed(which, atol, rtol):
    mtq, cfg, gemm = _case(which)
    torch.manual_seed(2)
    plain = OneLayerLinear().half().cuda()
    data = [plain.get_input().half().cuda() for _ in range(8)]
    dynamic = copy.deepcopy(plain)
    mtq.quantize(dynamic, copy.deepcopy(cfg))                      # no forward loop: input amax stays dynamic
    dynamic_c = copy.deepcopy(dynamic)
    mtq.compress(dynamic_c)
    calibrated = copy.deepcopy(plain)
    mtq.quantize(calibrated, copy.deepcopy(cfg), lambda m: [m(b) for b in data])
    calibrated_c = copy.deepcopy(calibrated)
    mtq.compress(calibrated_c)
    with torch.no_grad():
        for x in data:
            want = plain(x)
            for fake, packed in ((dynamic, dynamic_c), (calibrated, calibrated_c)):
                module = fake.net[0]
                through_gemm = gemm(module, x, module.weight, bias=module.bias)
                assert torch.allclose(want, through_gemm, atol=atol, rtol=rtol)
                assert torch.allclose(through_gemm, fake(x), atol=atol / 2)
                assert torch.allclose(through_gemm, packed(x), atol=atol / 2)


def test_compress_switches_the_gemm_on(tmp_path):
    """Reference backends/test_gemm_registry.py:107-131 and compress.py:124-128."""
    import b200q as mtq

    def quantized():
        torch.manual_seed(3)
        model = SimpleLinear().cuda()
        data = [model.get_input().cuda() for _ in range(8)]
        mtq.quantize(model, copy.deepcopy(mtq.FP8_DEFAULT_CFG), lambda m: [m(b) for b in data])
        return model

    packed, fake, off = quantized(), quantized(), quantized()
    assert not hasattr(packed.net[0], "_use_real_quant_gemm")
    mtq.compress(packed)
    assert packed.net[0]._use_real_quant_gemm is True
    assert not hasattr(fake.net[0], "_use_real_quant_gemm")
    mtq.compress(off, config={"quant_gemm": False})
    assert not getattr(off.net[0], "_use_real_quant_gemm", False)
    from b200q import backends
    backends.enable_real_quant_gemm(fake)
    assert fake.net[0]._use_real_quant_gemm is True
    backends.disable_real_quant_gemm(fake)
    assert fake.net[0]._use_real_quant_gemm is False


def _calibrated_and_compressed(mtq, model, config, calib_data):
    def forward_loop(m):
        for batch in calib_data:
            m(batch)

    mtq.quantize(model, config, forward_loop)
    fake = model(calib_data[0].clone())
    mtq.compress(model)
    return fake


def test_nvfp4_compressed_forward_stays_close_to_the_fake_quantised_one():
    """Reference tests/gpu/torch/quantization/backends/test_nvfp4_gemm.py:77-101 (its tolerance)."""
    mtq, config, _ = _case("nvfp4")
    torch.manual_seed(0)
    model = OneLayerLinear(64, 32).to(torch.float16).cuda()
    calib_data = [model.get_input(2).to(torch.float16).cuda() for _ in range(8)]
    fake = _calibrated_and_compressed(mtq, model, config, calib_data)
    real = model(calib_data[0].clone())
    assert torch.allclose(fake, real, atol=0.2), float((fake - real).abs().max())


@pytest.mark.parametrize("which", ["fp8", "nvfp4"])
def test_the_registry_finds_the_gemm_of_a_compressed_layer(which):
    """Reference tests/gpu/torch/quantization/backends/test_fp8_per_tensor_gemm.py:29-52, and the same for
    NVFP4: the first layer of a compressed model matches its format's GEMM."""
    from b200q.backends import gemm_registry

    mtq, config, apply = _case(which)
    torch.manual_seed(0)
    model = (SimpleLinear() if which == "fp8" else OneLayerLinear(64, 32)).to(torch.float16).cuda()
    calib_data = [model.get_input().to(torch.float16).cuda() for _ in range(8)]
    _calibrated_and_compressed(mtq, model, config, calib_data)
    assert gemm_registry.find_match(model.net[0], calib_data[0].clone(), [], {}) == apply
