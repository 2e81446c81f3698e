"""The reference's export-helper tests (tests/gpu/torch/export/test_export.py) on this library: the format a
quantised model reports, weight block sizes, scaling factors from weights and from quantisers, the common
amax of q / k / v projections, and the state-dict post-processing with KV-cache scales.  Same toy models,
configurations and known answers; rows for formats outside this library's path (KV-cache dtype of attention
plugins, per-layer configuration records of the TensorRT-LLM exporter) are absent."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


@pytest.fixture(scope="module")
def export():
    from b200q import export

    return export


class ToyModel(nn.Module):
    def __init__(self, dims=(10, 10, 10, 10)):
        super().__init__()
        self.linears = nn.Sequential(*(nn.Linear(dims[i], dims[i + 1]) for i in range(len(dims) - 1)))

    def forward(self, x):
        return self.linears(x)


class SmallLinearModelwithCustomWeight(nn.Module):
    def __init__(self, weights):
        super().__init__()
        for name, w in zip(("q_proj", "k_proj", "v_proj", "o_proj"), weights):
            layer = nn.Linear(w.shape[1], w.shape[0], bias=False)
            with torch.no_grad():
                layer.weight.copy_(w)
            setattr(self, name, layer)

    def forward(self, x):
        return self.o_proj(self.v_proj(self.k_proj(self.q_proj(x))))


_NVFP4 = {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, "axis": None}
partial_fp8_config = {"quant_cfg": {"*.1.weight_quantizer": {"num_bits": (4, 3), "axis": None},
                                    "*.1.input_quantizer": {"num_bits": (4, 3), "axis": None},
                                    "default": {"num_bits": 8, "enable": False}}, "algorithm": "max"}
partial_w4a8_config = {
    "quant_cfg": {"*.2.weight_quantizer": [{"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                                           {"num_bits": (4, 3), "axis": None, "enable": True}],
                  "*.2.input_quantizer": {"num_bits": (4, 3), "axis": None, "enable": True},
                  "default": {"num_bits": 8, "enable": False}}, "algorithm": "awq_lite"}
partial_nvfp4_config = {"quant_cfg": {"*.1.weight_quantizer": dict(_NVFP4, enable=True),
                                      "*.1.input_quantizer": dict(_NVFP4, enable=True),
                                      "default": {"enable": False}}, "algorithm": "max"}
partial_nvfp4_awq_config = {"quant_cfg": {"*.2.weight_quantizer": dict(_NVFP4, enable=True),
                                          "*.2.input_quantizer": dict(_NVFP4, enable=True),
                                          "*.1.weight_quantizer": dict(_NVFP4, enable=False),
                                          "*.1.input_quantizer": dict(_NVFP4, enable=False),
                                          "default": {"enable": False}}, "algorithm": "awq_lite"}
partial_int4_awq_config = {
    "quant_cfg": {"*.2.weight_quantizer": {"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                  "*.2.input_quantizer": {"enable": False}, "default": {"enable": False}},
    "algorithm": {"method": "awq_lite", "alpha_step": 0.1}}


def _only(which):
    return {"quant_cfg": {f"*{name}_quantizer": {"num_bits": (4, 3), "axis": None, "enable": name == which}
                          for name in ("weight", "input", "output")} | {"default": {"enable": False}},
            "algorithm": "max"}


def _toy(mtq, config):
    torch.manual_seed(0)
    model = ToyModel().cuda()
    mtq.quantize(model, config, lambda m: m(torch.randn(1, 4, 10, device="cuda")))
    return model


@pytest.mark.parametrize(("config", "expected"), [
    (partial_fp8_config, "fp8"), (partial_w4a8_config, "w4a8_awq"), (partial_nvfp4_config, "nvfp4"),
    (partial_nvfp4_awq_config, "nvfp4_awq"), (partial_int4_awq_config, "int4_awq")])
def test_get_quantization_format(mtq, export, config, expected):
    """Reference test_export.py:68-81."""
    assert export.get_quantization_format(_toy(mtq, config)) == expected


@pytest.mark.parametrize(("weight", "group_size", "expected"), [
    ([[0.0, 0.35, 0.28, 7.0], [0.49, 0.84, -0.77, 0.07]], 2, [[0.05, 1.0], [0.12, 0.11]]),
    ([[0.127, 0.0, 1.27, -12.7], [0.0, 127.0, 0.254, 2.54]], 0, [0.1, 1.0]),
    ([[0.0, 0.0, 0.0, 0.0], [0.0, -0.127, 0.254, 2.54]], 0, [1.0, 0.02]),            # zero replaced with 1.0
    ([[0.0, 0.84, -0.77, 0.07], [0.0, 0.0, 0.0, 0.0]], 2, [[0.12, 0.11], [1.0, 1.0]])])
def test_get_scaling_factor_from_weight(export, weight, group_size, expected):
    """Reference test_export.py:163-196, exact as there: fp32 amax / 7 per group, amax / 127 per row."""
    weight = torch.tensor(weight, device="cuda")
    got = export.get_scaling_factor_from_weight(weight, group_size)
    assert list(got.shape) == ([2, 4 // group_size] if group_size else [2])
    assert torch.equal(got.cpu(), torch.tensor(expected))


_QKVO = ([[0.1, 0.3], [0.22, 0.45]], [[0.44, 0.32], [0.11, 0.95]], [[0.9, 0.03], [0.92, 0.8]],
         [[0.01, 0.97], [0.29, 0.77]])


@pytest.mark.parametrize("negate", [False, True])
@pytest.mark.parametrize("config_name", ["FP8_DEFAULT_CFG", "NVFP4_DEFAULT_CFG"])
def test_adjust_attn_amax_values(mtq, export, config_name, negate):
    """Reference test_export.py:277-320: q, k and v end with their common maximum, o keeps its own."""
    weights = [torch.tensor(w) for w in _QKVO]
    if negate:
        weights[1][1, 1] *= -1
        weights[3][0, 1] *= -1
    model = SmallLinearModelwithCustomWeight(weights).cuda()
    mtq.quantize(model, getattr(mtq, config_name), lambda m: m(torch.randn(1, 4, 2, device="cuda")))
    export.adjust_attn_amax_values(model)
    for layer in (model.q_proj, model.k_proj, model.v_proj):
        assert layer.weight_quantizer.amax.item() == pytest.approx(0.95, rel=1e-6)
    assert model.o_proj.weight_quantizer.amax.item() == pytest.approx(0.97, rel=1e-6)


@pytest.mark.parametrize(("config", "expected"), [
    ("FP8_DEFAULT_CFG", 0), ("INT8_WEIGHT_ONLY_CFG", 0), ("INT8_SMOOTHQUANT_CFG", 0), ("NVFP4_DEFAULT_CFG", 16),
    ("NVFP4_AWQ_LITE_CFG", 16), ("W4A8_AWQ_BETA_CFG", 128), ("INT4_AWQ_CFG", 128), (partial_nvfp4_config, 16)])
def test_get_weight_block_size(mtq, export, config, expected):
    """Reference test_export.py:323-352."""
    model = _toy(mtq, getattr(mtq, config) if isinstance(config, str) else config)
    for module in model.modules():
        size = export.get_weight_block_size(module)
        wq = getattr(module, "weight_quantizer", None)
        if wq is not None and (isinstance(wq, mtq.nn.SequentialQuantizer) or wq.is_enabled):
            assert size == expected
        else:
            assert size == 0


@pytest.mark.parametrize(("which", "expected_amax"), [
    ("weight", [0.45, 0.95, 0.92, 0.97]), ("input", [1.0, 0.67, 0.68, 0.9]), ("output", [0.67, 0.68, 0.9, 0.88])])
def test_get_scaling_factor(mtq, export, which, expected_amax):
    """Reference test_export.py:355-390: amax / 448 of every enabled quantiser, in module order."""
    model = SmallLinearModelwithCustomWeight([torch.tensor(w) for w in _QKVO]).cuda()
    mtq.quantize(model, _only(which), lambda m: m(torch.ones(1, 2, 2, device="cuda")))
    expected = list(expected_amax)
    for module in model.modules():
        if isinstance(module, mtq.nn.TensorQuantizer) and module.is_enabled:
            scale = export.get_scaling_factor(module)
            want = torch.tensor(expected.pop(0) / 448, dtype=scale.dtype, device=scale.device)
            assert torch.allclose(scale, want, rtol=1e-3, atol=1e-3)
    assert not expected


def _quantised_toy(mtq, dims, config):
    torch.manual_seed(0)
    model = ToyModel(dims).cuda()
    mtq.quantize(model, config, lambda m: m(torch.randn(1, 4, dims[0], device="cuda")))
    return model


def test_export_per_tensor_quantized_weight(mtq, export):
    """Reference tests/unit/torch/export/test_export_weight.py:49-78: a layer whose quantisers are off is
    left alone; an FP8 layer gets E4M3 weights, ``weight_scale`` and ``input_scale``, no second scale."""
    model = _quantised_toy(mtq, (32, 256, 32, 128), partial_fp8_config)
    untouched, fp8 = model.linears[0], model.linears[1]
    export.export_quantized_weight(untouched, torch.float32)
    assert untouched.weight.dtype == torch.float32
    assert not untouched.weight_quantizer.is_enabled and not untouched.input_quantizer.is_enabled
    assert not untouched.output_quantizer.is_enabled
    for name in ("weight_scale", "weight_scale_2", "input_scale", "output_scale"):
        assert not hasattr(untouched, name), name
    export.export_quantized_weight(fp8, torch.float32)
    assert fp8.weight.dtype == torch.float8_e4m3fn
    assert hasattr(fp8, "weight_scale") and hasattr(fp8, "input_scale")
    assert not hasattr(fp8, "weight_scale_2") and not hasattr(fp8, "output_scale")
    assert hasattr(fp8, "weight_quantizer") and hasattr(fp8, "input_quantizer")
    assert not fp8.output_quantizer.is_enabled


def test_export_per_block_quantized_weight(mtq, export):
    """Reference tests/unit/torch/export/test_export_weight.py:81-98 (and its GPU twin): a W4A8 layer gets
    packed uint8 weights, both weight scales and the input scale."""
    model = _quantised_toy(mtq, (32, 256, 256, 32), partial_w4a8_config)
    layer = model.linears[2]
    export.export_quantized_weight(layer, torch.float32)
    assert layer.weight.dtype == torch.uint8
    for name in ("weight_quantizer", "weight_scale", "weight_scale_2", "input_scale", "input_quantizer"):
        assert hasattr(layer, name), name
    assert not layer.output_quantizer.is_enabled and not hasattr(layer, "output_scale")


@pytest.mark.parametrize(("output_bits", "expected"), [((4, 3), "FP8"), (8, "INT8")])
def test_get_kv_cache_dtype(mtq, export, output_bits, expected):
    """Reference test_export.py:256-274: the cache format is read off the enabled output quantisers."""
    config = {"quant_cfg": {"*.1.weight_quantizer": {"num_bits": (4, 3), "axis": None},
                            "*.1.input_quantizer": {"num_bits": (4, 3), "axis": None},
                            "*output_quantizer": {"num_bits": output_bits, "axis": None, "enable": True},
                            "default": {"enable": False}}, "algorithm": "max"}
    model = _toy(mtq, config)
    assert export.get_kv_cache_dtype(list(model.modules())) == expected
    assert export.get_kv_cache_dtype(_toy(mtq, partial_fp8_config)) is None


def test_get_kv_cache_scaling_factor(mtq, export):
    """Scales of the key / value quantisers of an attention module: amax / 448, at least 1 for an FP8 cache
    (reference modelopt/torch/export/quant_utils.py:348-370)."""
    from b200q.config import QuantizerAttributeConfig

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.k_bmm_quantizer = mtq.nn.TensorQuantizer(QuantizerAttributeConfig(num_bits=(4, 3), axis=None))
            self.v_bmm_quantizer = mtq.nn.TensorQuantizer(QuantizerAttributeConfig(num_bits=(4, 3), axis=None))

    attention = Attention().cuda()
    attention.k_bmm_quantizer.amax = torch.tensor(0.128, device="cuda")
    attention.v_bmm_quantizer.amax = torch.tensor(896.0, device="cuda")
    k, v = export.get_kv_cache_scaling_factor(attention)
    assert k.item() == 1.0 and v.item() == 2.0
    assert export.get_kv_cache_scaling_factor(nn.Linear(2, 2)) == [None, None]
    assert export.get_kv_cache_bias(attention) == [None, None]


@pytest.mark.parametrize("quantization", ["fp8", "int8_sq", "int8_wo"])
def test_from_quantized_weight_undoes_to_quantized_weight(export, quantization):
    """Reference modelopt/torch/export/quant_utils.py:741-857: packing then unpacking returns every weight to
    within half a quantisation step (an eighth of the value for E4M3's three mantissa bits)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    weight = torch.randn(64, 128, device="cuda", generator=g, dtype=torch.float32)
    if quantization == "fp8":
        scale = (weight.abs().max() / 448.0).reshape(1)
        tolerance = (weight.abs() / 16 + scale * 2.0 ** -10) * (1 + 1e-5)
    else:
        scale = weight.abs().amax(dim=1) / 127.0
        tolerance = (scale / 2)[:, None] * (1 + 1e-6)
    packed = export.to_quantized_weight(weight, scale, quantization)
    assert packed.element_size() == 1
    back = export.from_quantized_weight(packed, scale, quantization, torch.float32)
    assert back.dtype == torch.float32 and bool(((back - weight).abs() <= tolerance).all())
    assert export.from_quantized_weight(weight, None, quantization, torch.bfloat16).dtype == torch.bfloat16


def _kv_config(output_bits):
    return {"quant_cfg": {"*.1.weight_quantizer": {"num_bits": (4, 3), "axis": None},
                          "*.1.input_quantizer": {"num_bits": (4, 3), "axis": None},
                          "*output_quantizer": {"num_bits": output_bits, "axis": None, "enable": True},
                          "default": {"enable": False}}, "algorithm": "max"}


@pytest.mark.parametrize(("config", "expected"), [
    (partial_fp8_config, {"exclude_modules": ["linears.0", "linears.2"], "kv_cache_quant_algo": None, "quant_algo": "FP8"}),
    (partial_w4a8_config, {"exclude_modules": ["linears.0", "linears.1"], "group_size": 128, "has_zero_point": False,
                           "kv_cache_quant_algo": None, "pre_quant_scale": True, "quant_algo": "W4A8_AWQ"}),
    (partial_nvfp4_config, {"exclude_modules": ["linears.0", "linears.2"], "group_size": 16,
                            "kv_cache_quant_algo": None, "quant_algo": "NVFP4"}),
    (partial_nvfp4_awq_config, {"exclude_modules": ["linears.0", "linears.1"], "group_size": 16, "has_zero_point": False,
                                "pre_quant_scale": True, "kv_cache_quant_algo": None, "quant_algo": "NVFP4_AWQ"}),
    (partial_int4_awq_config, {"exclude_modules": ["linears.0", "linears.1"], "group_size": 128, "has_zero_point": False,
                               "kv_cache_quant_algo": None, "pre_quant_scale": True, "quant_algo": "W4A16_AWQ"}),
    (_kv_config((4, 3)), {"exclude_modules": ["linears.0", "linears.2"], "quant_algo": "FP8", "kv_cache_quant_algo": "FP8"}),
    (_kv_config(8), {"exclude_modules": ["linears.0", "linears.2"], "quant_algo": "FP8", "kv_cache_quant_algo": "INT8"})])
def test_get_quant_config(mtq, export, config, expected):
    """Reference test_export.py:393-466: the quantisation record written beside an exported checkpoint."""
    assert export.get_quant_config(_toy(mtq, config))["quantization"] == expected
