"""Layers that share their input (q / k / v behind one normalisation layer) made fusable and exported, against
what the reference produced on the CPU (tests/golden/make_golden_model.py, ``golden_export_fusion``:
``preprocess_linear_fusion``, ``fuse_prequant_layernorm``, ``_export_quantized_weight``,
``postprocess_state_dict``).  NVFP4 and FP8 run this library's own calibration first; for the AWQ formats the
block starts from the reference's state after its search (folded weights, pre-quant scales, input amax), so
that the comparison is of the fusion step and not of near-ties between search candidates."""
import copy

import numpy as np
import pytest
import torch
from torch import nn

from _util import load, tensor_from_f32, to_f32
from test_api_gpu import bits_of

pytestmark = pytest.mark.gpu


class SharedInputBlock(nn.Module):
    def __init__(self, hidden=128):
        super().__init__()
        self.input_layernorm = nn.LayerNorm(hidden)
        self.q_proj = nn.Linear(hidden, 128, bias=False)
        self.k_proj = nn.Linear(hidden, 64, bias=False)
        self.v_proj = nn.Linear(hidden, 64, bias=False)

    def forward(self, x):
        h = self.input_layernorm(x)
        return torch.cat([self.q_proj(h), self.k_proj(h), self.v_proj(h)], dim=-1)


def _bf16(g, key):
    return tensor_from_f32(to_f32(g[key], "bf16"), "bf16")


def _raw(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy() if t.dtype == torch.int8 else bits_of(t)


def _block(g):
    model = SharedInputBlock().to(torch.bfloat16).cuda()
    with torch.no_grad():
        for k, p in model.state_dict().items():
            p.copy_(_bf16(g, f"base_{k}").reshape(p.shape))
    return model


@pytest.mark.parametrize("tag", ["nvfp4", "fp8", "int4_awq", "w4a8_awq"])
def test_shared_input_layers_export_like_the_reference(tag):
    import b200q as mtq
    from b200q import export
    from b200q.model_calib import enable_stats_collection, finish_stats_collection

    g = load("export_fusion")
    model = _block(g)
    batches = [_bf16(g, f"x{i}") for i in range(2)]
    int4 = copy.deepcopy(mtq.INT4_AWQ_CFG)
    int4["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 32, "type": "static"}
    cfg = copy.deepcopy({"nvfp4": mtq.NVFP4_DEFAULT_CFG, "fp8": mtq.FP8_DEFAULT_CFG, "int4_awq": int4,
                         "w4a8_awq": mtq.W4A8_AWQ_BETA_CFG}[tag])
    awq = "awq" in tag
    if awq:
        cfg["algorithm"] = "max"

    def loop(m):
        for b in batches:
            m(b)

    mtq.quantize(model, cfg, loop)
    layers = {"q": model.q_proj, "k": model.k_proj, "v": model.v_proj}
    if awq:                                   # the reference's state after its search
        for name, lin in layers.items():
            with torch.no_grad():
                lin.weight.copy_(_bf16(g, f"{tag}_pre_{name}_weight").reshape(lin.weight.shape))
            lin.input_quantizer.pre_quant_scale = _bf16(g, f"{tag}_pre_{name}_pqs").cuda()
            if f"{tag}_pre_{name}_in_amax" in g:
                amax = tensor_from_f32(to_f32(g[f"{tag}_pre_{name}_in_amax"], "f32"), "f32").cuda()
                lin.input_quantizer.amax = amax.reshape(lin.input_quantizer.amax.shape)
            lin.weight_quantizer.reset_amax()
            enable_stats_collection(lin.weight_quantizer)
            lin.weight_quantizer(lin.weight)
            finish_stats_collection(lin.weight_quantizer)
    assert export.get_quantization_format(model.q_proj) == str(g[f"{tag}_format"])
    fused = export.requantize_resmooth_fused_llm_layers(model, batches[0])
    assert fused == ({} if tag == "fp8" else {"q_proj": ["q_proj", "k_proj", "v_proj"]})
    if awq:
        assert all(lin.fused_with_prequant and not hasattr(lin.input_quantizer, "_pre_quant_scale")
                   for lin in layers.values())
    sd = export.export_hf_state_dict(model, torch.bfloat16)
    assert sorted(sd.keys()) == list(g[f"{tag}_keys"])
    if tag != "fp8":                          # one GEMM serves the three: they agree on these
        for key in ("input_scale", "weight_scale_2"):
            if f"q_proj.{key}" in sd:
                assert torch.equal(sd[f"q_proj.{key}"], sd[f"k_proj.{key}"]) and \
                    torch.equal(sd[f"q_proj.{key}"], sd[f"v_proj.{key}"]), key
    for k, v in sd.items():
        ref = g[f"{tag}_sd_{k}"]
        assert str(v.dtype) == str(g[f"{tag}_dt_{k}"]), k
        assert tuple(v.shape) == ref.shape, k
        assert np.array_equal(_raw(v), ref), k
