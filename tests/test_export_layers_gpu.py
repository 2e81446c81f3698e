"""Per-layer checkpoint export (weight, weight_scale, weight_scale_2, input_scale, pre_quant_scale)
against the state dict the reference's exporter produced on CPU."""
import copy

import numpy as np
import pytest
import torch

from _util import load, tensor_from_f32, to_f32
from test_api_gpu import MLP, bits_of

pytestmark = pytest.mark.gpu


def _raw(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.int8:
        return t.view(torch.uint8).numpy()
    return bits_of(t)


@pytest.mark.parametrize("tag", ["fp8", "nvfp4", "int8_sq", "int4_awq"])
def test_export_hf_state_dict_matches_reference(tag):
    import b200q as mtq
    from b200q import export

    g = load("export_layers")
    model = MLP().to(torch.bfloat16).cuda()
    with torch.no_grad():
        model.up_proj.weight.copy_(tensor_from_f32(to_f32(g["w_up"], "bf16"), "bf16"))
        model.down_proj.weight.copy_(tensor_from_f32(to_f32(g["w_down"], "bf16"), "bf16"))
    batches = [tensor_from_f32(to_f32(g[f"x{i}"], "bf16"), "bf16") for i in range(2)]
    int4 = copy.deepcopy(mtq.INT4_AWQ_CFG)
    int4["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 32, "type": "static"}
    cfg = {"fp8": mtq.FP8_DEFAULT_CFG, "int8_sq": mtq.INT8_SMOOTHQUANT_CFG, "int4_awq": int4,
           "nvfp4": mtq.NVFP4_DEFAULT_CFG}[tag]

    def loop(m):
        for b in batches:
            m(b)

    mtq.quantize(model, copy.deepcopy(cfg), loop)
    for name in ("up_proj", "down_proj"):
        assert export.get_quantization_format(getattr(model, name)) == str(g[f"{tag}_{name}_format"])
    sd = export.export_hf_state_dict(model, torch.bfloat16)
    assert sorted(sd.keys()) == list(g[f"{tag}_keys"])
    for k, v in sd.items():
        ref = g[f"{tag}_sd_{k}"]
        assert str(v.dtype) == str(g[f"{tag}_dt_{k}"]), k
        assert tuple(v.shape) == ref.shape, k
        got = _raw(v)
        if tag in ("fp8", "nvfp4"):
            # max calibration only: every byte and scale equals the reference's
            assert np.array_equal(got, ref), k
        elif v.dtype in (torch.float32, torch.bfloat16):
            a = v.float().cpu().numpy()
            b = ref if v.dtype == torch.float32 else to_f32(ref, "bf16")
            assert np.allclose(a, b, rtol=2e-2), k
        elif tag == "int8_sq":
            d = np.abs(got.view(np.int8).astype(np.int32) - ref.view(np.int8).astype(np.int32))
            assert d.max() <= 1 and (d != 0).mean() < 0.02, k      # a smoothing-scale bf16 flip moves few codes by one
        else:
            assert got.shape == ref.shape                            # awq: the chosen alpha may be a near-tie
