"""Model-level golden vectors: run the REFERENCE's mtq.quantize / mtq.compress on CPU for a small
MLP and store what it produced (amax buffers, AWQ losses and scales, packed weights).

    python tests/golden/make_golden_model.py --ref /path/to/TensorRT-Model-Optimizer

Uses the same import shims as make_golden.py.
"""
from __future__ import annotations

import argparse
import copy
import sys
from pathlib import Path

import numpy as np
import torch
from torch import nn

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_golden import bits, import_reference  # noqa: E402


class MLP(nn.Module):
    """Llama-style MLP names so that the wildcard patterns behave as on a real model."""

    def __init__(self, hidden=128, inter=256):
        super().__init__()
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.up_proj(x)))


def make_model(seed, dtype, hidden=128, inter=256):
    torch.manual_seed(seed)
    m = MLP(hidden, inter)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn_like(p) * 0.05)
    return m.to(dtype)


def make_batches(seed, n, dtype, hidden=128, tokens=48):
    g = torch.Generator().manual_seed(seed)
    mag = torch.exp(torch.randn(hidden, generator=g))
    return [(torch.randn(tokens, hidden, generator=g) * mag).to(dtype) for _ in range(n)]


def golden_awq(mtq, out, fixture="awq", hidden=128, inter=256, tokens=48):
    """awq_lite through the reference.  ``awq`` is the 128 -> 256 -> 128 MLP with 48 tokens per batch;
    ``awq128`` (hidden 256, intermediate 512, 128 tokens per batch) has token counts and channel counts
    that are multiples of 128."""
    cases = {}
    for tag, dtype in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        model = make_model(11, dtype, hidden, inter)
        batches = make_batches(12, 2, dtype, hidden, tokens)
        cases[f"{tag}_w_up"] = bits(model.up_proj.weight)
        cases[f"{tag}_w_down"] = bits(model.down_proj.weight)
        for i, b in enumerate(batches):
            cases[f"{tag}_x{i}"] = bits(b)
        cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
        cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.05, "debug": True}

        def loop(m):
            for b in batches:
                m(b)

        mtq.quantize(model, cfg, loop)
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            st = lin.awq_lite
            cases[f"{tag}_{name}_alphas"] = np.array(list(st.loss.keys()), dtype=np.float64)
            cases[f"{tag}_{name}_losses"] = np.array([float(v) for v in st.loss.values()], dtype=np.float64)
            cases[f"{tag}_{name}_best_alpha"] = np.array(st.best_alpha, dtype=np.float64)
            cases[f"{tag}_{name}_best_scale"] = st.best_scale.float().numpy()
            cases[f"{tag}_{name}_act_scale"] = st.act_scale.float().numpy()
            cases[f"{tag}_{name}_weight_scale"] = st.weight_scale.float().numpy()
            cases[f"{tag}_{name}_pqs"] = bits(lin.input_quantizer._pre_quant_scale)
            cases[f"{tag}_{name}_w_folded"] = bits(lin.weight)
            cases[f"{tag}_{name}_w_amax"] = bits(lin.weight_quantizer._amax)
        y = model(batches[0])
        cases[f"{tag}_y_fake"] = bits(y)
    np.savez_compressed(out / f"{fixture}.npz", **cases)


def golden_flows(mtq, out):
    """INT8 / FP8 / NVFP4 max calibration: the amax buffers the reference ends up with, and the
    packed weights of mtq.compress for NVFP4."""
    cases = {}
    dtype = torch.bfloat16
    batches = make_batches(22, 3, dtype)
    for i, b in enumerate(batches):
        cases[f"x{i}"] = bits(b)
    base = make_model(21, dtype)
    cases["w_up"] = bits(base.up_proj.weight)
    cases["w_down"] = bits(base.down_proj.weight)

    def loop(m):
        for b in batches:
            m(b)

    for tag, cfg in (("int8", mtq.INT8_DEFAULT_CFG), ("fp8", mtq.FP8_DEFAULT_CFG), ("nvfp4", mtq.NVFP4_DEFAULT_CFG)):
        model = copy.deepcopy(base)
        mtq.quantize(model, copy.deepcopy(cfg), loop)
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            cases[f"{tag}_{name}_in_amax"] = bits(lin.input_quantizer._amax.float().reshape(-1))
            cases[f"{tag}_{name}_w_amax"] = bits(lin.weight_quantizer._amax.float().reshape(-1))
        if tag != "nvfp4":  # the reference has no CPU kernel for NVFP4 fake quant
            cases[f"{tag}_y"] = bits(model(batches[0]))
        else:
            mtq.compress(model)
            for name in ("up_proj", "down_proj"):
                lin = getattr(model, name)
                cases[f"nvfp4_{name}_packed"] = bits(lin.weight.data)
                cases[f"nvfp4_{name}_scale"] = bits(lin.weight_quantizer._scale)
                cases[f"nvfp4_{name}_double_scale"] = bits(lin.weight_quantizer._double_scale.reshape(1))
            cases["nvfp4_state_keys"] = np.array(sorted(model.state_dict().keys()))
    for tag, cfg in (("int8", mtq.INT8_DEFAULT_CFG), ("fp8", mtq.FP8_DEFAULT_CFG)):
        model = copy.deepcopy(base)
        c = copy.deepcopy(cfg)
        c["algorithm"] = "mse"
        mtq.quantize(model, c, loop)
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            cases[f"{tag}_mse_{name}_in_amax"] = bits(lin.input_quantizer._amax.float().reshape(-1))
            cases[f"{tag}_mse_{name}_w_amax"] = bits(lin.weight_quantizer._amax.float().reshape(-1))
    np.savez_compressed(out / "flows.npz", **cases)


def golden_export_layers(mtq, out):
    """Per-layer checkpoint export of the reference (_export_quantized_weight + postprocess_state_dict)
    after mtq.quantize, for FP8, INT8 SmoothQuant, INT4 AWQ and NVFP4."""
    from modelopt.torch.export.quant_utils import get_quantization_format, postprocess_state_dict
    from modelopt.torch.export.unified_export_hf import _export_quantized_weight

    cases = {}
    dtype = torch.bfloat16
    batches = make_batches(42, 2, dtype)
    for i, b in enumerate(batches):
        cases[f"x{i}"] = bits(b)
    base = make_model(41, dtype)
    cases["w_up"] = bits(base.up_proj.weight)
    cases["w_down"] = bits(base.down_proj.weight)

    def loop(m):
        for b in batches:
            m(b)

    int4 = copy.deepcopy(mtq.INT4_AWQ_CFG)
    int4["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 32, "type": "static"}
    for tag, cfg in (("fp8", mtq.FP8_DEFAULT_CFG), ("int8_sq", mtq.INT8_SMOOTHQUANT_CFG), ("int4_awq", int4),
                     ("nvfp4", mtq.NVFP4_DEFAULT_CFG)):
        model = copy.deepcopy(base)
        mtq.quantize(model, copy.deepcopy(cfg), loop)
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            cases[f"{tag}_{name}_format"] = np.array(get_quantization_format(lin))
            _export_quantized_weight(lin, dtype)
        sd = postprocess_state_dict(model.state_dict(), 448.0, None)
        cases[f"{tag}_keys"] = np.array(sorted(sd.keys()))
        for k, v in sd.items():
            cases[f"{tag}_sd_{k}"] = bits(v)
            cases[f"{tag}_dt_{k}"] = np.array(str(v.dtype))
    np.savez_compressed(out / "export_layers.npz", **cases)


class SharedInputBlock(nn.Module):
    """A normalisation layer feeding three projections, as the attention input of a decoder layer."""

    def __init__(self, hidden=128):
        super().__init__()
        self.input_layernorm = nn.LayerNorm(hidden)
        self.q_proj = nn.Linear(hidden, 128, bias=False)
        self.k_proj = nn.Linear(hidden, 64, bias=False)
        self.v_proj = nn.Linear(hidden, 64, bias=False)

    def forward(self, x):
        h = self.input_layernorm(x)
        return torch.cat([self.q_proj(h), self.k_proj(h), self.v_proj(h)], dim=-1)


def make_shared_input_block(seed, dtype):
    torch.manual_seed(seed)
    m = SharedInputBlock()
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "layernorm" in name:
                p.copy_(1.0 + 0.1 * torch.randn_like(p) if name.endswith("weight") else 0.05 * torch.randn_like(p))
            else:
                p.copy_(torch.randn_like(p) * (0.03 + 0.02 * "qkv".index(name[0])))
    return m.to(dtype)


def golden_export_fusion(mtq, out):
    """Layers that share their input, made fusable by the reference (preprocess_linear_fusion, then
    fuse_prequant_layernorm for the AWQ format) and exported layer by layer.  Stored: the state of the
    block before the fusion step (weights, pre-quant scales, amax) and the exported state dict after it."""
    from modelopt.torch.export.quant_utils import (fuse_prequant_layernorm, get_quantization_format,
                                                   postprocess_state_dict, preprocess_linear_fusion)
    from modelopt.torch.export.unified_export_hf import _export_quantized_weight

    cases = {}
    dtype = torch.bfloat16
    batches = make_batches(52, 2, dtype)
    for i, b in enumerate(batches):
        cases[f"x{i}"] = bits(b)
    base = make_shared_input_block(51, dtype)
    for k, v in base.state_dict().items():
        cases[f"base_{k}"] = bits(v)

    def loop(m):
        for b in batches:
            m(b)

    int4 = copy.deepcopy(mtq.INT4_AWQ_CFG)
    int4["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 32, "type": "static"}
    for tag, cfg in (("nvfp4", mtq.NVFP4_DEFAULT_CFG), ("int4_awq", int4), ("w4a8_awq", mtq.W4A8_AWQ_BETA_CFG),
                     ("fp8", mtq.FP8_DEFAULT_CFG)):
        model = copy.deepcopy(base)
        mtq.quantize(model, copy.deepcopy(cfg), loop)
        layers = [model.q_proj, model.k_proj, model.v_proj]
        for name, lin in zip("qkv", layers):      # what the fusion step starts from
            cases[f"{tag}_pre_{name}_weight"] = bits(lin.weight)
            if hasattr(lin.input_quantizer, "_pre_quant_scale"):
                cases[f"{tag}_pre_{name}_pqs"] = bits(lin.input_quantizer._pre_quant_scale)
            if getattr(lin.input_quantizer, "_amax", None) is not None:
                cases[f"{tag}_pre_{name}_in_amax"] = bits(lin.input_quantizer._amax.float().reshape(-1))
        fmt = get_quantization_format(layers[0])
        cases[f"{tag}_format"] = np.array(str(fmt))
        if fmt != "fp8":                                          # unified_export_hf.py:186-196
            preprocess_linear_fusion(layers)
        if "awq" in fmt:
            fuse_prequant_layernorm(model.input_layernorm, layers)
        for lin in layers:
            _export_quantized_weight(lin, dtype)
        sd = postprocess_state_dict(model.state_dict(), 448.0, None)
        cases[f"{tag}_keys"] = np.array(sorted(sd.keys()))
        for k, v in sd.items():
            cases[f"{tag}_sd_{k}"] = bits(v)
            cases[f"{tag}_dt_{k}"] = np.array(str(v.dtype))
    np.savez_compressed(out / "export_fusion.npz", **cases)


def golden_clip_smooth(mtq, out):
    """awq_clip / awq_full on INT4 block-32 weights (losses per clip ratio and block, the chosen
    block amax) and INT8 smoothquant (pre-quant scale, smoothed weight, amax buffers)."""
    cases = {}
    for tag, dtype in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        batches = make_batches(32, 2, dtype, tokens=80)      # 80 tokens: the sampler keeps every token
        for i, b in enumerate(batches):
            cases[f"{tag}_x{i}"] = bits(b)

        def loop(m):
            for b in batches:
                m(b)

        for method in ("awq_clip", "awq_full"):
            model = make_model(31, dtype)
            if method == "awq_clip":
                cases[f"{tag}_w_up"] = bits(model.up_proj.weight)
                cases[f"{tag}_w_down"] = bits(model.down_proj.weight)
            cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
            cfg["quant_cfg"]["*weight_quantizer"]["block_sizes"] = {-1: 32, "type": "static"}
            cfg["algorithm"] = {"method": method, "debug": True, "max_tokens_per_batch": 32}
            if method == "awq_full":
                cfg["algorithm"]["alpha_step"] = 0.1
            mtq.quantize(model, cfg, loop)
            for name in ("up_proj", "down_proj"):
                lin = getattr(model, name)
                st = lin.awq_clip
                k = f"{tag}_{method}_{name}"
                cases[k + "_ratios"] = np.array(list(st.loss.keys()), dtype=np.float64)
                cases[k + "_losses"] = np.stack([v.float().numpy() for v in st.loss.values()])
                cases[k + "_w_amax"] = bits(st.w_amax)
                cases[k + "_best_clip"] = bits(lin.weight_quantizer._amax)
                cases[k + "_num_tokens"] = np.array(st.num_tokens)
                if method == "awq_full":
                    cases[k + "_pqs"] = bits(lin.input_quantizer._pre_quant_scale)
                    cases[k + "_best_alpha"] = np.array(lin.awq_lite.best_alpha, dtype=np.float64)
            cases[f"{tag}_{method}_y"] = bits(model(batches[0]))

        model = make_model(31, dtype)
        mtq.quantize(model, copy.deepcopy(mtq.INT8_SMOOTHQUANT_CFG), loop)
        for name in ("up_proj", "down_proj"):
            lin = getattr(model, name)
            k = f"{tag}_sq_{name}"
            cases[k + "_pqs"] = bits(lin.input_quantizer._pre_quant_scale)
            cases[k + "_in_amax"] = bits(lin.input_quantizer._amax.reshape(-1))
            cases[k + "_w_amax"] = bits(lin.weight_quantizer._amax.reshape(-1))
            cases[k + "_w"] = bits(lin.weight)
            cases[k + "_amax_for_smoothing"] = lin.input_quantizer._amax_for_smoothing.float().numpy()
        cases[f"{tag}_sq_y"] = bits(model(batches[0]))
    np.savez_compressed(out / "clip_smooth.npz", **cases)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a TensorRT-Model-Optimizer checkout")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    mtq = import_reference(args.ref)
    if args.only == "export_layers":
        golden_export_layers(mtq, HERE)
        print("wrote export_layers")
        return
    if args.only == "export_fusion":
        golden_export_fusion(mtq, HERE)
        print("wrote export_fusion")
        return
    if args.only == "awq128":
        golden_awq(mtq, HERE, "awq128", hidden=256, inter=512, tokens=128)
        print("wrote awq128")
        return
    if args.only == "clip_smooth":
        golden_clip_smooth(mtq, HERE)
        print("wrote clip_smooth")
        return
    golden_awq(mtq, HERE)
    golden_awq(mtq, HERE, "awq128", hidden=256, inter=512, tokens=128)
    print("wrote awq, awq128")
    golden_flows(mtq, HERE)
    print("wrote flows")
    golden_clip_smooth(mtq, HERE)
    print("wrote clip_smooth")
    golden_export_layers(mtq, HERE)
    print("wrote export_layers")
    golden_export_fusion(mtq, HERE)
    print("wrote export_fusion")


if __name__ == "__main__":
    main()
