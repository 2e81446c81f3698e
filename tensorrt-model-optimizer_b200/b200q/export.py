"""Export-side weight packers (reference: modelopt/torch/export/quant_utils.py:68-91,697-834):
the on-disk layouts deployment frameworks read, produced by the same kernels as the in-memory
real-quant tensors plus the transposed INT4 packer."""
from __future__ import annotations

import torch

from . import ops
from .qtensor import FP8QTensor, NVFP4QTensor, QTensorWrapper

__all__ = ["get_scaling_factor_from_weight", "pack_int4_in_uint8", "to_quantized_weight", "from_quantized_weight",
           "get_quantization_format", "get_weight_block_size", "get_scaling_factor", "get_activation_scaling_factor",
           "get_weight_scaling_factor", "get_weight_scaling_factor_2", "get_prequant_scaling_factor",
           "export_quantized_weight", "postprocess_state_dict", "export_hf_state_dict", "adjust_attn_amax_values", "all_items_same", "process_layer_quant_config", "get_quant_config",
           "convert_hf_quant_config_format", "export_hf_checkpoint",
           "preprocess_linear_fusion", "fuse_prequant_layernorm", "fuse_prequant_to_linear", "requantize_resmooth_fused_llm_layers",
           "get_kv_cache_dtype", "get_kv_cache_scaling_factor", "get_kv_cache_bias",
           "KV_CACHE_FP8", "KV_CACHE_INT8", "KV_CACHE_NVFP4", "KV_CACHE_NVFP4_AFFINE",
           "QUANTIZATION_FP8", "QUANTIZATION_INT8_SQ", "QUANTIZATION_INT8_WO", "QUANTIZATION_INT4_AWQ",
           "QUANTIZATION_W4A8_AWQ", "QUANTIZATION_NVFP4", "QUANTIZATION_NVFP4_AWQ", "QUANTIZATION_FP8_PB_WO",
           "QUANTIZATION_FP8_PC_PT"]

QUANTIZATION_FP8 = "fp8"
QUANTIZATION_INT8_SQ = "int8_sq"
QUANTIZATION_INT8_WO = "int8_wo"
QUANTIZATION_INT4_AWQ = "int4_awq"
QUANTIZATION_W4A8_AWQ = "w4a8_awq"
QUANTIZATION_NVFP4 = "nvfp4"
QUANTIZATION_NVFP4_AWQ = "nvfp4_awq"
QUANTIZATION_FP8_PB_WO = "fp8_pb_wo"
QUANTIZATION_FP8_PC_PT = "fp8_pc_pt"


def _true_div(a: torch.Tensor, value: float) -> torch.Tensor:
    return a / torch.full((), value, dtype=a.dtype, device=a.device)


def get_scaling_factor_from_weight(weight, group_size) -> torch.Tensor:
    """fp32 amax / 7 per (row, group) for int4_awq (group_size > 0) or amax / 127 per row."""
    n, k = weight.shape
    if group_size != 0:
        if k % group_size != 0:
            raise NotImplementedError("Weight shape is not divisible for block size for block quantization.")
        amax = ops.amax_blocks(weight, group_size).reshape(n, k // group_size)
        maxbound = 7.0
    else:
        amax = ops.amax_axis3(weight, 1, n, k)
        maxbound = 127.0
    s = _true_div(amax, maxbound)
    s[s == 0] = 1.0
    return s


def pack_int4_in_uint8(weight, weights_scaling_factor):
    """uint8 [out/2, in]: two output channels per byte (low nibble = even row), signed nibbles."""
    out_dim = weight.shape[-2]
    assert out_dim % 2 == 0, f"Cannot pack weight. Out dimension {out_dim} is not an even number."
    if weight.dim() == 3:
        return torch.stack([ops.int4_export_pack(weight[e], weights_scaling_factor[e])
                            for e in range(weight.shape[0])])
    return ops.int4_export_pack(weight, weights_scaling_factor)


def _quotient(weight, scale):
    """``weight / scale`` with torch's type promotion, formed as an fp32 division rounded to the
    result type — what the CPU kernels compute.  (On CUDA torch would first round a 0-dim fp32
    scale to a 16-bit weight's type, which changes the last bit of the quotient.)"""
    rt = torch.result_type(weight, scale)
    return (weight.float() / scale.float()).to(rt).contiguous()


def _fp8(weight, scale_broadcast):
    """torch's e4m3 cast of the promoted quotient, through the cast kernel."""
    q = _quotient(weight, scale_broadcast)
    one = torch.ones(1, dtype=q.dtype, device=q.device)
    return ops.fp8_quantize(q, one, 1, 1, q.numel()).reshape(weight.shape)


def to_quantized_weight(weight, weights_scaling_factor, quantization: str, weights_scaling_factor2=None,
                        block_size=None):
    """Convert a weight to its packed checkpoint form for ``quantization``."""
    if weights_scaling_factor is not None:
        weights_scaling_factor = weights_scaling_factor.to(weight.device)
    if weights_scaling_factor2 is not None:
        weights_scaling_factor2 = weights_scaling_factor2.to(weight.device)
    if isinstance(weight, QTensorWrapper):
        return weight.data
    if quantization == QUANTIZATION_FP8:
        if weight.dtype == torch.float8_e4m3fn:
            return weight
        s = weights_scaling_factor.unsqueeze(-1) if weight.dim() == 3 else weights_scaling_factor
        return _fp8(weight, s)
    if quantization in (QUANTIZATION_INT8_SQ, QUANTIZATION_INT8_WO):
        q = _quotient(weight, weights_scaling_factor[:, None])
        one = torch.ones(1, dtype=q.dtype, device=q.device)
        return ops.int8_quantize(q, one, 1, 1, q.numel()).reshape(weight.shape)
    if quantization == QUANTIZATION_FP8_PB_WO:
        return FP8QTensor.quantize(weight, weights_scaling_factor.squeeze(),
                                   block_sizes={-1: block_size, -2: block_size})[0]._quantized_data
    if quantization == QUANTIZATION_FP8_PC_PT:
        return _fp8(weight, weights_scaling_factor[:, None])
    if quantization in (QUANTIZATION_INT4_AWQ, QUANTIZATION_W4A8_AWQ):
        return pack_int4_in_uint8(weight, weights_scaling_factor)
    if quantization in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        assert block_size is not None, "Block size not passed. Unable to quantize to NVFP4 format."
        assert weights_scaling_factor2 is not None, (
            "Weights scaling factor 2 not passed. Unable to quantize to NVFP4 format")
        return NVFP4QTensor.quantize(weight, block_size, weights_scaling_factor,
                                     weights_scaling_factor2)[0]._quantized_data
    raise NotImplementedError(f"quantization format {quantization} not supported")


def from_quantized_weight(weight, weights_scaling_factor, quantization: str, torch_dtype):
    """Back from the checkpoint form to ``torch_dtype`` for the one-byte formats with one scale per tensor or
    per row (FP8, INT8); anything wider is only cast (reference modelopt/torch/export/quant_utils.py:837-857,
    the same two torch operations, so the values are the reference's)."""
    if weight.element_size() >= 2 or weights_scaling_factor is None or not quantization:
        return weight.to(torch_dtype)
    if quantization == QUANTIZATION_FP8:
        return weight.view(torch.float8_e4m3fn).to(torch_dtype) * weights_scaling_factor.to(torch_dtype)
    if quantization in (QUANTIZATION_INT8_SQ, QUANTIZATION_INT8_WO):
        return weight.to(torch_dtype) * weights_scaling_factor[:, None].to(torch_dtype)
    raise NotImplementedError(f"quantization format {quantization} not supported")


# ---------------------------------------------------------------- per-layer checkpoint export --
# Reference: modelopt/torch/export/quant_utils.py:214-321,412-533,860-983 and
# modelopt/torch/export/unified_export_hf.py:233-392 (for nn.Linear-like modules with the
# ``weight`` / ``weight_quantizer`` / ``input_quantizer`` attribute names).

QUANTIZATION_NONE = None


def get_quantization_format(module):
    """The checkpoint format name implied by a layer's quantisers (None if not quantised)."""
    from .nn import SequentialQuantizer

    wq = getattr(module, "weight_quantizer", None)
    iq = getattr(module, "input_quantizer", None)
    if wq is not None and wq.is_enabled:
        if isinstance(wq, SequentialQuantizer):
            assert len(wq) == 2 and wq[0].num_bits == 4 and wq[1].num_bits == (4, 3), \
                "Unsupported SequentialQuantizer configuration"
            return QUANTIZATION_W4A8_AWQ
        if wq.num_bits == 4:
            assert wq.block_sizes and wq.block_sizes[-1] > 0, "Invalid block_sizes for INT4 quantizer"
            return QUANTIZATION_INT4_AWQ
        if wq.num_bits == 8:
            return QUANTIZATION_INT8_SQ if iq is not None and iq.is_enabled else QUANTIZATION_INT8_WO
        if wq.num_bits == (4, 3):
            if wq.block_sizes:
                if not wq.fake_quant:
                    raise NotImplementedError("export of real-quantised per-block FP8 weights")
                return QUANTIZATION_FP8_PB_WO
            return QUANTIZATION_FP8_PC_PT if wq.axis == 0 else QUANTIZATION_FP8
        if wq.num_bits == (2, 1):
            scale_bits = wq.block_sizes.get("scale_bits")
            if iq is not None and hasattr(iq, "_pre_quant_scale"):
                return QUANTIZATION_NVFP4_AWQ
            if scale_bits == (4, 3):
                return QUANTIZATION_NVFP4
        raise NotImplementedError(f"Unsupported quantizer with num_bits: {wq.num_bits}")
    for _, child in module.named_children():
        fmt = get_quantization_format(child)
        if fmt is not QUANTIZATION_NONE:
            return fmt
    return QUANTIZATION_NONE


def get_weight_block_size(module) -> int:
    from .nn import SequentialQuantizer

    wq = getattr(module, "weight_quantizer", None)
    if wq is None:
        return 0
    if isinstance(wq, SequentialQuantizer):
        wq = wq[0]
    if not wq.is_enabled or not wq.block_sizes:
        return 0
    return wq.block_sizes[-1]


def adjust_attn_amax_values(module):
    """Give the weight quantisers of the q / k / v projections among ``module``'s children their common
    maximum amax, as a fused QKV GEMM needs (reference modelopt/torch/export/quant_utils.py:185-211)."""
    layers = []
    for name, child in module.named_children():
        for prefix in ("q", "k", "v"):
            if prefix in name and hasattr(child, "weight_quantizer") and hasattr(child.weight_quantizer, "amax") \
                    and child.weight_quantizer.amax is not None:
                layers.append(child)
    if not layers:
        raise ValueError("No projection layers with the specified prefixes ('q', 'k', 'v') have amax attributes")
    common = torch.stack([layer.weight_quantizer.amax.float().reshape(()) for layer in layers]).max()
    assert common > 0, "max_amax must be positive."
    for layer in layers:
        layer.weight_quantizer.amax.copy_(common)


def get_scaling_factor(quantizer):
    """fp32 scaling factor of a quantiser: amax / maxbound (amax / (6 * 448) for NVFP4)."""
    if not quantizer.is_enabled:
        return None
    amax = quantizer.export_amax()
    if amax is None:
        return None
    if quantizer.num_bits == (2, 1):
        s = NVFP4QTensor.get_weights_scaling_factor_2_from_quantizer(quantizer)
    else:
        s = _true_div(amax.float(), float(quantizer.maxbound))
    assert torch.all(s > 0), f"scaling factor {s} not positive."
    return s


def get_kv_cache_dtype(modules):
    """"FP8" / "INT8" / "NVFP4" / "NVFP4_AFFINE" from the enabled ``k_bmm_quantizer`` / ``v_bmm_quantizer`` /
    ``output_quantizer`` of a module or list of modules, None without one (reference
    modelopt/torch/export/quant_utils.py:373-409)."""
    if isinstance(modules, torch.nn.Module):
        modules = [modules]
    bits, affine = [], True
    for module in modules:
        for name in ("k_bmm_quantizer", "v_bmm_quantizer", "output_quantizer"):
            q = getattr(module, name, None)
            if q is not None and q.is_enabled:
                bits.append(q.num_bits)
                affine &= getattr(q, "_bias_value", None) is not None
    if (4, 3) in bits:
        return KV_CACHE_FP8
    if 8 in bits:
        return KV_CACHE_INT8
    if (2, 1) in bits:
        return KV_CACHE_NVFP4_AFFINE if affine else KV_CACHE_NVFP4
    return QUANTIZATION_NONE


def get_kv_cache_bias(kv_module):
    return [getattr(getattr(kv_module, name, None), "_bias_value", None) for name in ("k_bmm_quantizer", "v_bmm_quantizer")]


def get_kv_cache_scaling_factor(kv_module):
    """[k scale, v scale] of an attention module with KV-cache quantisers, at least 1 for an FP8 cache
    (reference modelopt/torch/export/quant_utils.py:348-370); [None, None] without the quantisers."""
    if not hasattr(kv_module, "k_bmm_quantizer") or not hasattr(kv_module, "v_bmm_quantizer"):
        return [None, None]
    factors = [get_scaling_factor(getattr(kv_module, name)) for name in ("k_bmm_quantizer", "v_bmm_quantizer")]
    if get_kv_cache_dtype(kv_module) == KV_CACHE_FP8:
        factors = [f.clamp(min=1.0) for f in factors]
    return factors


def get_activation_scaling_factor(module):
    iq = getattr(module, "input_quantizer", None)
    if iq is None:
        return None
    if get_quantization_format(module) in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        return NVFP4QTensor.get_activation_scaling_factor(iq)
    return get_scaling_factor(iq)


def get_weight_scaling_factor(module):
    from .nn import SequentialQuantizer

    wq = getattr(module, "weight_quantizer", None)
    if wq is None:
        return None
    if isinstance(wq, SequentialQuantizer):
        return get_scaling_factor(wq[0])
    if get_quantization_format(module) in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        s2 = NVFP4QTensor.get_weights_scaling_factor_2_from_quantizer(wq)
        return NVFP4QTensor.get_weights_scaling_factor(module.weight, wq.block_sizes[-1], s2.to(module.weight.device))[0]
    return get_scaling_factor(wq)


def get_weight_scaling_factor_2(module):
    from .nn import SequentialQuantizer

    wq = getattr(module, "weight_quantizer", None)
    if wq is None:
        return None
    if get_quantization_format(module) in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        return NVFP4QTensor.get_weights_scaling_factor_2_from_quantizer(wq)
    if not isinstance(wq, SequentialQuantizer) or not wq[-1].is_enabled:
        return None
    assert len(wq) == 2, "only 2 sequential quantization layers are supported"
    return get_scaling_factor(wq[-1])


def get_prequant_scaling_factor(module):
    iq = getattr(module, "input_quantizer", None)
    s = iq._pre_quant_scale.squeeze() if iq is not None and hasattr(iq, "_pre_quant_scale") else None
    if s is not None:
        assert torch.all(s > 0), f"prequant scaling factor {s} not positive."
    return s


@torch.no_grad()
def export_quantized_weight(module, dtype: torch.dtype):
    """Replace ``module.weight`` by its packed checkpoint form and register ``weight_scale``,
    ``weight_scale_2`` and ``input_scale`` buffers, as the reference's per-layer export does."""
    fmt = get_quantization_format(module)
    if fmt is QUANTIZATION_NONE:
        return
    block_size = get_weight_block_size(module)
    wq, iq = module.weight_quantizer, getattr(module, "input_quantizer", None)
    weight = module.weight
    if fmt == QUANTIZATION_FP8:
        wq._amax = wq._amax.to(torch.float32)
        if wq._amax.dim() == 1:
            ws = torch.tensor(wq.amax.item() / wq.maxbound)
        else:
            ws = _true_div(wq.amax, float(wq.maxbound)).clone()
        module.register_buffer("weight_scale", ws)
        if iq is not None and hasattr(iq, "_amax"):
            iq._amax = iq._amax.to(torch.float32)
            module.register_buffer("input_scale", get_activation_scaling_factor(module).squeeze())
    else:
        module.register_buffer("weight_scale", get_weight_scaling_factor(module))
        if iq is not None and iq.is_enabled and iq.amax is not None:
            module.register_buffer("input_scale", get_activation_scaling_factor(module).squeeze())
    if fmt in (QUANTIZATION_NVFP4_AWQ, QUANTIZATION_NVFP4, QUANTIZATION_W4A8_AWQ):
        module.register_buffer("weight_scale_2", get_weight_scaling_factor_2(module).squeeze())
    weight_scale = getattr(module, "weight_scale", None)
    weight_scale_2 = getattr(module, "weight_scale_2", None)
    if fmt in (QUANTIZATION_NVFP4, QUANTIZATION_NVFP4_AWQ):
        weight_scale = NVFP4QTensor.get_weights_scaling_factor(weight, block_size, weight_scale_2)[0]
    packed = to_quantized_weight(weight.to(dtype), weight_scale, fmt, weight_scale_2, block_size)
    module.weight = torch.nn.Parameter(packed, requires_grad=False)
    if weight_scale is not None:
        module.register_buffer("weight_scale", weight_scale)


KV_CACHE_FP8, KV_CACHE_INT8, KV_CACHE_NVFP4, KV_CACHE_NVFP4_AFFINE = "FP8", "INT8", "NVFP4", "NVFP4_AFFINE"


def postprocess_state_dict(state_dict: dict, maxbound: float = 0.0, quantization: str | None = None) -> dict:
    """Drop quantiser state (``_amax``, output quantisers, real-quant scale buffers), rename
    ``input_quantizer._pre_quant_scale`` to ``pre_quant_scale``, turn the amax of KV-cache quantisers
    (``[kv]_bmm_quantizer._amax``) into ``k_proj.k_scale`` / ``v_proj.v_scale`` = amax / ``maxbound`` (at least
    1 for an FP8 cache, ``quantization`` naming the cache format) and squeeze ``[1, a, b]`` scales
    (reference modelopt/torch/export/quant_utils.py:860-983)."""
    from .nn import RealQuantLinear

    skip = ("output_quantizer", "_amax", "_bias_value", "input_quantizer._pre_quant_scale")
    replacements = {"k_bmm_quantizer._amax": "k_proj.k_scale", "v_bmm_quantizer._amax": "v_proj.v_scale",
                    "k_bmm_quantizer._bias_value": "k_proj.k_bias", "v_bmm_quantizer._bias_value": "v_proj.v_bias",
                    "input_quantizer._pre_quant_scale": "pre_quant_scale"}
    out = {}
    for key, value in state_dict.items():
        if all(s not in key for s in skip):
            out[key] = value
            continue
        for old, new in replacements.items():
            if not key.endswith(old):
                continue
            if "_amax" in key:
                assert quantization in (KV_CACHE_FP8, KV_CACHE_NVFP4, KV_CACHE_NVFP4_AFFINE), (
                    "Invalid KV cache quantization format.")
                assert maxbound > 0, "Maxbound must be greater than zero."
                value = _true_div(value.float(), float(maxbound))
                if quantization == KV_CACHE_FP8:
                    value = value.clamp(min=1.0)
            out[key[: -len(old)] + new] = value
            break
    for key, value in list(out.items()):
        if "scale" in key and isinstance(value, torch.Tensor) and value.dim() == 3 and value.shape[0] == 1:
            out[key] = value.squeeze(0)
    scale_names = getattr(RealQuantLinear, "list_of_scale_tensors", ["_scale", "_double_scale", "_scale_zeros"])
    for key in [k for k in out if any(k.endswith("weight_quantizer." + q) for q in scale_names)]:
        del out[key]
    seen = {}
    for key in list(out):
        v = out[key]
        if isinstance(v, torch.Tensor):
            if v.data_ptr() in seen and v.numel() > 0:
                del out[key]          # a tied weight: keep the first name
            else:
                seen[v.data_ptr()] = key
    return out


# ------------------------------------------------------------- layers that share their input --
# Reference: modelopt/torch/export/quant_utils.py:986-1011,1104-1187 and
# modelopt/torch/export/unified_export_hf.py:90-232.  Linear layers fed the same tensor (q / k / v, gate / up)
# are served by one fused GEMM at deployment: they must agree on the input scale, on a per-tensor weight scale
# and on the AWQ pre-quant scale, which can then move into the normalisation layer in front of them.

def all_items_same(item_list):
    return all(x == item_list[0] for x in item_list)


@torch.no_grad()
def _update_pre_quant_scale(module, new_pre_quant_scale):
    """Re-smooth ``module`` to another pre-quant scale: the weight takes old / new (in fp32), the weight
    quantiser is calibrated again on the new weight."""
    from .model_calib import enable_stats_collection, finish_stats_collection

    old = module.input_quantizer._pre_quant_scale
    dtype, device = module.weight.dtype, module.weight.device
    module.weight = torch.nn.Parameter(
        (module.weight.to(torch.float32) * old.to(dtype=torch.float32, device=device)
         / new_pre_quant_scale.to(dtype=torch.float32, device=device)).to(dtype),
        requires_grad=module.weight.requires_grad)
    module.input_quantizer.pre_quant_scale = new_pre_quant_scale
    module.weight_quantizer.reset_amax()
    enable_stats_collection(module.weight_quantizer)
    module.weight_quantizer(module.weight)
    finish_stats_collection(module.weight_quantizer)


@torch.no_grad()
def preprocess_linear_fusion(modules, resmooth_only=False):
    """Make the quantised linear layers ``modules`` fusable: the mean of their pre-quant scales for all
    (weights re-smoothed and re-calibrated), the maximum of their per-tensor input amax and of their
    per-tensor weight amax (the second quantiser of a sequential pair)."""
    from .nn import SequentialQuantizer

    assert all_items_same([get_quantization_format(m) for m in modules]), "Modules have different quantization formats"
    first = modules[0]
    if hasattr(first, "input_quantizer"):
        if first.input_quantizer.pre_quant_scale is not None:
            mean = torch.mean(torch.stack([m.input_quantizer.pre_quant_scale for m in modules]), dim=0)
            for m in modules:
                if not torch.equal(m.input_quantizer.pre_quant_scale, mean):
                    _update_pre_quant_scale(m, mean)
        if resmooth_only:
            return
        if first.input_quantizer.is_enabled and first.input_quantizer.amax is not None:
            assert first.input_quantizer.amax.numel() == 1, "Only support scalar input quant amax"
            common = torch.max(torch.stack([m.input_quantizer.amax for m in modules]))
            for m in modules:
                m.input_quantizer.amax = common
    if hasattr(first, "weight_quantizer"):
        wq = first.weight_quantizer
        if isinstance(wq, SequentialQuantizer):
            if wq[-1].is_enabled:
                assert len(wq) == 2
                common = torch.max(torch.stack([m.weight_quantizer[-1].amax for m in modules]))
                for m in modules:
                    m.weight_quantizer[-1].amax = common
        elif wq.is_enabled and wq.amax is not None and wq.amax.numel() == 1:
            common = torch.max(torch.stack([m.weight_quantizer.amax for m in modules]))
            for m in modules:
                m.weight_quantizer.amax = common


@torch.no_grad()
def fuse_prequant_layernorm(layernorm_module, modules):
    """Move the (common) pre-quant scale of ``modules`` into the weight and bias of the normalisation layer
    that feeds them; the layers lose their ``_pre_quant_scale`` and are marked ``fused_with_prequant``."""
    scale = modules[0].input_quantizer._pre_quant_scale
    layernorm_module.weight = torch.nn.Parameter(layernorm_module.weight * scale)
    if getattr(layernorm_module, "bias", None) is not None:
        layernorm_module.bias = torch.nn.Parameter(layernorm_module.bias * scale)
    for m in modules:
        delattr(m.input_quantizer, "_pre_quant_scale")
        m.fused_with_prequant = True


# (class-name fragments of the parent, layer that takes the scale, layer that gives it up): the output channels
# of v_proj are the input channels of o_proj (through the attention average), those of up_proj the input
# channels of down_proj (through the elementwise product with the gate).
_PRE_QUANT_SCALE_MOVES = ((("LlamaAttention", "Qwen3Attention", "Qwen3MoeAttention"), "v_proj", "o_proj"),
                          (("LlamaMLP", "Qwen3MLP", "Qwen3MoeMLP"), "up_proj", "down_proj"))


@torch.no_grad()
def fuse_prequant_to_linear(model, fuse_grouped_heads=False):
    """Move the pre-quant scale of o_proj / down_proj into the output channels of the layer whose output they
    read (v_proj / up_proj) where the module classes are known to allow it (reference
    modelopt/torch/export/quant_utils.py:1013-1102).  With grouped-query attention o_proj has more input
    channels than v_proj has outputs: with ``fuse_grouped_heads`` the scale is first averaged over the query
    heads that share a key / value head (o_proj is re-smoothed to the averaged scale), otherwise the pair is
    skipped.  The taking layer's weight quantiser is calibrated again; the giving layer loses its
    ``_pre_quant_scale`` and is marked ``fused_with_prequant``."""
    import warnings

    from .model_calib import enable_stats_collection, finish_stats_collection

    for parent in model.modules():
        kind = type(parent).__name__
        for fragments, taker_name, giver_name in _PRE_QUANT_SCALE_MOVES:
            if not any(f in kind for f in fragments):
                continue
            taker, giver = parent.get_submodule(taker_name), parent.get_submodule(giver_name)
            scale = getattr(getattr(giver, "input_quantizer", None), "_pre_quant_scale", None)
            if scale is None:
                continue
            out_channels = taker.weight.shape[-2]
            if scale.numel() != out_channels:
                if not fuse_grouped_heads or "attention" not in kind.lower():
                    warnings.warn(f"Skipping pattern fuse prequant for {kind}: pre_quant_scale dim {scale.numel()} "
                                  f"!= out_channel dim {out_channels}")
                    continue
                kv_heads = parent.config.num_key_value_heads
                head_dim = out_channels // kv_heads
                queries_per_kv = scale.numel() // out_channels
                per_kv_head = scale.view(kv_heads, queries_per_kv, head_dim).mean(dim=1)
                _update_pre_quant_scale(giver, per_kv_head.unsqueeze(1).expand(kv_heads, queries_per_kv, head_dim).reshape(-1))
                scale = per_kv_head.reshape(-1)
            taker.weight = torch.nn.Parameter(taker.weight * scale.view(-1, 1), requires_grad=taker.weight.requires_grad)
            if getattr(taker, "bias", None) is not None:
                taker.bias = torch.nn.Parameter(taker.bias * scale, requires_grad=taker.bias.requires_grad)
            taker.weight_quantizer.reset_amax()
            enable_stats_collection(taker.weight_quantizer)
            taker.weight_quantizer(taker.weight)
            finish_stats_collection(taker.weight_quantizer)
            delattr(giver.input_quantizer, "_pre_quant_scale")
            giver.fused_with_prequant = True


def _is_layernorm(module) -> bool:
    name = type(module).__name__
    return any(key in name for key in ("LayerNorm", "RMSNorm"))


@torch.no_grad()
def requantize_resmooth_fused_llm_layers(model, fake_input=None):
    """Find the quantised linear layers that are fed the same tensor by one forward pass with every
    quantiser off, make each such group fusable (``preprocess_linear_fusion``; FP8 layers keep their own
    scales, as in the reference) and, for AWQ formats, move the group's pre-quant scale into the
    normalisation layer whose output they read.  ``fake_input`` defaults to the two-token id tensor the
    reference feeds a causal language model.  Returns {first layer's name: names of its group}."""
    from .conversion import set_quantizer_by_cfg_context
    from .nn import is_quantized_linear

    by_input, by_output, handles, names = {}, {}, [], {}
    whole = get_quantization_format(model)
    if whole is not QUANTIZATION_NONE and "nvfp4_awq" in whole:
        fuse_prequant_to_linear(model)

    def saw_input(module, args, output):
        by_input.setdefault(args[0], []).append(module)

    def saw_output(module, args, output):
        by_output[output] = module

    for name, module in model.named_modules():
        names[module] = name
        if _is_layernorm(module):
            handles.append(module.register_forward_hook(saw_output))
        elif is_quantized_linear(module) and (module.input_quantizer.is_enabled or module.weight_quantizer.is_enabled):
            handles.append(module.register_forward_hook(saw_input))
    try:
        if fake_input is None:
            device = next(model.parameters()).device
            fake_input = torch.ones([1, 2], dtype=torch.long, device=device)
        with set_quantizer_by_cfg_context(model, {"*": {"enable": False}}):
            model(fake_input)
    finally:
        for h in handles:
            h.remove()
    fused = {}
    for tensor, modules in by_input.items():
        fmt = get_quantization_format(modules[0])
        if len(modules) > 1 and fmt not in (QUANTIZATION_FP8, QUANTIZATION_NONE):
            preprocess_linear_fusion(modules)
            fused[names[modules[0]]] = [names[m] for m in modules]
        if fmt is not QUANTIZATION_NONE and "awq" in fmt and tensor in by_output \
                and hasattr(modules[0].input_quantizer, "_pre_quant_scale"):
            fuse_prequant_layernorm(by_output[tensor], modules)
    return fused


# ------------------------------------------------------ the quantisation record of a checkpoint --
# Reference: modelopt/torch/export/quant_utils.py:536-694 (process_layer_quant_config) and :1190-1290
# (get_quant_config): what ``hf_quant_config.json`` says beside the packed tensors.

# format name -> (deployment algorithm name, carries a group size, is an AWQ format)
_ALGORITHM_OF_FORMAT = {
    QUANTIZATION_FP8: ("FP8", False, False),
    QUANTIZATION_FP8_PC_PT: ("FP8_PER_CHANNEL_PER_TOKEN", False, False),
    QUANTIZATION_INT4_AWQ: ("W4A16_AWQ", True, True),
    QUANTIZATION_W4A8_AWQ: ("W4A8_AWQ", True, True),
    QUANTIZATION_INT8_WO: ("W8A16", False, False),
    QUANTIZATION_INT8_SQ: ("W8A8_SQ_PER_CHANNEL", False, False),
    QUANTIZATION_NVFP4: ("NVFP4", True, False),
    QUANTIZATION_NVFP4_AWQ: ("NVFP4_AWQ", True, True),
    "w4a8_nvfp4_fp8": ("W4A8_NVFP4_FP8", True, True),
    "w4a8_mxfp4_fp8": ("W4A8_MXFP4_FP8", True, False),
}


def _exclusion_patterns(unquantized, quantized):
    """The fewest-characters description of the unquantised layers by patterns cut at dots: for each layer
    the shortest ``prefix*`` (else the pair ``prefix`` + ``prefix.*``, else the name itself) that cannot
    match a quantised layer; a layer already covered by chosen patterns adds nothing."""
    forbidden = set()
    for name in quantized:
        forbidden.add(name)
        forbidden.update(name[:i] + "*" for i in range(len(name) + 1))
    chosen = set()
    for name in unquantized:
        cuts = [i for i, ch in enumerate(name) if ch == "."]
        options = [o for i in cuts for o in ([name[:i] + "*"], [name[:i], name[:i] + ".*"])] + [[name]]
        for option in options:
            if any(pattern in forbidden for pattern in option):
                continue
            if not all(pattern in chosen for pattern in option):
                chosen.update(option)
            break
    return chosen


def process_layer_quant_config(layer_config_dict: dict) -> dict:
    """``{"<layer>.quantization": format, "<layer>.awq_block_size": n}`` -> the record of the whole model: one
    algorithm with the excluded modules when every quantised layer has the same settings, else
    ``MIXED_PRECISION`` with the settings layer by layer."""
    layers, excluded, kinds = {}, [], {}
    for key, fmt in layer_config_dict.items():
        if "awq_block_size" in key:
            continue
        layer = key.rsplit(".", 1)[0]
        algorithm, grouped, awq = _ALGORITHM_OF_FORMAT.get(fmt, (fmt, False, False))
        if algorithm is QUANTIZATION_NONE:
            excluded.append(layer)
            continue
        record = {"quant_algo": algorithm}
        if grouped:
            record["group_size"] = layer_config_dict.get(layer + ".awq_block_size", 0)
        if awq:
            record.update(has_zero_point=False, pre_quant_scale=True)
        layers[layer] = record
        kinds[str(record)] = record
    out = {"quant_algo": None, "kv_cache_quant_algo": None}
    if len(kinds) > 1:
        out["quant_algo"] = "MIXED_PRECISION"
        out["quantized_layers"] = layers
    elif len(kinds) == 1:
        out.update(next(iter(kinds.values())))
        out["exclude_modules"] = sorted(_exclusion_patterns(excluded, layers.keys()))
    else:
        out["quantized_layers"] = {}
    return out


def get_quant_config(model) -> dict:
    """The quantisation record of a (fully, partly or mixed-precision) quantised model:
    ``{"producer": {...}, "quantization": {...}}``."""
    per_layer, kv_format = {}, QUANTIZATION_NONE
    for name, module in model.named_modules():
        if hasattr(module, "weight_quantizer") or hasattr(module, "input_quantizer"):
            per_layer[name + ".quantization"] = get_quantization_format(module)
            per_layer[name + ".awq_block_size"] = get_weight_block_size(module)
        if any(getattr(getattr(module, q, None), "is_enabled", False)
               for q in ("k_bmm_quantizer", "v_bmm_quantizer", "output_quantizer")):
            mine = get_kv_cache_dtype(module)
            assert kv_format in (QUANTIZATION_NONE, mine), "Do not support mixed precision kv cache quantization"
            kv_format = mine
    quantization = {"quant_algo": None, "kv_cache_quant_algo": None}
    quantization.update(process_layer_quant_config(per_layer))
    if kv_format is not QUANTIZATION_NONE:
        quantization["kv_cache_quant_algo"] = kv_format
    return {"producer": {"name": "b200q", "version": "0.40"}, "quantization": quantization}


@torch.no_grad()
def export_hf_state_dict(model, dtype: torch.dtype | None = None, fake_input=None) -> dict:
    """Packed state dict of a quantised model with the checkpoint's names (``weight``,
    ``weight_scale``, ``weight_scale_2``, ``input_scale``, ``pre_quant_scale``).  The model's
    linear layers are converted in place.  Layers that share their input are first made fusable
    (``requantize_resmooth_fused_llm_layers``) when the model is a Hugging Face model (it has a ``config``;
    the reference's two-token input is used) or when ``fake_input`` gives the tensor to trace it with."""
    from .nn import is_quantized_linear

    if dtype is None:
        dtype = next(p.dtype for p in model.parameters() if p.is_floating_point())
    if fake_input is not None or hasattr(model, "config"):
        requantize_resmooth_fused_llm_layers(model, fake_input)
    for _, m in model.named_modules():
        if is_quantized_linear(m) and get_quantization_format(m) is not QUANTIZATION_NONE:
            export_quantized_weight(m, dtype)
    return postprocess_state_dict(model.state_dict())


def convert_hf_quant_config_format(record: dict) -> dict:
    """The quantisation record in the shape Hugging Face's ``config.json`` carries as ``quantization_config``
    (reference modelopt/torch/export/convert_hf_config.py:21-117): the scheme of the one weight / activation
    group for FP8 and NVFP4, the ignored modules, the KV-cache scheme, ``quant_method`` "modelopt"."""
    q = record.get("quantization", {})
    algorithm = q.get("quant_algo")
    scheme = {"FP8": {"dynamic": False, "num_bits": 8, "type": "float"},
              "NVFP4": {"dynamic": False, "num_bits": 4, "type": "float", "group_size": q.get("group_size", 16)}}
    out = {}
    if algorithm in scheme:
        out["config_groups"] = {"group_0": {"input_activations": dict(scheme[algorithm]),
                                            "weights": dict(scheme[algorithm]), "targets": ["Linear"]}}
    out["ignore"] = q.get("exclude_modules") or []
    if algorithm:
        out["quant_algo"] = algorithm
    kv = q.get("kv_cache_quant_algo")
    if kv:
        out["kv_cache_scheme"] = dict(scheme["FP8"]) if kv == "FP8" else kv
    if record.get("producer"):
        out["producer"] = record["producer"]
    out["quant_method"] = "modelopt"
    return out


def export_hf_checkpoint(model, dtype: torch.dtype | None = None, export_dir="exported_model", fake_input=None):
    """Write the packed checkpoint of a quantised model to ``export_dir``: ``hf_quant_config.json`` (the
    quantisation record), the tensors under their checkpoint names, and — for a Hugging Face model, saved
    with its own ``save_pretrained`` — ``config.json`` with the record as ``quantization_config``; any other
    module is written as ``model.safetensors`` (reference modelopt/torch/export/unified_export_hf.py:556-615).
    The model's linear layers are converted in place."""
    import json
    from pathlib import Path

    export_dir = Path(export_dir)
    export_dir.mkdir(parents=True, exist_ok=True)
    record = get_quant_config(model)            # read before the layers are converted
    state = export_hf_state_dict(model, dtype, fake_input)
    quantised = record["quantization"]["quant_algo"] is not None
    if quantised:
        (export_dir / "hf_quant_config.json").write_text(json.dumps(record, indent=4))
    if hasattr(model, "save_pretrained"):
        model.save_pretrained(export_dir, state_dict=dict(state))      # it empties the dictionary it is given
        config_path = export_dir / "config.json"
        config = json.loads(config_path.read_text())
        if quantised:
            config["quantization_config"] = convert_hf_quant_config_format(record)
        config_path.write_text(json.dumps(config, indent=4))
    else:
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in state.items()}, str(export_dir / "model.safetensors"))
    return state, record
