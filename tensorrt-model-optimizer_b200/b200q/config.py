"""Quantisation format dictionaries and the quantiser attribute record, with the names and
contents of ``modelopt/torch/quantization/config.py`` (formats :147-388, attributes :661-955,
algorithm options :958-1150) for the formats this package accelerates."""
from __future__ import annotations

import copy
from dataclasses import dataclass, fields
from typing import Any

__all__ = ["QuantizerAttributeConfig", "INT8_DEFAULT_CFG", "INT8_WEIGHT_ONLY_CFG", "FP8_DEFAULT_CFG",
           "INT4_BLOCKWISE_WEIGHT_ONLY_CFG", "INT4_AWQ_CFG", "NVFP4_DEFAULT_CFG", "NVFP4_AWQ_LITE_CFG",
           "INT8_SMOOTHQUANT_CFG", "NVFP4_AWQ_CLIP_CFG", "NVFP4_AWQ_FULL_CFG",
           "FP8_PER_CHANNEL_PER_TOKEN_CFG", "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG", "W4A8_AWQ_BETA_CFG", "W4A8_NVFP4_FP8_CFG",
           "W4A8_MXFP4_FP8_CFG", "NVFP4_MLP_WEIGHT_ONLY_CFG", "NVFP4_MLP_ONLY_CFG", "MXFP4_MLP_WEIGHT_ONLY_CFG",
           "FP8_KV_CFG", "FP8_AFFINE_KV_CFG", "NVFP4_KV_CFG", "NVFP4_AFFINE_KV_CFG", "NVFP4_KV_ROTATE_CFG",
           "MXFP8_DEFAULT_CFG", "MXFP6_DEFAULT_CFG", "MXFP4_DEFAULT_CFG", "MXINT8_DEFAULT_CFG",
           "choices", "need_calibration"]

_default_disabled_quantizer_cfg = {
    "nn.BatchNorm1d": {"*": {"enable": False}},
    "nn.BatchNorm2d": {"*": {"enable": False}},
    "nn.BatchNorm3d": {"*": {"enable": False}},
    "nn.LeakyReLU": {"*": {"enable": False}},
    "*lm_head*": {"enable": False},
    "*proj_out.*": {"enable": False},
    "*block_sparse_moe.gate*": {"enable": False},
    "*router*": {"enable": False},
    "*mlp.gate.*": {"enable": False},
    "*mlp.shared_expert_gate.*": {"enable": False},
    "*linear_attn.conv1d*": {"enable": False},
    "*mixer.conv1d*": {"enable": False},
    "*output_layer*": {"enable": False},
    "output.*": {"enable": False},
    "default": {"enable": False},
}

INT8_DEFAULT_CFG = {
    "quant_cfg": {
        "*weight_quantizer": {"num_bits": 8, "axis": 0},
        "*input_quantizer": {"num_bits": 8, "axis": None},
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "max",
}

INT8_WEIGHT_ONLY_CFG = {
    "quant_cfg": {
        "*weight_quantizer": {"num_bits": 8, "axis": 0},
        "*input_quantizer": {"enable": False},
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "max",
}

FP8_DEFAULT_CFG = {
    "quant_cfg": {
        "*weight_quantizer": {"num_bits": (4, 3), "axis": None},
        "*input_quantizer": {"num_bits": (4, 3), "axis": None},
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "max",
}

INT4_BLOCKWISE_WEIGHT_ONLY_CFG = {
    "quant_cfg": {
        "*weight_quantizer": {"num_bits": 4, "block_sizes": {-1: 128}, "enable": True},
        "*input_quantizer": {"enable": False},
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "max",
}

INT4_AWQ_CFG = {
    "quant_cfg": {
        "*weight_quantizer": {"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
        "*input_quantizer": {"enable": False},
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": {"method": "awq_lite", "alpha_step": 0.1},
}

_nvfp4 = {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)},
          "axis": None, "enable": True}

NVFP4_DEFAULT_CFG = {
    "quant_cfg": {
        "*weight_quantizer": copy.deepcopy(_nvfp4),
        "*input_quantizer": copy.deepcopy(_nvfp4),
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "max",
}

NVFP4_AWQ_LITE_CFG = {
    "quant_cfg": {
        "*weight_quantizer": copy.deepcopy(_nvfp4),
        "*input_quantizer": copy.deepcopy(_nvfp4),
        **_default_disabled_quantizer_cfg,
    },
    "algorithm": "awq_lite",
}

INT8_SMOOTHQUANT_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": 8, "axis": 0}, "*input_quantizer": {"num_bits": 8, "axis": None},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "smoothquant",
}

_nvfp4 = {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, "axis": None,
          "enable": True}
NVFP4_AWQ_CLIP_CFG = {"quant_cfg": {"*weight_quantizer": dict(_nvfp4), "*input_quantizer": dict(_nvfp4),
                                    **_default_disabled_quantizer_cfg}, "algorithm": {"method": "awq_clip"}}
NVFP4_AWQ_FULL_CFG = {"quant_cfg": {"*weight_quantizer": dict(_nvfp4), "*input_quantizer": dict(_nvfp4),
                                    **_default_disabled_quantizer_cfg},
                      "algorithm": {"method": "awq_full", "alpha_step": 0.1}}


FP8_PER_CHANNEL_PER_TOKEN_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": (4, 3), "axis": 0},
                  "*input_quantizer": {"num_bits": (4, 3), "type": "dynamic", "block_sizes": {-1: None}},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "max",
}
FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": (4, 3), "block_sizes": {-1: 128, -2: 128}, "enable": True},
                  "*input_quantizer": {"enable": False}, **_default_disabled_quantizer_cfg},
    "algorithm": "max",
}
W4A8_AWQ_BETA_CFG = {
    "quant_cfg": {"*weight_quantizer": [{"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                                        {"num_bits": (4, 3), "axis": None, "enable": True}],
                  "*input_quantizer": {"num_bits": (4, 3), "axis": None, "enable": True},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "awq_lite",
}
W4A8_NVFP4_FP8_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": (2, 1), "axis": None, "enable": True,
                                        "block_sizes": {-1: 32, "type": "dynamic", "scale_bits": (4, 3)}},
                  "*input_quantizer": {"num_bits": (4, 3), "axis": None, "enable": True},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "max",
}
W4A8_MXFP4_FP8_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": (2, 1), "enable": True,
                                        "block_sizes": {-1: 32, "type": "dynamic", "scale_bits": (8, 0)}},
                  "*input_quantizer": {"num_bits": (4, 3), "axis": None}, **_default_disabled_quantizer_cfg},
    "algorithm": None,
}
NVFP4_MLP_WEIGHT_ONLY_CFG = {
    "quant_cfg": {"*mlp*weight_quantizer": {"num_bits": (2, 1), "enable": True, "pass_through_bwd": True,
                                            "block_sizes": {-1: 32, "type": "dynamic", "scale_bits": (4, 3)}},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "max",
}
NVFP4_MLP_ONLY_CFG = {
    "quant_cfg": {"*mlp*weight_quantizer": {"num_bits": (2, 1), "enable": True, "pass_through_bwd": True,
                                            "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}},
                  "*mlp*input_quantizer": {"num_bits": (2, 1), "enable": True, "pass_through_bwd": True,
                                           "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}},
                  **_default_disabled_quantizer_cfg},
    "algorithm": "max",
}
MXFP4_MLP_WEIGHT_ONLY_CFG = {
    "quant_cfg": {"*mlp*weight_quantizer": {"num_bits": (2, 1), "enable": True, "pass_through_bwd": True,
                                            "block_sizes": {-1: 32, "type": "dynamic", "scale_bits": (8, 0)}},
                  **_default_disabled_quantizer_cfg},
    "algorithm": None,
}


# KV-cache quantisers (`*[kv]_bmm_quantizer`) exist on attention modules converted by a model
# plugin; on models without them these patterns match nothing.
FP8_KV_CFG = {"quant_cfg": {"*[kv]_bmm_quantizer": {"num_bits": (4, 3), "axis": None, "enable": True},
                            "default": {"enable": False}}, "algorithm": "max"}
FP8_AFFINE_KV_CFG = {"quant_cfg": {"*[kv]_bmm_quantizer": {"num_bits": (4, 3), "axis": None,
                                                           "bias": {-2: None, -4: None, "type": "static"}},
                                   "default": {"enable": False}}, "algorithm": "max"}
NVFP4_KV_CFG = {"quant_cfg": {"*[kv]_bmm_quantizer": {"num_bits": (2, 1), "axis": None, "enable": True,
                                                      "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}},
                              "default": {"enable": False}}, "algorithm": "max"}
NVFP4_AFFINE_KV_CFG = {"quant_cfg": {"*[kv]_bmm_quantizer": {"num_bits": (2, 1), "axis": None, "enable": True,
                                                             "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)},
                                                             "bias": {-2: None, -4: None, "type": "static"}},
                                     "default": {"enable": False}}, "algorithm": "max"}


NVFP4_KV_ROTATE_CFG = {
    "quant_cfg": {"*q_bmm_quantizer": {"enable": False, "rotate": True},
                  "*k_bmm_quantizer": {"num_bits": (2, 1), "axis": None, "enable": True, "rotate": True,
                                       "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}},
                  "*v_bmm_quantizer": {"num_bits": (2, 1), "axis": None, "enable": True,
                                       "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}}},
    "algorithm": "max",
}


def _mx(num_bits):
    return {"num_bits": num_bits, "block_sizes": {-1: 32, "type": "dynamic", "scale_bits": (8, 0)}, "enable": True}


MXFP8_DEFAULT_CFG = {"quant_cfg": {"*weight_quantizer": _mx((4, 3)), "*input_quantizer": _mx((4, 3)),
                                   **_default_disabled_quantizer_cfg}, "algorithm": None}
MXFP6_DEFAULT_CFG = {"quant_cfg": {"*weight_quantizer": _mx((3, 2)), "*input_quantizer": _mx((3, 2)),
                                   **_default_disabled_quantizer_cfg}, "algorithm": None}
MXFP4_DEFAULT_CFG = {"quant_cfg": {"*weight_quantizer": _mx((2, 1)), "*input_quantizer": _mx((2, 1)),
                                   **_default_disabled_quantizer_cfg}, "algorithm": None}
MXINT8_DEFAULT_CFG = {"quant_cfg": {"*weight_quantizer": _mx(8), "*input_quantizer": _mx(8),
                                    **_default_disabled_quantizer_cfg}, "algorithm": None}

choices = {"FP8_PER_CHANNEL_PER_TOKEN_CFG", "FP8_2D_BLOCKWISE_WEIGHT_ONLY_CFG", "W4A8_AWQ_BETA_CFG", "W4A8_NVFP4_FP8_CFG", "W4A8_MXFP4_FP8_CFG", "NVFP4_MLP_WEIGHT_ONLY_CFG", "NVFP4_MLP_ONLY_CFG", "MXFP4_MLP_WEIGHT_ONLY_CFG",
           "INT8_SMOOTHQUANT_CFG", "NVFP4_AWQ_CLIP_CFG", "NVFP4_AWQ_FULL_CFG", "MXFP8_DEFAULT_CFG", "MXFP6_DEFAULT_CFG", "MXFP4_DEFAULT_CFG", "MXINT8_DEFAULT_CFG","INT8_DEFAULT_CFG", "INT8_WEIGHT_ONLY_CFG", "FP8_DEFAULT_CFG", "INT4_BLOCKWISE_WEIGHT_ONLY_CFG",
           "INT4_AWQ_CFG", "NVFP4_DEFAULT_CFG", "NVFP4_AWQ_LITE_CFG"}


@dataclass
class QuantizerAttributeConfig:
    """Attributes of one TensorQuantizer (same field names and defaults as the reference record)."""

    enable: bool = True
    num_bits: Any = 8                     # int, or (E, M) for floating formats
    axis: Any = None                      # kept (quantisation) axis / axes; None = per tensor
    fake_quant: bool = True
    unsigned: bool = False
    narrow_range: bool = False
    learn_amax: bool = False
    type: str = "static"                  # "static" | "dynamic"
    block_sizes: dict | None = None       # {dim: size, "type": ..., "scale_bits": ...}
    bias: dict | None = None
    trt_high_precision_dtype: str = "Float"
    calibrator: Any = "max"               # "max" | "histogram" | (class, args, kwargs) | instance
    rotate: bool = False
    pass_through_bwd: bool = False

    def __post_init__(self):
        if isinstance(self.num_bits, list):
            self.num_bits = tuple(self.num_bits)
        if isinstance(self.num_bits, tuple) and not all(isinstance(x, int) and x > 0 for x in self.num_bits):
            raise ValueError("num_bits must be a positive integer or a tuple of positive integers.")
        if isinstance(self.num_bits, int):
            if self.num_bits < 1:
                raise ValueError("num_bits must be a positive integer or a tuple of positive integers.")
        elif not (isinstance(self.num_bits, tuple) and len(self.num_bits) == 2):
            raise ValueError("num_bits must be a positive integer or a tuple of positive integers.")
        if isinstance(self.num_bits, tuple):
            # reference config.py:710-746: the floating formats that exist, and only E4M3 without dynamic blocks
            if self.num_bits not in ((4, 3), (5, 2), (2, 1), (1, 2), (0, 3), (3, 0), (3, 2), (2, 3)):
                raise ValueError("Supported FPx quantization formats: FP8 (E4M3, E5M2), FP6(E3M2, E2M3), FP4(E2M1).")
            if self.num_bits != (4, 3) and (self.block_sizes is None or self.block_sizes.get("type") != "dynamic"):
                raise ValueError("Only blockwise dynamic quantization is supported with quantization formats "
                                 f"E{self.num_bits[0]}M{self.num_bits[1]}.")
        if self.learn_amax:
            raise ValueError("learn_amax is deprecated and reserved for backward compatibility.")
        if self.type not in ("static", "dynamic"):
            raise ValueError("type must be 'static' or 'dynamic'")
        if self.block_sizes is not None:
            if self.axis is not None:
                raise ValueError("axis must be None when block_sizes is not None.")
            bs = {}
            for k, v in self.block_sizes.items():
                if isinstance(k, str) and k.lstrip("-").isdigit():
                    k = int(k)
                if isinstance(k, str):
                    if k not in ("type", "scale_bits", "scale_block_sizes"):
                        raise ValueError(f"Unknown block_sizes key {k!r}")
                    if k == "scale_bits" and isinstance(v, list):
                        v = tuple(v)
                bs[k] = v
            self.block_sizes = bs

    @staticmethod
    def _get_block_quant_axes_and_sizes(block_sizes):
        if block_sizes is None:
            return None
        return {k: v for k, v in block_sizes.items() if isinstance(k, int) and v is not None}

    def dict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}


def _checked_init(init):
    """A configuration that says nothing but ``enable=True`` is refused, as the reference's validator refuses
    it (config.py:683-707): enabling needs to know what to enable."""
    def __init__(self, *args, **kwargs):
        if not args and set(kwargs) == {"enable"} and kwargs["enable"] is True:
            raise ValueError("Invalid quantizer config: Cannot specify only {'enable': True}. "
                             "Additional parameters are required when enabling quantization.")
        init(self, *args, **kwargs)
    return __init__


QuantizerAttributeConfig.__init__ = _checked_init(QuantizerAttributeConfig.__init__)


def need_calibration(config) -> bool:
    """True when ``config`` needs calibration data (reference config.py:1205-1231): any algorithm other than
    "max", or some enabled quantiser other than a weight quantiser whose ``type`` is not "dynamic".  A dynamic
    ``block_sizes`` type alone does not count as dynamic: NVFP4 activations take their second-level scale
    from a calibrated per-tensor amax."""
    if config.get("algorithm") not in ("max", None):
        return True

    def not_dynamic(c):
        return bool(c.get("enable", True) and c.get("type", "") != "dynamic"
                    and c.get("*", {}).get("enable", True))

    for name, cfg in config.get("quant_cfg", {}).items():
        if "weight_quantizer" in str(name):
            continue
        cfgs = cfg if isinstance(cfg, (list, tuple)) else [cfg]
        if any(not_dynamic(c if isinstance(c, dict) else c.to_dict()) for c in cfgs):
            return True
    return False
