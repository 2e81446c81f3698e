"""User entry points: ``quantize``, ``calibrate``, ``compress`` and helpers (reference:
modelopt/torch/quantization/model_quant.py:53-231,499-523; compress.py:53-222)."""
from __future__ import annotations

import fnmatch
import inspect
import warnings

import torch
from torch import nn

from .conversion import convert_to_quantized_model, set_quantizer_attribute
from .model_calib import awq, max_calibrate, mse_calibrate, smoothquant
from .nn import QuantLinear, RealQuantLinear, SequentialQuantizer, TensorQuantizer
from .qtensor import pack_real_quantize_weight

__all__ = ["quantize", "calibrate", "compress", "restore_from_modelopt_state", "postprocess_amax", "disable_quantizer", "enable_quantizer",
           "print_quant_summary", "fold_weight", "modelopt_state"]

def _awq_variant(variant):
    def run(model, forward_loop=None, **opts):
        return awq(model, forward_loop, algorithm=variant, **opts)
    return run


_ALGORITHMS = {"max": max_calibrate, "mse": mse_calibrate, "smoothquant": smoothquant,
               "awq_lite": _awq_variant("awq_lite"), "awq_clip": _awq_variant("awq_clip"),
               "awq_full": _awq_variant("awq_full")}


def calibrate(model: nn.Module, algorithm="max", forward_loop=None) -> nn.Module:
    """Run a calibration algorithm on a converted model.

    ``algorithm``: ``"max"``, ``"mse"``, ``"smoothquant"``, ``"awq_lite"``, ``"awq_clip"``,
    ``"awq_full"``, ``None`` (skip), or a dict
    ``{"method": name, **options}``.  ``forward_loop(model)`` must push the calibration data
    through the model; it may be called more than once."""
    if algorithm is None:
        return model
    if forward_loop is not None and not inspect.signature(forward_loop).parameters:
        # the older calling form (reference model_quant.py:79-100): a loop over a captured model
        warnings.warn("forward_loop should take the model as its argument; a loop without arguments is "
                      "accepted for backward compatibility.", DeprecationWarning)
        bare_loop = forward_loop
        forward_loop = lambda model: bare_loop()  # noqa: E731
    opts = {}
    if isinstance(algorithm, dict):
        opts = {k: v for k, v in algorithm.items() if k != "method"}
        algorithm = algorithm["method"]
    fn = _ALGORITHMS.get(algorithm)
    if fn is None:
        raise NotImplementedError(f"calibration algorithm {algorithm!r} is outside the accelerated path "
                                  f"(built: {sorted(_ALGORITHMS)})")
    was_training = model.training
    model.eval()
    fn(model, forward_loop, **opts)
    model.train(was_training)
    _record_mode(model, f"{algorithm}_calibrate")
    return model


def quantize(model: nn.Module, config: dict, forward_loop=None) -> nn.Module:
    """Convert ``model`` in place (``nn.Linear`` -> ``QuantLinear``), configure its quantisers from
    ``config["quant_cfg"]`` and calibrate with ``config["algorithm"]``."""
    convert_to_quantized_model(model, config)
    _record_mode(model, "quantize", config)
    return calibrate(model, config.get("algorithm", "max"), forward_loop)


def compress(model: nn.Module, config=None) -> nn.Module:
    """Real-quantise the weights: every enabled weight quantiser that supports it is switched to
    real-quant mode and the weight is replaced by its packed form (``QTensorWrapper``); scales are
    kept as ``_scale`` / ``_double_scale`` buffers of the quantiser.

    ``config`` may carry ``{"compress": {pattern: bool}}`` to choose layers by name and
    ``{"quant_gemm": bool}`` (default on, as in the reference's compress.py:124-128): layers whose input and
    weight quantisers are both enabled are marked to run a registered real-quantisation GEMM."""
    from .backends.gemm_registry import disable_real_quant_gemm, enable_real_quant_gemm

    patterns = (config or {}).get("compress", {"default": True}) if isinstance(config, dict) else {"default": True}
    with SequentialQuantizer.convert_to_single_quantizer(model):
        for name, m in model.named_modules():
            if not isinstance(m, QuantLinear):
                continue
            wq = m.weight_quantizer
            chosen = patterns.get("default", False)
            for p, v in patterns.items():
                if p != "default" and fnmatch.fnmatch(name, p):
                    chosen = v
            if not (chosen and wq.is_enabled and wq._is_real_quantize_support()):
                continue
            m.__class__ = RealQuantLinear
            wq._fake_quant = False
            wq._dequantize = False
        pack_real_quantize_weight(model)
    quant_gemm = bool(config.get("quant_gemm", True)) if isinstance(config, dict) else True
    (enable_real_quant_gemm if quant_gemm else disable_real_quant_gemm)(model)
    _record_mode(model, "real_quantize", {"quant_gemm": quant_gemm})
    return model


def postprocess_amax(model: nn.Module, key: str, post_process_fn) -> nn.Module:
    """Replace the amax of every calibrated quantiser whose name matches the wildcard ``key`` by
    ``post_process_fn(amax)`` (reference model_quant.py:121-133)."""
    assert isinstance(key, str), "key should be a string"
    for name, m in model.named_modules():
        if isinstance(m, TensorQuantizer) and hasattr(m, "_amax") and fnmatch.fnmatch(name, key):
            m.amax = post_process_fn(m.amax)
    return model


def disable_quantizer(model: nn.Module, wildcard_or_filter_func):
    set_quantizer_attribute(model, wildcard_or_filter_func, {"enable": False})


def enable_quantizer(model: nn.Module, wildcard_or_filter_func):
    set_quantizer_attribute(model, wildcard_or_filter_func, {"enable": True})


def print_quant_summary(model: nn.Module):
    count = 0
    for name, m in model.named_modules():
        if isinstance(m, TensorQuantizer):
            print(f"{name:80} {m}")
            count += 1
    print(f"{count} TensorQuantizers found in model")


@torch.no_grad()
def fold_weight(model: nn.Module):
    """Replace each weight by its fake-quantised value and disable the weight quantiser."""
    for _, m in model.named_modules():
        if isinstance(m, QuantLinear) and m.weight_quantizer.is_enabled and m.weight_quantizer._fake_quant:
            m.weight.data.copy_(m.weight_quantizer(m.weight).to(m.weight.dtype))
            m.weight_quantizer.disable()


def _record_mode(model, mode, config=None):
    st = model.__dict__.setdefault("_b200q_state", [])
    st.append((mode, config))


def modelopt_state(model: nn.Module) -> dict:
    """Everything besides ``state_dict()`` that is needed to rebuild a quantised model: the modes
    applied so far with their configurations, the per-quantiser Python state (properties and buffer
    shapes, reference nn/modules/tensor_quantizer.py:1000-1072) and, for compressed models, the
    metadata of the packed weights (reference compress.py:179-193, qtensor/base_qtensor.py:130-136)."""
    from .qtensor import QTensorWrapper

    def qstate(m):
        if isinstance(m, SequentialQuantizer):
            return {"is_sequential_quantizer": True, "members": [q.get_modelopt_state() for q in m]}
        return m.get_modelopt_state()

    return {
        "modelopt_state_dict": list(model.__dict__.get("_b200q_state", [])),
        "quantizer_state": {n: qstate(m) for n, m in model.named_modules()
                            if isinstance(m, (TensorQuantizer, SequentialQuantizer))
                            and not any(isinstance(p, SequentialQuantizer) and n.startswith(pn + ".")
                                        for pn, p in model.named_modules())},
        "q_tensor_state": {n: dict(m.weight.get_state(), device=str(m.weight.device))
                           for n, m in model.named_modules()
                           if isinstance(m, QuantLinear) and isinstance(m.weight, QTensorWrapper)},
    }


@torch.no_grad()
def restore_from_modelopt_state(model: nn.Module, state: dict) -> nn.Module:
    """Rebuild the quantised structure of a freshly constructed ``model`` from ``modelopt_state``:
    modules are converted, every quantiser gets its properties and empty buffers of the recorded
    shapes, compressed layers get packed-weight placeholders.  ``model.load_state_dict(...)`` then
    restores the values (reference opt/conversion.py:444-611 for this path's modes)."""
    from .conversion import replace_quant_module, set_quantizer_by_cfg
    from .qtensor import QTensorWrapper

    assert not model.__dict__.get("_b200q_state"), "Model already has modelopt state!"
    modes = state.get("modelopt_state_dict", [])
    replace_quant_module(model)
    for mode, cfg in modes:
        if mode == "quantize" and cfg is not None:
            set_quantizer_by_cfg(model, cfg["quant_cfg"])       # also builds SequentialQuantizers
    named = dict(model.named_modules())
    for name, st in state.get("quantizer_state", {}).items():
        q = named.get(name)
        if q is None:
            raise KeyError(f"quantizer {name} of the saved state does not exist in the model")
        if st.get("is_sequential_quantizer"):
            for member, ms in zip(q, st["members"]):
                member.set_from_modelopt_state(ms)
        else:
            q.set_from_modelopt_state(st)
        q.to(next((p.device for p in model.parameters()), torch.device("cpu")))
    for name, meta in state.get("q_tensor_state", {}).items():
        m = named[name]
        m.__class__ = RealQuantLinear
        packed = torch.empty(meta["quantized_data.shape"], dtype=meta["quantized_data.dtype"], device=m.weight.device)
        m.weight = QTensorWrapper(packed, metadata=dict(meta["metadata"]))
    for mode, cfg in modes:
        if mode == "real_quantize":
            from .backends.gemm_registry import disable_real_quant_gemm, enable_real_quant_gemm
            (enable_real_quant_gemm if (cfg or {}).get("quant_gemm", True) else disable_real_quant_gemm)(model)
    model.__dict__["_b200q_state"] = list(modes)
    return model
