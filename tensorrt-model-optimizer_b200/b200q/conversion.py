"""Model conversion: class-patch ``nn.Linear`` into ``QuantLinear`` and configure the quantisers
from a wildcard dictionary (reference: modelopt/torch/quantization/conversion.py:56-301)."""
from __future__ import annotations

import fnmatch
from contextlib import contextmanager

from torch import nn

from .config import QuantizerAttributeConfig
from .nn import QuantLinear, QuantModule, SequentialQuantizer, TensorQuantizer

__all__ = ["replace_quant_module", "set_quantizer_by_cfg", "set_quantizer_attribute",
           "set_quantizer_by_cfg_context", "convert_to_quantized_model", "register", "unregister",
           "QuantModuleRegistry"]


class _QuantModuleRegistry:
    """User-registered quantised classes by the exact type they replace (reference
    modelopt/torch/quantization/nn/modules/quant_module.py ``QuantModuleRegistry`` with
    conversion.py:330-400).  ``nn.Linear`` is built in and not listed here."""

    def __init__(self):
        self._by_original: dict[type, type] = {}

    def get(self, original_cls):
        return self._by_original.get(original_cls)

    def __contains__(self, original_cls):
        return original_cls in self._by_original

    def register(self, original_cls, quantized_cls):
        assert hasattr(quantized_cls, "_setup"), (
            "Quantized class must have a _setup method which initializes various quantizers.")
        assert issubclass(quantized_cls, original_cls), "the quantized class must derive from the class it replaces"
        self._by_original[original_cls] = quantized_cls

    def unregister(self, original_cls):
        if original_cls not in self._by_original:
            raise KeyError(f"{original_cls} is not registered")
        del self._by_original[original_cls]


QuantModuleRegistry = _QuantModuleRegistry()


def register(original_cls, quantized_cls):
    """Register ``quantized_cls`` (a subclass of ``original_cls`` with a ``_setup()`` that creates its
    quantisers and a ``forward`` that calls them) to replace modules of exactly ``original_cls``."""
    QuantModuleRegistry.register(original_cls, quantized_cls)


def unregister(original_cls):
    QuantModuleRegistry.unregister(original_cls)


def replace_quant_module(model: nn.Module):
    """Convert, in place, every ``nn.Linear`` (exact type or subclass not yet converted) and every module
    whose exact type has a registered quantised class (class patch, then ``_setup()``)."""
    for m in list(model.modules()):
        if isinstance(m, nn.Linear) and not isinstance(m, QuantModule):
            QuantLinear.convert(m)
            continue
        quantized_cls = QuantModuleRegistry.get(type(m))
        if quantized_cls is not None:
            m.__class__ = quantized_cls
            m._setup()
    return model


def _match(pattern, name: str) -> bool:
    if callable(pattern):
        return bool(pattern(name))
    return fnmatch.fnmatch(name, pattern)


def set_quantizer_attribute(model: nn.Module, wildcard_or_filter, attribute, parent_class=None):
    """Apply ``attribute`` (a dict / QuantizerAttributeConfig, or a list of them for a
    SequentialQuantizer) to every quantiser whose full name matches."""
    for name, module in list(model.named_modules()):
        if not isinstance(module, (TensorQuantizer, SequentialQuantizer)) or not _match(wildcard_or_filter, name):
            continue
        if parent_class is not None:
            parent = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
            if not isinstance(parent, parent_class):
                continue
        if isinstance(attribute, (list, tuple)):
            if not isinstance(module, SequentialQuantizer):
                parent = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
                seq = SequentialQuantizer(*(TensorQuantizer() for _ in attribute))
                seq.to(next(iter(module.buffers()), None).device if list(module.buffers()) else "cpu")
                setattr(parent, name.rpartition(".")[2], seq)
                module = seq
            module.set_from_attribute_config([_as_cfg(a, None) for a in attribute])
        else:
            if isinstance(module, SequentialQuantizer) and isinstance(attribute, dict):
                # a dictionary changes what it names in every member (reference tensor_quantizer.py:1182-1196)
                module.set_from_attribute_config([dict(attribute)] * len(module))
                continue
            if isinstance(module, SequentialQuantizer):
                parent =model.get_submodule(name.rpartition(".")[0]) if "." in name else model
                module = TensorQuantizer()
                setattr(parent, name.rpartition(".")[2], module)
            module.set_from_attribute_config(_as_cfg(attribute, module))


def _as_cfg(attribute, module):
    """Dictionaries pass through: a configured quantiser changes only what they name
    (``TensorQuantizer.set_from_attribute_config``)."""
    return attribute if isinstance(attribute, QuantizerAttributeConfig) else dict(attribute)


def set_quantizer_by_cfg(model: nn.Module, quant_cfg: dict):
    """``quant_cfg`` maps wildcards (or ``nn.<Class>`` names) to attribute dictionaries; the
    ``"default"`` entry is applied first, then the others in order.  Entries are applied as complete
    records, ``{"enable": ...}`` alone as a switch (``_full_entries``); ``set_quantizer_attribute`` with a
    dictionary changes only what the dictionary names."""
    quant_cfg = _full_entries(dict(quant_cfg))
    if "default" in quant_cfg:
        set_quantizer_attribute(model, "*", quant_cfg["default"])
        quant_cfg.pop("default")
    for pattern, cfg in quant_cfg.items():
        if isinstance(pattern, str) and pattern.startswith("nn."):
            cls = getattr(nn, pattern[3:], None)
            if cls is None:
                continue
            for sub_pattern, sub_cfg in cfg.items():
                set_quantizer_attribute(model, sub_pattern, sub_cfg, parent_class=cls)
        else:
            set_quantizer_attribute(model, pattern, cfg)


@contextmanager
def set_quantizer_by_cfg_context(model: nn.Module, quant_cfg: dict):
    """Temporarily apply ``quant_cfg`` (only switches and attributes; buffers are kept)."""
    saved = {}
    for name, m in model.named_modules():
        if isinstance(m, TensorQuantizer):
            saved[name] = {k: v for k, v in m.__dict__.items() if k.startswith("_") and k not in
                           ("_parameters", "_buffers", "_modules") and not k.startswith("_forward")
                           and not k.startswith("_backward") and not k.startswith("_state_dict")
                           and not k.startswith("_load_state") and k != "_non_persistent_buffers_set"}
    set_quantizer_by_cfg(model, quant_cfg)
    try:
        yield
    finally:
        for name, m in model.named_modules():
            if name in saved:
                m.__dict__.update(saved[name])


def _full_entries(quant_cfg: dict, strict: bool = False) -> dict:
    """The entries of a configuration dictionary as complete attribute records: what an entry does not name
    takes its default (``enable`` included), as in the reference, whose configuration model turns every entry
    into a QuantizerAttributeConfig before it is applied (config.py QuantizeConfig).  An entry that names
    nothing but ``enable`` is a switch and stays a dictionary, so that it leaves the format of a configured
    quantiser alone; with ``strict`` (the quantize() entry) ``{"enable": True}`` alone is refused there too."""
    def full(entry):
        if isinstance(entry, (list, tuple)):
            return [full(e) for e in entry]
        if isinstance(entry, dict):
            if set(entry) == {"enable"} and not (strict and entry["enable"] is True):
                return dict(entry)
            return QuantizerAttributeConfig(**entry)
        return entry

    out = {}
    for pattern, entry in quant_cfg.items():
        if isinstance(pattern, str) and pattern.startswith("nn.") and isinstance(entry, dict):
            out[pattern] = {sub: full(e) for sub, e in entry.items()}
        else:
            out[pattern] = full(entry)
    return out


def convert_to_quantized_model(model: nn.Module, config: dict):
    replace_quant_module(model)
    set_quantizer_by_cfg(model, _full_entries(config.get("quant_cfg", {}), strict=True))
    return model
