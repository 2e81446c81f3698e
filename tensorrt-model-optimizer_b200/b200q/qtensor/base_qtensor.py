"""Base classes of the real-quantised tensors (reference:
modelopt/torch/quantization/qtensor/base_qtensor.py:39-229)."""
from __future__ import annotations

import torch

__all__ = ["BaseQuantizedTensor", "QTensorWrapper", "pack_real_quantize_weight"]


class BaseQuantizedTensor:
    """Packed data plus the shape and dtype of the tensor it came from."""

    _quantized_data: torch.Tensor

    def __init__(self, original_shape, original_dtype, quantized_data):
        self.metadata = {"shape": original_shape, "dtype": original_dtype}
        self._quantized_data = quantized_data

    @classmethod
    def quantize(cls, input, block_size):
        raise NotImplementedError

    def dequantize(self, dtype=None, **kwarg):
        raise NotImplementedError


class QTensorWrapper(torch.nn.Parameter):
    """Makes a quantised tensor usable as ``module.weight`` (an ``nn.Parameter`` over the packed
    bytes that carries the metadata needed to rebuild the quantised-tensor object)."""

    def __new__(cls, qtensor, metadata: dict | None = None):
        data = qtensor._quantized_data if isinstance(qtensor, BaseQuantizedTensor) else qtensor
        inst = super().__new__(cls, data, requires_grad=False)
        if metadata is None:
            inst.metadata = qtensor.metadata
            inst.metadata["qtensor_class"] = qtensor.__class__
        else:
            assert all(k in metadata for k in ("qtensor_class", "shape", "dtype")), f"metadata: {metadata}"
            inst.metadata = metadata
        return inst

    def dim(self):
        return len(self.metadata["shape"])

    def to(self, *args, **kwargs):
        device, dtype, *_ = torch._C._nn._parse_to(*args, **kwargs)
        if device:
            self.data = self.data.to(device=device)
        dtype = dtype if dtype else self.metadata["dtype"]
        return QTensorWrapper(self.metadata["qtensor_class"](self.metadata["shape"], dtype, self.data))

    def get_qtensor(self):
        return self.metadata["qtensor_class"](self.metadata["shape"], self.metadata["dtype"], self.data)

    def get_state(self):
        return {"metadata": self.metadata, "quantized_data.shape": self.data.shape,
                "quantized_data.dtype": self.data.dtype}


def _nvfp4_groupable(m, wq) -> bool:
    """A weight whose real quantisation is plain NVFP4 (block 16, E4M3 block scales, nothing applied to
    the weight first): these are quantised together, two launches per device and dtype."""
    bs = wq._block_sizes or {}
    w = m.weight
    return (wq._num_bits == (2, 1) and bs.get("scale_bits") == (4, 3) and bs.get(-1) == 16
            and bs.get("type") == "dynamic" and not getattr(wq, "_rotate", False)
            and getattr(wq, "pre_quant_scale", None) is None and getattr(wq, "_bias", None) is None
            and w.dim() == 2 and w.shape[-1] % 16 == 0 and w.is_floating_point()
            and w.dtype in (torch.float32, torch.float16, torch.bfloat16)
            and (w.is_cuda or torch.cuda.is_available()))


def _pack_nvfp4_grouped(items):
    """items: [(module, weight quantiser)].  CUDA weights: one ``NvFp4Group`` (abs-max launch + quantise
    launch) per device and dtype.  Host weights: streamed through the GPU by ``pipeline.pack_host_tensors``
    and left on the host.  A quantiser that carries a calibrated ``_amax`` has it used as the global
    abs-max, as ``NVFP4QTensor.quantize`` is given it by ``_real_quantize``."""
    from .. import ops
    from ..pipeline import pack_host_tensors
    from .nvfp4_tensor import NVFP4QTensor

    def finish(m, wq, packed, scales, s2):
        wq._set_buffer("_scale", scales)
        wq._set_buffer("_double_scale", s2)
        wq._dequantize = True
        m.weight = QTensorWrapper(NVFP4QTensor(m.weight.shape, m.weight.dtype, packed))

    by = {}
    for m, wq in items:
        by.setdefault((m.weight.device, m.weight.dtype), []).append((m, wq))
    for (dev, _), lst in by.items():
        amax = [wq._amax if hasattr(wq, "_amax") and wq._amax.numel() == 1 else None for _, wq in lst]
        if dev.type == "cuda":
            grp = ops.NvFp4Group([m.weight.data for m, _ in lst], separate_outputs=True)
            packed, scales, s2 = grp.run(amax_values={i: a for i, a in enumerate(amax) if a is not None})
            for i, (m, wq) in enumerate(lst):
                finish(m, wq, packed[i], scales[i], s2[i].clone())
        else:
            res = pack_host_tensors([m.weight.data for m, _ in lst], "cuda", amax)
            for (m, wq), (p, sc, s2) in zip(lst, res):
                finish(m, wq, p, sc, s2)


def pack_real_quantize_weight(module, force_quantize: bool = False):
    """Replace the weight of every sub-module whose weight quantiser is in real-quant mode by its
    packed form (the quantiser keeps the scales as buffers).  Plain NVFP4 weights are packed together by
    the grouped kernels (``_pack_nvfp4_grouped``); every other format goes through its quantiser one
    weight at a time, as the reference does for all of them
    (modelopt/torch/quantization/qtensor/base_qtensor.py:196-229)."""
    from ..nn import SequentialQuantizer

    with torch.no_grad():
        grouped, single = [], []
        for name, m in module.named_modules():
            wq = getattr(m, "weight_quantizer", None)
            if wq is None or getattr(m, "weight", None) is None or m.weight.is_meta:
                continue
            if isinstance(wq, SequentialQuantizer):
                wq = wq[0]
            if wq.is_enabled and not wq._fake_quant and m.weight.element_size() > 1:
                if force_quantize:
                    wq._dequantize = False
                (grouped if _nvfp4_groupable(m, wq) else single).append((m, wq))
        if grouped:
            _pack_nvfp4_grouped(grouped)
        for m, wq in single:
            m.weight = QTensorWrapper(wq(m.weight))
