"""TEST AND BENCHMARK INFRASTRUCTURE ONLY — never imported by the library.

Loads what ``oracle/build_ref.py`` compiled from the reference checkout into ``oracle/_ref/``: the
reference's own CUDA extensions (``modelopt_cuda_ext``: fake_tensor_quant*, INT4/NF4 pack kernels;
``modelopt_cuda_ext_fp8``: fake_e4m3fy*; ``modelopt_cuda_ext_mx``: fused_amax_convert) and its Triton
NVFP4 kernels (``fp4_fake_quant_block``, ``fp4_dequantize``).  They are a second oracle next to the
numpy restatement — the reference's GPU arithmetic run as it is — and the GPU-side baseline of the
benchmark.  Every loader returns None when the artefact is not there, so callers skip."""
from __future__ import annotations

import importlib.machinery
import importlib.util
import sys
from pathlib import Path

_REF = Path(__file__).resolve().parent / "_ref"
_cache: dict = {}


def _extension(name: str):
    if name in _cache:
        return _cache[name]
    mod = None
    so = _REF / name / f"{name}.so"
    if so.exists():
        import torch  # noqa: F401  (libtorch must be mapped before the module's symbols resolve)

        loader = importlib.machinery.ExtensionFileLoader(name, str(so))
        spec = importlib.util.spec_from_file_location(name, str(so), loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
    _cache[name] = mod
    return mod


def cuda_ext():
    """fake_tensor_quant, fake_tensor_quant_with_axis, INT4_quantize, INT4_dequantize, NF4_*."""
    return _extension("modelopt_cuda_ext")


def cuda_ext_fp8():
    """fake_e4m3fy(inputs, amax), fake_e4m3fy_with_axis(inputs, amax, axis)."""
    return _extension("modelopt_cuda_ext_fp8")


def cuda_ext_mx():
    """fused_amax_convert(inputs, block_size, format, scale_format, global_amax), Types."""
    return _extension("modelopt_cuda_ext_mx")


def triton_fp4():
    """The module holding fp4_fake_quant_block and fp4_dequantize (needs triton and a GPU to run)."""
    if "triton_fp4" in _cache:
        return _cache["triton_fp4"]
    mod = None
    src = _REF / "triton_ref" / "fp4_kernel.py"
    if src.exists():
        try:
            spec = importlib.util.spec_from_file_location("modelopt_ref_fp4_kernel", str(src))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[spec.name] = mod
            spec.loader.exec_module(mod)
        except ImportError:
            mod = None
    _cache["triton_fp4"] = mod
    return mod
