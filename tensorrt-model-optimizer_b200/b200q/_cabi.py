"""ctypes binding of ``libb200q.so`` (the C ABI declared in ``include/b200q.h``).

There is no fallback: importing this module without the built library raises, and every call
checks the returned status and raises ``RuntimeError`` with the library's own message.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libb200q.so"

F32, F16, BF16 = 0, 1, 2

_p, _i, _i64, _f, _d = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double


class NvFp4Desc(C.Structure):
    """Mirror of ``b200q_nvfp4_desc``."""

    _fields_ = [("x", _p), ("packed", _p), ("scales", _p), ("amax", _p), ("s2", _p),
                ("nblocks", _i64), ("tile_begin", _i64)]


class HistDesc(C.Structure):
    """Mirror of ``b200q_hist_desc``."""

    _fields_ = [("counts", _p), ("edges", _p), ("bin_width", C.c_float), ("nbins", _i)]


# name -> argtypes (restype is int unless listed in _RESTYPES)
SIGNATURES = {
    "b200q_strerror": [_i],
    "b200q_version": [],
    "b200q_sm_count": [],
    "b200q_amax_tensor": [_p, _i64, _i, _p, _p],
    "b200q_amax_axis": [_p, _i64, _i64, _i64, _i, _p, _p],
    "b200q_amax_blocks": [_p, _i64, _i, _i, _p, _p],
    "b200q_fake_int_tensor": [_p, _p, _i64, _i, _p, _i, _i, _i, _p],
    "b200q_fake_int_axis": [_p, _p, _i64, _i64, _i64, _i, _p, _i, _i, _i, _p],
    "b200q_fake_int_rows_dynamic": [_p, _p, _i64, _i64, _i, _p, _i, _i, _i, _p],
    "b200q_fake_e4m3_tensor": [_p, _p, _i64, _i, _p, _p],
    "b200q_fake_e4m3_axis": [_p, _p, _i64, _i64, _i64, _i, _p, _p],
    "b200q_nvfp4_quantize": [_p, _i64, _i, _p, _p, _p, _p, _p, _i, _p],
    "b200q_nvfp4_dequantize": [_p, _p, _p, _p, _i64, _i, _p],
    "b200q_nvfp4_fake": [_p, _p, _i64, _i, _p, _p],
    "b200q_nvfp4_group_tile_elems": [],
    "b200q_nvfp4_group_amax": [_p, _i, _i64, _i, _p],
    "b200q_nvfp4_group_quantize": [_p, _i, _i64, _i, _p],
    "b200q_nvfp4_group_quantize_noalloc": [_p, _i, _i, _p],
    "b200q_nvfp4_group_max_tensors_noalloc": [],
    "b200q_int4_quantize": [_p, _i64, _i, _i, _p, _p, _p, _p],
    "b200q_int4_dequantize": [_p, _p, _p, _i64, _i, _i, _p],
    "b200q_fp8_quantize": [_p, _p, _p, _i64, _i64, _i64, _i, _p],
    "b200q_int8_quantize": [_p, _p, _p, _i64, _i64, _i64, _i, _p],
    "b200q_hist_collect": [_p, _i64, _i, _i, _f, _p, _p],
    "b200q_hist_collect_open": [_p, _i64, _i, _i, _f, _i, _p, _p, _p],
    "b200q_hist_collect_shared": [_p, _i64, _i, _i, _p, _i, _p, _p, _i, _p],
    "b200q_hist_entropy": [_p, _i, _i, _i, _i, _p, _f, _p, _p, _p],
    "b200q_hist_mse": [_p, _i, _p, _d, _i, _i, _p, _p, _p],
    "b200q_hist_percentile": [_p, _i, _p, _f, _d, _p, _p],
    "b200q_hist_percentile_batch": [_p, _i, C.c_double, _p, _p],
    "b200q_mse_candidates": [_p, _i64, _i64, _i64, _i, _p, _i, _i, _i, _i, _i, _p, _p],
    "b200q_awq_scale_fake_int": [_p, _p, _p, _i64, _i64, _i, _i, _i, _i, _i, _p],
    "b200q_sq_diff_sum": [_p, _p, _i64, _i, _p, _p],
    "b200q_awq_gemm_sqerr": [_p, _p, _p, _i64, _i64, _i64, _p, _p, _p, _p],
    "b200q_awq_scale_acts": [_p, _p, _p, _i64, _i64, _i, _i, _p],
    "b200q_awq_search_fused": [_p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _i, _i, _i, _p, _p, _p, _p],
    "b200q_awq_search_prequant": [_p, _p, _p, _i, _i64, _i64, _i64, _p, _p, _p, _p],
    "b200q_fp8_gemm": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _p, _p],
    "b200q_qgemm_tile_override": [_i],
    "b200q_fp8_gemm_operand": [_p, _p, _p, _i64, _i, _i, _p],
    "b200q_nvfp4_gemm": [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _p, _p],
    "b200q_nvfp4_swizzle_scales": [_p, _p, _i64, _i64, _p],
    "b200q_awq_gemm_sqerr_splitk": [_p, _p, _p, _i64, _i64, _i64, _i, _p, _p, _p, _p, _p, _p],
    "b200q_int4_export_pack": [_p, _p, _i, _p, _i64, _i64, _i, _i, _p],
    "b200q_nvfp4_quantize_blocks": [_p, _i64, _i, _i, _p, _p, _p, _p, _p, _i, _p],
    "b200q_nvfp4_fake_blocks": [_p, _p, _i64, _i, _i, _p, _p],
    "b200q_nvfp4_dequantize_blocks": [_p, _p, _p, _p, _i64, _i, _i, _p],
    "b200q_awq_clip_loss": [_p, _p, _p, _p, _i, _p, _i64, _i64, _i, _i, _i, _i, _i, _i, _p],
    "b200q_hadamard": [_p, _p, _i64, _i, _i, _f, _p],
    "b200q_mx_fake": [_p, _p, _i64, _i, _i, _i, _p],
    "b200q_mxfp4_quantize": [_p, _i64, _i, _i, _p, _p, _p],
}
_RESTYPES = {"b200q_strerror": C.c_char_p}
_NO_STATUS = {"b200q_strerror", "b200q_version", "b200q_sm_count", "b200q_nvfp4_group_tile_elems",
              "b200q_nvfp4_group_max_tensors_noalloc", "b200q_qgemm_tile_override"}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python tensorrt-model-optimizer_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the kernels)")
    lib = C.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of sync
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, _i)
    return lib


lib = _load()


class B200QError(RuntimeError):
    def __init__(self, name: str, status: int):
        self.status = status
        super().__init__(f"{name} failed: {lib.b200q_strerror(status).decode()} (status {status})")


def call(name: str, *args) -> int:
    """Call an entry point; raise on a non-zero status."""
    r = getattr(lib, name)(*args)
    if name not in _NO_STATUS and r != 0:
        raise B200QError(name, r)
    return r
