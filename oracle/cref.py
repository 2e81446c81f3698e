"""ctypes access to the C restatement (oracle/nvfp4_ref.c) — test / baseline infrastructure."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle_ref.so"


def load(build: bool = True) -> C.CDLL:
    if build and (not LIB.exists() or LIB.stat().st_mtime < (HERE / "nvfp4_ref.c").stat().st_mtime):
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True)
    lib = C.CDLL(str(LIB))
    lib.nvfp4_ref_amax_bf16.argtypes = [C.c_void_p, C.c_int64, C.c_int]
    lib.nvfp4_ref_amax_bf16.restype = C.c_float
    lib.nvfp4_ref_quantize_bf16.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_void_p, C.c_void_p, C.c_int]
    lib.nvfp4_ref_quantize_bf16.restype = C.c_float
    return lib


def nvfp4_quantize_bf16(lib, x_bits: np.ndarray, amax: float = -1.0, threads: int = 1, out=None):
    """x_bits: uint16 array (bf16 bit patterns), size a multiple of 16 -> (packed, scales, s2)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    nblocks = x_bits.size // 16
    packed, scales = out if out is not None else (np.empty(nblocks * 8, dtype=np.uint8),
                                                  np.empty(nblocks, dtype=np.uint8))
    s2 = lib.nvfp4_ref_quantize_bf16(x_bits.ctypes.data, nblocks, amax, packed.ctypes.data,
                                     scales.ctypes.data, threads)
    return packed, scales, np.float32(s2)
