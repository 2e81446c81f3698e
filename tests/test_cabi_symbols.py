"""The shared library loads without a GPU and exports every symbol include/b200q.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "b200q.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported_and_bound():
    from b200q import _cabi

    names = declared_functions()
    assert len(names) >= 20
    lib = ctypes.CDLL(str(_cabi.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200q.h but not exported"
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(names)


def test_argument_validation_without_gpu():
    """Bad arguments are rejected on the host before any CUDA call."""
    from b200q import _cabi

    lib = _cabi.lib
    assert lib.b200q_version() >= 100
    assert lib.b200q_amax_tensor(None, 16, 2, None, None) == -1          # NULL
    buf = ctypes.create_string_buffer(256)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.b200q_amax_tensor(p16, 16, 7, p16, None) == -2           # dtype
    assert lib.b200q_amax_tensor(p16 + 2, 16, 2, p16, None) == -3       # alignment
    assert lib.b200q_amax_tensor(p16, 0, 2, p16, None) == -4            # shape
    assert lib.b200q_fake_int_tensor(p16, p16, 16, 0, p16, 40, 0, 1, None) == -5  # bits
    assert b"aligned" in lib.b200q_strerror(-3)


def test_reference_extensions_load_without_a_gpu():
    """oracle/_ref (the reference's own CUDA extensions, built by oracle/build_ref.py where a checkout of the
    reference exists) loads without a GPU and exports what the GPU tests call.  Skipped when not built."""
    import pytest

    from oracle import ref_ext

    ext, ext8, extmx = ref_ext.cuda_ext(), ref_ext.cuda_ext_fp8(), ref_ext.cuda_ext_mx()
    if ext is None or ext8 is None or extmx is None:
        pytest.skip("oracle/_ref was not built")
    for name in ("fake_tensor_quant", "fake_tensor_quant_with_axis", "INT4_quantize", "INT4_dequantize"):
        assert callable(getattr(ext, name))
    for name in ("fake_e4m3fy", "fake_e4m3fy_with_axis"):
        assert callable(getattr(ext8, name))
    assert callable(extmx.fused_amax_convert) and hasattr(extmx.Types, "E2M1") and hasattr(extmx.Types, "E8M0")
