"""Builds the reference's own CUDA extensions (and stages its Triton NVFP4 kernels) into ``oracle/_ref/``
— TEST INFRASTRUCTURE: a second oracle and the GPU-side baseline, never imported by the library.

    python oracle/build_ref.py --ref /path/to/TensorRT-Model-Optimizer

The three extensions are compiled from the sources where they lie in the reference checkout
(modelopt/torch/quantization/src/tensor_quant.cpp + tensor_quant_gpu.cu, tensor_quant_gpu_fp8.cu,
tensor_quant_mx.cu) with torch.utils.cpp_extension for sm_100, with the flags the reference's own
loader passes (modelopt/torch/quantization/extensions.py:27-71: fast-math for the mx extension only).
Nothing of the reference is copied into the tracked tree: ``oracle/_ref/`` is git-ignored; it travels to
the GPU box with the built library.  ``triton/fp4_kernel.py`` is Python and is staged there as a file.
``oracle/ref_ext.py`` loads what this script built.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

EXTENSIONS = {
    "modelopt_cuda_ext": (["src/tensor_quant.cpp", "src/tensor_quant_gpu.cu"], []),
    "modelopt_cuda_ext_fp8": (["src/tensor_quant_gpu_fp8.cu"], []),
    "modelopt_cuda_ext_mx": (["src/tensor_quant_mx.cu"], ["--use_fast_math"]),
}


def up_to_date(ref_root: str) -> bool:
    """True when every module exists and is newer than the sources it was compiled from."""
    q = Path(ref_root) / "modelopt" / "torch" / "quantization"
    for name, (sources, _) in EXTENSIONS.items():
        so = OUT / name / f"{name}.so"
        if not so.exists() or any((q / s).stat().st_mtime > so.stat().st_mtime for s in sources):
            return False
    return (OUT / "triton_ref" / "fp4_kernel.py").exists()


def build(ref_root: str, only=None) -> list:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    q = Path(ref_root) / "modelopt" / "torch" / "quantization"
    built = []
    for name, (sources, cuda_flags) in EXTENSIONS.items():
        if only and name not in only:
            continue
        bdir = OUT / name
        bdir.mkdir(parents=True, exist_ok=True)
        load(name, [str(q / s) for s in sources], extra_cuda_cflags=cuda_flags, build_directory=str(bdir),
             verbose=False)
        # keep the module only: objects and the ninja files name paths of the build machine
        for f in bdir.iterdir():
            if f.suffix != ".so":
                f.unlink()
        built.append(name)
    tri = q / "triton" / "fp4_kernel.py"
    if tri.exists() and not only:
        (OUT / "triton_ref").mkdir(parents=True, exist_ok=True)
        shutil.copyfile(tri, OUT / "triton_ref" / "fp4_kernel.py")
        built.append("triton_ref/fp4_kernel.py")
    return built


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("MODELOPT_REFERENCE_ROOT"), required="MODELOPT_REFERENCE_ROOT" not in os.environ)
    ap.add_argument("--only", nargs="*")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not Path(a.ref).exists():
        sys.exit(f"{a.ref} does not exist: nothing built")
    if not a.force and not a.only and up_to_date(a.ref):
        print("up to date")
    else:
        print("built:", ", ".join(build(a.ref, a.only)))
