"""Real-quantised GEMM back ends of ``RealQuantLinear`` (reference:
modelopt/torch/quantization/backends/__init__.py)."""
from .gemm_registry import (disable_real_quant_gemm, enable_real_quant_gemm, gemm_registry,  # noqa: F401
                            is_real_quant_gemm_enabled)
from .fp8_per_tensor_gemm import Fp8PerTensorLinear, fp8_per_tensor_gemm  # noqa: F401
from .nvfp4_gemm import Nvfp4Linear, nvfp4_gemm  # noqa: F401
from ..ops import check_qgemm_status as check_gemm_status, qgemm_status as gemm_status  # noqa: F401,E402
