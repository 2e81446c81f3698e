"""b200q — B200 (sm_100a) kernels behind the ``modelopt.torch.quantization`` API for the
quantize / calibrate path.  ``import b200q as mtq`` gives the reference's entry points
(``quantize``, ``calibrate``, ``compress``, the ``*_CFG`` dictionaries) for this path."""
from . import _cabi, ops  # noqa: F401  (loading the library is part of importing the package)
from . import backends, calib, dist, export, nn, qtensor, tensor_quant, utils  # noqa: F401
from .config import *  # noqa: F401,F403
from .conversion import (QuantModuleRegistry, register, replace_quant_module, set_quantizer_attribute,  # noqa: F401
                         set_quantizer_by_cfg, set_quantizer_by_cfg_context, unregister)
from .model_calib import awq_clip, awq_lite, histogram_calibrate, max_calibrate, mse_calibrate, smoothquant  # noqa: F401
from .model_quant import (calibrate, compress, disable_quantizer, enable_quantizer, fold_weight,  # noqa: F401
                          modelopt_state, postprocess_amax, print_quant_summary, quantize,
                          restore_from_modelopt_state)

__version__ = "0.1.0"
