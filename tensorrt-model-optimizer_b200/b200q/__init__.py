"""b200q — B200 (sm_100a) kernels behind the ``modelopt.torch.quantization`` API for the
quantize / calibrate path.  ``import b200q as mtq`` gives the reference's entry points
(``quantize``, ``calibrate``, ``compress``, the ``*_CFG`` dictionaries) for this path."""
from . import _cabi, ops  # noqa: F401  (loading the library is part of importing the package)

__version__ = "0.1.0"
