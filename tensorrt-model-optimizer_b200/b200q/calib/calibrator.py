"""Calibrator base class (reference: modelopt/torch/quantization/calib/calibrator.py:21-63)."""


class _Calibrator:
    """Collects statistics from tensors and turns them into an amax.

    Args:
        num_bits: bits of the quantiser the amax is for (int, or an (E, M) tuple).
        axis: quantisation axis (kept dimension); ``None`` = per tensor.
        unsigned: unsigned quantisation.
    """

    def __init__(self, num_bits=8, axis=None, unsigned=False):
        self._num_bits = num_bits
        self._axis = axis
        self._unsigned = unsigned

    def collect(self, x):
        raise NotImplementedError

    def reset(self):
        raise NotImplementedError

    def compute_amax(self, *args, **kwargs):
        raise NotImplementedError

    def __repr__(self):
        return f"num_bits={self._num_bits} axis={self._axis} unsigned={self._unsigned}"
