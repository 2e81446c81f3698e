"""CPU oracle for the quantize / calibrate hot path — TEST INFRASTRUCTURE, not a product path.

A numpy restatement of the arithmetic ModelOpt 0.40 performs on this path, written from the cited
reference lines and pinned against golden vectors produced by the reference itself
(``tests/golden/make_golden.py`` imports the reference and stores its inputs and outputs).  Only
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` may import it.  The library in ``tensorrt-model-optimizer_b200/`` never does.

Conventions: tensors are float32 numpy arrays holding values that are exactly representable in
the tensor's element type ``T`` ("f32", "f16" or "bf16"); wherever the reference rounds an
intermediate to ``T`` the oracle calls :func:`round_to`.  All float32 numpy arithmetic is IEEE
round-to-nearest-even, the same as the torch CPU kernels the reference runs.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

# --------------------------------------------------------------------------- element types -----


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 (round-to-nearest-even) -> float32."""
    x = np.ascontiguousarray(x, dtype=F32)
    u = x.view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = (u + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = r.view(F32).copy()
    nan = np.isnan(x)
    out[nan] = np.nan
    return out


def round_to(x: np.ndarray, T: str) -> np.ndarray:
    if T == "f32":
        return np.asarray(x, dtype=F32)
    if T == "f16":
        with np.errstate(over="ignore"):
            return np.asarray(x, dtype=F32).astype(np.float16).astype(F32)
    if T == "bf16":
        return round_bf16(x)
    raise ValueError(T)


# --------------------------------------------------------------------------- E4M3 / E2M1 -------

def _e4m3_table() -> np.ndarray:
    v = np.zeros(127, dtype=np.float64)
    for c in range(127):
        e, m = c >> 3, c & 7
        v[c] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
    return v


_E4M3 = _e4m3_table()  # codes 0x00..0x7E -> value (0x7E = 448)


def e4m3_encode(x: np.ndarray, mode: str) -> np.ndarray:
    """float32 -> E4M3 code (uint8), round-to-nearest-even.

    mode "sat":   |x| > 448 saturates to 448, NaN -> 0x7F (what cvt.rn.satfinite / __nv_fp8_e4m3
                  do; modelopt/torch/quantization/src/tensor_quant_gpu_fp8.cu:42).
    mode "torch": torch's ``.to(torch.float8_e4m3fn)``: |x| up to 464 rounds to 448, anything
                  larger and NaN become the NaN code with the sign kept
                  (modelopt/torch/quantization/qtensor/nvfp4_tensor.py:91, fp8_tensor.py:107).
    """
    x = np.asarray(x, dtype=F32)
    a = np.abs(x).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    ac = np.minimum(np.nan_to_num(a, nan=0.0), 448.0)
    hi = np.searchsorted(_E4M3, ac, side="left")          # first value >= a
    hi = np.minimum(hi, 126)
    lo = np.maximum(hi - 1, 0)
    vlo, vhi = _E4M3[lo], _E4M3[hi]
    mid = (vlo + vhi) / 2.0
    take_hi = (ac > mid) | ((ac == mid) & ((hi & 1) == 0))
    take_hi |= ac >= vhi
    code = np.where(take_hi, hi, lo).astype(np.uint8)
    if mode == "sat":
        code = np.where(np.isnan(a), np.uint8(0x7F), code | sign).astype(np.uint8)
    elif mode == "torch":
        bad = np.isnan(a) | (a > 464.0)
        code = np.where(bad, np.uint8(0x7F) | sign, code | sign).astype(np.uint8)
    else:
        raise ValueError(mode)
    return code


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    mag = (code & 0x7F).astype(np.int64)
    val = np.where(mag == 0x7F, np.nan, _E4M3[np.minimum(mag, 126)])
    val = np.where(code & 0x80, -val, val)
    return val.astype(F32)


E2M1_BOUNDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=F32)
E2M1_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, 0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=F32)


def e2m1_encode(v: np.ndarray) -> np.ndarray:
    """NVFP4QTensor._cast_fp4 (modelopt/torch/quantization/qtensor/nvfp4_tensor.py:119-140):
    sign bit from ``v < 0``; ordinal = number of bounds below |v|, plus one on the three ties
    0.75, 1.75, 3.5 (which makes every tie round to the even code); NaN sorts past every bound."""
    v = np.asarray(v, dtype=F32)
    sign = (v < 0).astype(np.uint8)
    a = np.abs(v)
    ordn = np.searchsorted(E2M1_BOUNDS, a, side="left").astype(np.uint8)
    ordn = np.where(np.isnan(a), np.uint8(7), ordn)
    tie = (a == F32(0.75)) | (a == F32(1.75)) | (a == F32(3.5))
    return ((sign << 3) + ordn + tie.astype(np.uint8)).astype(np.uint8)


# --------------------------------------------------------------------------- amax --------------

def reduce_amax(x: np.ndarray, axis=None, keepdims=True) -> np.ndarray:
    """modelopt/torch/quantization/utils.py:155-188: max(|max|, |min|) over the reduce axes."""
    x = np.asarray(x, dtype=F32)
    if axis is None:
        return np.maximum(np.abs(x.max()), np.abs(x.min())).astype(F32)
    axis = (axis,) if isinstance(axis, int) else tuple(axis)
    return np.maximum(np.abs(x.max(axis=axis, keepdims=keepdims)),
                      np.abs(x.min(axis=axis, keepdims=keepdims))).astype(F32)


def quant_axis_to_reduce_axis(ndim: int, axis):
    """utils.py:137-152."""
    if axis is None:
        return None
    axis = axis if isinstance(axis, (list, tuple)) else [axis]
    return tuple(i for i in range(ndim) if i not in axis and (i - ndim) not in axis)


def reduce_block_amax(x: np.ndarray, block: int) -> np.ndarray:
    """utils.py:52-98 for block_sizes={-1: block}."""
    x = np.asarray(x, dtype=F32)
    assert x.shape[-1] % block == 0
    return reduce_amax(x.reshape(*x.shape[:-1], x.shape[-1] // block, block), axis=-1, keepdims=False)


def pad_last(x: np.ndarray, block: int) -> np.ndarray:
    """reduce_block_padding on the last dim (utils.py:101-134)."""
    rem = x.shape[-1] % block
    if rem == 0:
        return x
    pad = [(0, 0)] * (x.ndim - 1) + [(0, block - rem)]
    return np.pad(x, pad)


# --------------------------------------------------------------------------- fake quant --------

EPS24 = F32(1.0 / (1 << 24))


def fake_int(x: np.ndarray, amax: np.ndarray, num_bits=8, unsigned=False, narrow_range=True,
             T="f32", cpu_flavour=False) -> np.ndarray:
    """Integer fake quantisation.

    GPU kernel (modelopt/torch/quantization/src/tensor_quant_gpu.cu:38-73): bound =
    2^(bits-1+unsigned)-1, lo = -(bound + !narrow); amax < 2^-24 -> 0; scale = bound/amax;
    clamp(rint(x*scale), lo, bound)/scale, cast to T.  ``cpu_flavour`` switches to the two
    differences of the torch fallback (tensor_quant.py:574-612): amax <= 2^-24 -> 0 and lo = 0 when
    unsigned.  ``amax`` broadcasts against ``x``.
    """
    x = np.asarray(x, dtype=F32)
    amax = np.asarray(amax, dtype=F32)
    bound = F32(2.0 ** (num_bits - 1 + int(unsigned)) - 1.0)
    lo = -bound if narrow_range else -bound - F32(1)
    if cpu_flavour and unsigned:
        lo = F32(0)
    dead = (amax <= EPS24) if cpu_flavour else (amax < EPS24)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        scale = (bound / amax).astype(F32)
        q = np.rint((x * scale).astype(F32))
        q = np.where(q > bound, bound, q)
        q = np.where(q < lo, lo, q).astype(F32)
        out = (q / scale).astype(F32)
    out = np.where(np.broadcast_to(dead, out.shape), F32(0), out)
    return round_to(out, T)


def fake_e4m3(x: np.ndarray, amax, T="f32", eager=False) -> np.ndarray:
    """FP8 E4M3 fake quantisation.

    Kernel flavour (src/tensor_quant_gpu_fp8.cu:35-101): scale = 448/amax and inv = 1/scale are
    true divisions, T(float(e4m3_satfinite(x*scale))*inv); amax None -> plain cast.
    ``eager`` restates ``_fp8_eager`` (tensor_quant.py:45-54) instead, where Python's
    ``448.0 / tensor`` and ``1 / tensor`` evaluate as ``tensor.reciprocal() * scalar``, which can
    differ from the true quotient in the last bit (the cast itself is the same while x*scale stays
    within the E4M3 range)."""
    x = np.asarray(x, dtype=F32)
    if amax is None:
        return round_to(e4m3_decode(e4m3_encode(x, "sat")), T)
    amax = np.asarray(amax, dtype=F32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        if eager:
            scale = ((F32(1.0) / amax).astype(F32) * F32(448.0)).astype(F32)
        else:
            scale = (F32(448.0) / amax).astype(F32)
        inv = (F32(1.0) / scale).astype(F32)
        y = e4m3_decode(e4m3_encode((x * scale).astype(F32), "sat"))
        return round_to((y * inv).astype(F32), T)


# --------------------------------------------------------------------------- NVFP4 -------------

def nvfp4_scale2(amax) -> np.float32:
    """weights_scaling_factor_2 = amax / (6*448) (nvfp4_tensor.py:55-60,94-97)."""
    return (F32(amax) / F32(2688.0)).astype(F32)


def nvfp4_block_scales(x: np.ndarray, s2, block=16, cast="torch") -> np.ndarray:
    """get_weights_scaling_factor (nvfp4_tensor.py:62-92) -> E4M3 codes [.., K/block]."""
    bamax = reduce_block_amax(x, block)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        t = (bamax / (F32(6.0) * F32(s2))).astype(F32)
    t = np.where(t == 0, F32(1.0), t)
    return e4m3_encode(t, cast)


def nvfp4_quantize(x: np.ndarray, block=16, amax=None, s2=None, scales=None, cast="torch"):
    """NVFP4QTensor.quantize, torch path (nvfp4_tensor.py:142-232).

    Returns (packed uint8 [.., K/2], scale codes uint8 [.., K/block], s2 float32)."""
    x = pad_last(np.asarray(x, dtype=F32), block)
    if s2 is None:
        s2 = nvfp4_scale2(reduce_amax(x) if amax is None else amax)
    s2 = F32(s2)
    if scales is None:
        scales = nvfp4_block_scales(x, s2, block, cast)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        d = (e4m3_decode(scales) * s2).astype(F32)
        v = (x.reshape(*x.shape[:-1], -1, block) / d[..., None]).astype(F32).reshape(x.shape)
    q = e2m1_encode(v)
    packed = ((q[..., 1::2] << 4) | q[..., 0::2]).astype(np.uint8)
    return packed, scales, s2


def nvfp4_dequantize(packed: np.ndarray, scales: np.ndarray, s2, block=16, T="f32") -> np.ndarray:
    """NVFP4QTensor.dequantize, standard path (nvfp4_tensor.py:279-297)."""
    q = np.empty((*packed.shape[:-1], packed.shape[-1] * 2), dtype=np.uint8)
    q[..., 1::2] = packed >> 4
    q[..., 0::2] = packed & 0x0F
    vals = E2M1_VALUES[q]
    with np.errstate(invalid="ignore", over="ignore"):
        d = (e4m3_decode(scales) * F32(s2)).astype(F32)
        out = (vals.reshape(*vals.shape[:-1], -1, block) * d[..., None]).astype(F32)
    return round_to(out.reshape(vals.shape), T)


def nvfp4_fake(x: np.ndarray, amax, block=16, T="f32") -> np.ndarray:
    """NVFP4 fake quantisation = dequantize(quantize(x)) with the saturating block-scale cast."""
    packed, scales, s2 = nvfp4_quantize(x, block, amax=amax, cast="sat")
    return nvfp4_dequantize(packed, scales, s2, block, T)


# --------------------------------------------------------------------------- INT4 --------------

def _roundf(z: np.ndarray) -> np.ndarray:
    """C roundf: half away from zero."""
    r = np.trunc(z)
    frac = np.abs(z - r)
    return r + np.where(frac >= 0.5, np.sign(z), 0).astype(F32)


def int4_scales(x: np.ndarray, block: int, T: str) -> np.ndarray:
    """scales = 7 / block_amax (qtensor/int4_tensor.py:58-64).  Python evaluates ``int / tensor``
    as ``tensor.reciprocal() * int`` in the tensor's type: T(T(1/amax) * 7)."""
    flat = pad_last(np.asarray(x, dtype=F32).reshape(-1), block).reshape(-1, block)
    bamax = reduce_amax(flat, axis=-1, keepdims=True)
    with np.errstate(divide="ignore", over="ignore"):
        rcp = round_to((F32(1.0) / bamax).astype(F32), T)
        return round_to((rcp * F32(7.0)).astype(F32), T)


def int4_quantize(x: np.ndarray, block: int, T="f32", scales=None, flavour="kernel"):
    """INT4QTensor.quantize (qtensor/int4_tensor.py:39-88).

    flavour "kernel": the CUDA kernel the reference uses on GPU (src/tensor_quant_gpu.cu:310-340):
      y = T(x*scale); clamp to [-8,7]; z = T(y+8); u = roundf(z); byte = u[2j]<<4 | u[2j+1].
    flavour "cpu": the torch fallback (int4_tensor.py:70-84): T(x*scale).round() (half-even),
      clamp, +8 — differs from the kernel at .5 ties and where T(y+8) rounds.
    Returns (packed uint8 [n/2], scales float32-valued-in-T [nblk,1])."""
    flat = pad_last(np.asarray(x, dtype=F32).reshape(-1), block).reshape(-1, block)
    if scales is None:
        scales = int4_scales(x, block, T)
    scales = np.asarray(scales, dtype=F32).reshape(-1, 1)
    with np.errstate(invalid="ignore", over="ignore"):
        y = round_to((flat * scales).astype(F32), T)
    if flavour == "kernel":
        y = np.fmax(F32(-8), np.fmin(F32(7), y))
        z = round_to((y + F32(8)).astype(F32), T)
        u = _roundf(z).astype(np.int64)
    else:
        u = (np.clip(np.rint(y), -8, 7) + 8).astype(np.int64)
    u = (u & 0xF).astype(np.uint8).reshape(-1)
    packed = ((u[0::2] << 4) | u[1::2]).astype(np.uint8)
    return packed, scales


def int4_dequantize(packed: np.ndarray, scales: np.ndarray, block: int, T="f32") -> np.ndarray:
    """INT4_dequantize (src/tensor_quant_gpu.cu:261-279): T(T(nibble-8)/scale)."""
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1)
    hi = (packed >> 4).astype(F32) - F32(8)
    lo = (packed & 0xF).astype(F32) - F32(8)
    vals = np.stack([hi, lo], axis=-1).reshape(-1, block)
    with np.errstate(divide="ignore", invalid="ignore"):
        return round_to((vals / np.asarray(scales, dtype=F32).reshape(-1, 1)).astype(F32), T).reshape(-1)


# --------------------------------------------------------------------------- FP8 / INT8 real ---

def fp8_quantize(x: np.ndarray, scales: np.ndarray, T="f32") -> np.ndarray:
    """FP8QTensor.quantize core (qtensor/fp8_tensor.py:107): (x / scales) in T, torch e4m3 cast.
    ``scales`` broadcasts against ``x`` and holds T-representable values."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        q = round_to((np.asarray(x, F32) / np.asarray(scales, F32)).astype(F32), T)
    return e4m3_encode(q, "torch")


def int8_quantize(x: np.ndarray, scales: np.ndarray, T="f32") -> np.ndarray:
    """INT8QTensor.quantize core (qtensor/int8_tensor.py:88): round-half-even of the T quotient,
    clamp to [-128, 127]."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        q = round_to((np.asarray(x, F32) / np.asarray(scales, F32)).astype(F32), T)
    return np.clip(np.rint(q), -128, 127).astype(np.int8)


# --------------------------------------------------------------------------- histogram ---------

def hist_bins(x: np.ndarray, nbins: int, range_max) -> np.ndarray:
    """Equal-width binning of |x| on [0, range_max] as the CUDA torch.histc does it (the kernel
    HistogramCalibrator.collect reaches on GPU, modelopt/torch/quantization/calib/histogram.py:118,128):
    bin = int(|x| * nbins / range_max) in float32, the right edge falls in the last bin, values
    outside the range are not counted.  Returns int64 counts."""
    a = np.abs(np.asarray(x, dtype=F32)).reshape(-1)
    rm = F32(range_max)
    a = a[a <= rm]
    b = ((a * F32(nbins)).astype(F32) / rm).astype(F32).astype(np.int64)
    b = np.minimum(b, nbins - 1)
    return np.bincount(b, minlength=nbins).astype(np.int64)


def hist_bins_open(x: np.ndarray, nbins: int, range_max, capacity: int):
    """Open-ended variant of hist_bins: bin width range_max / nbins, bins continue to `capacity`;
    returns (int64 counts [capacity], number of samples beyond the last bin or not finite).
    Same arithmetic as the reference applies after it has extended its range
    (modelopt/torch/quantization/calib/histogram.py:119-130), with the first batch's (nbins, range)."""
    a = np.abs(np.asarray(x, dtype=F32)).reshape(-1)
    rm = F32(range_max)
    cap_range = F32(np.float64(rm) * capacity / nbins) if capacity != nbins else rm
    with np.errstate(invalid="ignore"):
        ok = a <= cap_range
    beyond = int((~ok).sum())
    a = a[ok]
    b = ((a * F32(nbins)).astype(F32) / rm).astype(F32).astype(np.int64)
    b = np.where(a <= rm, np.minimum(b, nbins - 1), np.minimum(b, capacity - 1))
    return np.bincount(b, minlength=capacity).astype(np.int64), beyond


class HistogramOracle:
    """HistogramCalibrator.collect with torch_hist=True (calib/histogram.py:77-130) — range set by
    the first batch, later batches extend the bin count at the first batch's width."""

    def __init__(self, num_bins=2048):
        self.num_bins = num_bins
        self.hist = None
        self.edges = None

    def collect(self, x: np.ndarray):
        a = np.abs(np.asarray(x, dtype=F32))
        x_max = F32(a.max())
        if self.hist is None:
            self.hist = hist_bins(a, self.num_bins, x_max)
            self.edges = np.linspace(0, x_max, self.num_bins + 1, dtype=np.float64).astype(F32)
        else:
            if x_max > self.edges[-1]:
                width = F32(self.edges[1] - self.edges[0])
                self.num_bins = int(np.ceil(F32(x_max / width)))
                n = int(np.ceil(np.float64(F32(x_max + width)) / np.float64(width)))
                self.edges = (np.arange(n, dtype=np.float64) * np.float64(width)).astype(F32)
            h = hist_bins(a, self.num_bins, self.edges[-1])
            h[: self.hist.size] += self.hist
            self.hist = h


def percentile_amax(hist: np.ndarray, edges: np.ndarray, percentile: float):
    """_compute_amax_percentile (calib/histogram.py:328-343)."""
    total = hist.sum()
    cdf = np.cumsum(hist / total)
    idx = np.searchsorted(cdf, percentile / 100)
    return F32(edges[idx]), int(idx)


def entropy_amax(hist: np.ndarray, edges: np.ndarray, num_bits=8, unsigned=False, stride=1,
                 start_bin=128):
    """_compute_amax_entropy (calib/histogram.py:210-282), vectorised per candidate: merge the
    first i bins into 2^(bits-1+unsigned) levels, spread each level's mass evenly over its
    non-empty source bins, KL(reference || candidate) with the clipped tail folded into the
    reference's last bin; the LAST minimum wins."""
    bins = np.array(hist, dtype=np.int64)
    bins[0] = bins[1]
    nlev = 1 << (num_bits - 1 + int(unsigned))
    divs = []
    for i in range(start_bin, len(bins) + 1, stride):
        space = np.linspace(0, i, num=nlev + 1)
        dig = np.digitize(np.arange(i), space) - 1
        nz = bins[:i] != 0
        level_sum = np.bincount(dig[nz], weights=bins[:i][nz].astype(np.float64), minlength=nlev)
        level_cnt = np.bincount(dig[nz], minlength=nlev)
        with np.errstate(divide="ignore", invalid="ignore"):
            level_avg = np.where(level_cnt > 0, level_sum / level_cnt, 0.0)
        new_density = np.where(nz, level_avg[dig], 0.0)
        ref = bins[:i].astype(np.float64).copy()
        ref[-1] += bins[i:].sum()
        divs.append(_kl(ref, new_density))
    divs = np.array(divs)
    last_argmin = len(divs) - 1 - int(np.argmin(divs[::-1]))
    return F32(edges[last_argmin * stride + start_bin])


def _kl(pk: np.ndarray, qk: np.ndarray) -> float:
    """scipy.stats.entropy(pk, qk): both normalised to sum 1, sum(pk*log(pk/qk)), inf where
    qk == 0 < pk."""
    pk = pk / pk.sum()
    qk = qk / qk.sum()
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(pk > 0, pk * np.log(pk / qk), 0.0)
    t = np.where((pk > 0) & (qk == 0), np.inf, t)
    return float(t.sum())


# --------------------------------------------------------------------------- export packers ----

def export_scaling_factor(w: np.ndarray, group: int) -> np.ndarray:
    """get_scaling_factor_from_weight (modelopt/torch/export/quant_utils.py:68-91): fp32 amax/7 per
    (row, group) when group > 0, amax/127 per row when group == 0; zeros become 1."""
    w = np.asarray(w, dtype=F32)
    if group:
        amax = np.abs(w.reshape(w.shape[0], -1, group)).max(-1)
        s = (amax / F32(7.0)).astype(F32)
    else:
        s = (np.abs(w).max(-1) / F32(127.0)).astype(F32)
    s[s == 0] = 1.0
    return s


def pack_int4_export(w: np.ndarray, scales: np.ndarray, T="f32", scales_in_T=False) -> np.ndarray:
    """pack_int4_in_uint8 (quant_utils.py:697-738) for 2-D weights: signed nibbles
    clamp(round_half_even(w/scale), -8, 7), byte [r, c] = q[2r, c] & 15 | (q[2r+1, c] & 15) << 4."""
    w = np.asarray(w, dtype=F32)
    block = w.shape[1] // scales.shape[1]
    se = np.repeat(np.asarray(scales, dtype=F32), block, axis=1)
    q = (w / se).astype(F32)
    if scales_in_T:
        q = round_to(q, T)
    q = np.clip(np.rint(q), -8, 7).astype(np.int8)
    lo = q[0::2].astype(np.uint8) & 0x0F
    hi = q[1::2].astype(np.uint8) & 0x0F
    return (lo | (hi << 4)).astype(np.uint8)


# --------------------------------------------------------------------------- MX formats --------
# Element formats: name -> (exponent bits, mantissa bits, bias, max); "int8" handled apart.
MX_FORMATS = {"e4m3": (4, 3, 7, 448.0), "e5m2": (5, 2, 15, 57344.0), "e2m1": (2, 1, 1, 6.0),
              "e3m2": (3, 2, 3, 28.0), "e2m3": (2, 3, 1, 7.5), "int8": (0, 0, 0, 127.0)}


def minifloat_round(a: np.ndarray, fmt: str) -> np.ndarray:
    """Non-negative fp32 -> nearest value of the format (ties to even), saturating at its max.
    Restates convert_to_types (modelopt/torch/quantization/src/tensor_quant_mx.h:72-186): the
    table formats' bounds are the midpoints and its tie rule picks the even mantissa."""
    a = np.asarray(a, np.float32)
    _, mbits, bias, fmax = MX_FORMATS[fmt]
    if fmt == "int8":
        return np.clip(np.rint(a), -127, 127).astype(np.float32)
    _, ex = np.frexp(a)                       # a = m * 2^ex, m in [0.5, 1)
    e = np.maximum(ex - 1, 1 - bias)          # subnormals share the smallest normal exponent
    quantum = np.ldexp(np.float32(1), (e - mbits).astype(np.int32)).astype(np.float32)
    r = (np.rint(a / quantum) * quantum).astype(np.float32)
    r = np.where(np.isnan(a) | (r > fmax), np.float32(fmax), r)
    return r.astype(np.float32)


def mx_unscale_exponent(amax: np.ndarray, fmt: str) -> np.ndarray:
    """clamp(ceil(log2(amax / format_max))) read from the bits of the fp32 quotient
    (compute_scale_e8m0_NV, modelopt/torch/quantization/src/tensor_quant_mx.cu:105-137)."""
    ratio = (np.asarray(amax, np.float32) / np.float32(MX_FORMATS[fmt][3])).astype(np.float32)
    u = ratio.view(np.uint32)
    ef = ((u >> 23) & 0xFF).astype(np.int32)
    sf = (u & 0x7FFFFF).astype(np.int64)
    up = (sf > 0) & (ef != 0xFE) & ~((ef == 0) & (sf <= 0x400000))
    return np.where(up, ef - 126, ef - 127).astype(np.int32)


def mx_fake(x: np.ndarray, block: int, fmt: str, T="f32") -> np.ndarray:
    """MX fake quantisation over the last dim (amax_and_convert_kernel + quantize,
    modelopt/torch/quantization/src/tensor_quant_mx.cu:36-54,239-294); ragged tails are padded
    with zeros for the block amax.  A zero input gives +0 here (the reference leaves its sign
    variable unset for x == 0)."""
    x = np.asarray(x, np.float32)
    k = x.shape[-1]
    xp = pad_last(x, block)
    blocks = xp.reshape(-1, block)
    amax = np.abs(blocks).max(axis=1)
    e = mx_unscale_exponent(amax, fmt)
    e = np.where((amax == 0) | ~np.isfinite(amax), 0, e)
    scale = np.ldexp(np.float32(1), -e).astype(np.float32)[:, None]
    unscale = np.ldexp(np.float32(1), e).astype(np.float32)[:, None]
    with np.errstate(over="ignore", invalid="ignore"):
        q = minifloat_round((np.abs(blocks) * scale).astype(np.float32), fmt)
        y = np.copysign((q * unscale).astype(np.float32), blocks)
    y = y.reshape(xp.shape)[..., :k]
    return round_to(y, T)


def mxfp4_quantize(x: np.ndarray, block=32):
    """-> (packed uint8 [..., K/2], scale bytes [numel/block, 1]); MXFP4QTensor.quantize
    (modelopt/torch/quantization/qtensor/mxfp4_tensor.py:38-81): ties go to the smaller
    magnitude and every value that is not > 0 carries the sign bit."""
    x = np.asarray(x, np.float32)
    b = x.reshape(-1, block)
    amax = np.abs(b).max(axis=1, keepdims=True)
    with np.errstate(divide="ignore"):
        e = np.ceil(np.maximum(np.log2((amax / np.float32(6.0)).astype(np.float32)), np.float32(-127)))
    q = (b / np.exp2(e).astype(np.float32)).astype(np.float32)
    bounds = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    code = (np.abs(q)[..., None] > bounds).sum(-1).astype(np.uint8)
    code = code + np.where(q > 0, 0, 8).astype(np.uint8)
    code = code.reshape(*x.shape[:-1], x.shape[-1] // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8)
    return packed, (e + 127).astype(np.uint8)


def mxfp4_dequantize(packed: np.ndarray, scales: np.ndarray, block=32, T="f32") -> np.ndarray:
    """MXFP4QTensor.dequantize (modelopt/torch/quantization/qtensor/mxfp4_tensor.py:83-143)."""
    codes = np.stack([packed & 0xF, packed >> 4], axis=-1).reshape(*packed.shape[:-1], -1)
    mags = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float32)[codes & 7]
    v = np.where(codes & 8, -mags, mags).astype(np.float32)
    v = v.reshape(-1, block) * np.exp2(scales.reshape(-1, 1).astype(np.float32) - 127).astype(np.float32)
    return round_to(v.reshape(codes.shape).astype(np.float32), T)


# --------------------------------------------------------------------------- real-quant GEMMs ---
# The reference hands these products to library kernels (torch._scaled_mm, and TensorRT-LLM's
# nvfp4_gemm, which is not in the reference tree): the oracle is the defining sum in float64, so a
# comparison with it carries the fp32-accumulation tolerance stated in the tests.

def fp8_to_gemm_operand(x: np.ndarray, scale, T="f32", fused=False) -> np.ndarray:
    """_to_fp8 (backends/fp8_per_tensor_gemm.py:35-37): (x / scale).clamp(-448, 448).to(e4m3) with an
    fp32 0-dim scale: the quotient float(x) / scale is rounded to x's dtype (eager evaluation;
    ``fused`` keeps it in fp32, as a compiled graph of the expression does)."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        q = (np.asarray(x, F32) / F32(scale)).astype(F32)
        if not fused:
            q = round_to(q, T)
    return e4m3_encode(np.clip(q, F32(-448.0), F32(448.0)), "torch")


def fp8_gemm(a8: np.ndarray, b8: np.ndarray, scale_a, scale_b, bias=None, T="f32") -> np.ndarray:
    """_fp8_gemm_impl (backends/fp8_per_tensor_gemm.py:41-55): a8 [m, k], b8 [n, k] E4M3 codes;
    T(sum_k a b * scale_a * scale_b + bias)."""
    acc = e4m3_decode(a8).astype(np.float64) @ e4m3_decode(b8).astype(np.float64).T
    y = acc * np.float64(F32(scale_a)) * np.float64(F32(scale_b))
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return round_to(y.astype(F32), T)


def nvfp4_gemm(a4: np.ndarray, sfa: np.ndarray, b4: np.ndarray, sfb: np.ndarray, alpha, bias=None,
               T="f32") -> np.ndarray:
    """_fp4_linear (backends/nvfp4_gemm.py:33-69): a4 [m, k/2], b4 [n, k/2] packed E2M1, sfa
    [m, k/16], sfb [n, k/16] E4M3 codes (row-major); T(T(alpha * sum) + bias)."""
    a = nvfp4_dequantize(a4, sfa, 1.0).astype(np.float64)
    b = nvfp4_dequantize(b4, sfb, 1.0).astype(np.float64)
    y = round_to(((a @ b.T) * np.float64(F32(alpha))).astype(F32), T)
    if bias is not None:
        y = round_to((y + np.asarray(bias, F32)).astype(F32), T)
    return y


def nvfp4_swizzle_scales(scales: np.ndarray) -> np.ndarray:
    """Block scales [rows, cols] (bytes) in the 128-row x 4-scale tile order of the block-scaled
    tensor-core instructions: byte (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4 of tile
    [r / 128][c / 4]; rows padded to 128, cols to 16."""
    rows, cols = scales.shape
    rt, ct = -(-rows // 128), -(-cols // 16) * 4
    padded = np.zeros((rt * 128, ct * 4), dtype=np.uint8)
    padded[:rows, :cols] = scales
    t = padded.reshape(rt, 4, 32, ct, 4)            # [row tile, r / 32, r % 32, col tile, c % 4]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(-1)


# --------------------------------------------------------------------------- awq_lite ----------
# modelopt/torch/quantization/model_calib.py:588-627 (helpers) and :645-690 (the patched forward).
# Statistics are reduced in the tensor dtype T (torch accumulates a bf16 / fp16 mean in fp32 and
# rounds once), then widened to fp32; the search itself is fp32 except where it multiplies tensors.

FP32_TINY = F32(np.finfo(np.float32).tiny)
_TINY = {"f32": FP32_TINY, "f16": F32(np.finfo(np.float16).tiny), "bf16": F32(2.0 ** -126)}


def awq_weight_scale(w: np.ndarray, block: int, T="f32") -> np.ndarray:
    """get_weight_scale (:588-603): mean over rows of |W| / (block amax + tiny), everything in T."""
    w = np.asarray(w, dtype=F32)
    rows, cols = w.shape
    wp = pad_last(w, block)
    blocks = np.abs(wp).reshape(-1, block)
    amax = blocks.max(axis=1, keepdims=True)
    denom = round_to(amax + _TINY[T], T)
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = round_to(blocks / denom, T).reshape(rows, -1)[:, :cols]
    return round_to(scale.mean(axis=0, dtype=F32), T)


def awq_act_scale(x: np.ndarray, T="f32") -> np.ndarray:
    """get_act_scale (:605-606): per input channel, the mean of |x| over tokens, in T."""
    x = np.abs(np.asarray(x, dtype=F32)).reshape(-1, x.shape[-1])
    return round_to(x.mean(axis=0, dtype=F32), T)


def awq_get_scale(act_scale: np.ndarray, weight_scale: np.ndarray, alpha) -> np.ndarray:
    """get_scale (:608-621), fp32: a^alpha / (w^(1-alpha) + tiny), clamped to [1e-4, 1e4], divided by
    sqrt(max * min)."""
    a, w = np.asarray(act_scale, dtype=F32), np.asarray(weight_scale, dtype=F32)
    alpha = F32(alpha)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        s = (np.power(a, alpha) / (np.power(w, F32(1) - alpha) + FP32_TINY)).astype(F32)
        s = np.clip(s, F32(1e-4), F32(1e4)).astype(F32)
        return (s / np.sqrt((s.max() * s.min()).astype(F32))).astype(F32)


def awq_fake_weight(w: np.ndarray, s: np.ndarray, block: int, T="f32", num_bits=4) -> np.ndarray:
    """The weight the search evaluates: pre_quant_scale multiply in T, dynamic per-block amax in T,
    integer fake quant with narrow_range False (nn/modules/tensor_quantizer.py:882-883, 633-686)."""
    v = round_to(np.asarray(w, dtype=F32) * round_to(s, T)[None, :], T)
    rows, cols = v.shape
    vp = pad_last(v, block).reshape(-1, block)
    amax = np.abs(vp).max(axis=1, keepdims=True)
    return fake_int(vp, amax, num_bits, False, False, T).reshape(rows, -1)[:, :cols]


def awq_linear(x: np.ndarray, w: np.ndarray, T="f32") -> np.ndarray:
    """F.linear without bias: products summed in fp32, the result rounded to T."""
    return round_to(np.asarray(x, dtype=F32) @ np.asarray(w, dtype=F32).T, T)


def awq_lite_search(w: np.ndarray, batches: list, block: int, alphas, T="f32", num_bits=4):
    """One linear layer through the cache pass and the search pass: returns (weight_scale,
    act_scale, {alpha: loss}, best_alpha, best_scale).  ``alphas`` are the keys of the reference's loss
    dictionary: the elements of torch.arange(0, 1 + step, step) in fp32 as Python floats (:569-571).  loss = sum over batches of
    mean(float(T(out - out_actual))^2) (:623-627); the first minimum wins (:632-633)."""
    wsc = awq_weight_scale(w, block, T)
    asc = np.zeros(w.shape[1], dtype=F32)
    for x in batches:
        asc = (asc + awq_act_scale(x, T)).astype(F32)
    asc = (asc / F32(len(batches))).astype(F32)
    losses = {}
    for alpha in alphas:
        s = awq_get_scale(asc, wsc, alpha)
        wq = awq_fake_weight(w, s, block, T, num_bits)
        with np.errstate(divide="ignore"):
            xs = round_to((F32(1) / s).astype(F32), T)
        total = F32(0)
        for x in batches:
            x2 = np.asarray(x, dtype=F32).reshape(-1, x.shape[-1])
            out = awq_linear(round_to(x2 * xs[None, :], T), wq, T)
            ref = awq_linear(x2, w, T)
            d = round_to(out - ref, T)
            total = F32(total + F32(np.mean(d.astype(np.float64) ** 2)))
        losses[alpha] = float(total)
    best = min(losses, key=losses.get)
    return wsc, asc, losses, best, awq_get_scale(asc, wsc, best)
