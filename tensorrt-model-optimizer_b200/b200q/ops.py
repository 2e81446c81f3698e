"""Tensor-level wrappers over the C ABI.

Each function takes CUDA tensors, allocates the outputs with torch (plumbing only), and launches
the kernel on torch's current stream of the tensor's device.  CPU tensors are rejected: there is
no fallback implementation.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch

from . import _cabi
from ._cabi import call

_DT = {torch.float32: _cabi.F32, torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"b200q kernels take float32/float16/bfloat16 tensors, got {t.dtype}") from None


def _cuda(t: torch.Tensor, what="input") -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"b200q: {what} must be a CUDA tensor (no CPU path exists)")
    return t


def _prep(x: torch.Tensor, align: int = 16) -> torch.Tensor:
    """Contiguous, aligned view of x (copies only when it has to)."""
    _cuda(x)
    x = x.contiguous()
    if x.data_ptr() % align:
        x = x.clone(memory_format=torch.contiguous_format)
    return x


_SAME_DEVICE = contextlib.nullcontext()


def _on(device):
    """Context that makes ``device`` current for a launch; free when it already is (the usual case: the
    full device guard costs several microseconds per call, as much as a small kernel's launch)."""
    index = device.index
    if index is None or index == torch.cuda.current_device():
        return _SAME_DEVICE
    return torch.cuda.device(device)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _amax_f32(amax: torch.Tensor, device) -> torch.Tensor:
    return amax.detach().to(device=device, dtype=torch.float32).contiguous()


# --------------------------------------------------------------------------- amax --------------

def amax_tensor(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 0-dim abs-max of x; with ``out`` (fp32, 1 element) the running max is updated in place."""
    x = _prep(x)
    if out is None:
        out = torch.zeros((), dtype=torch.float32, device=x.device)
    with _on(x.device):
        call("b200q_amax_tensor", x.data_ptr(), x.numel(), dtype_code(x), out.data_ptr(), _stream(x))
    return out


def amax_axis3(x: torch.Tensor, outer: int, axis: int, inner: int,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [axis] abs-max of contiguous x viewed as [outer, axis, inner]."""
    x = _prep(x)
    assert x.numel() == outer * axis * inner
    if out is None:
        out = torch.zeros(axis, dtype=torch.float32, device=x.device)
    with _on(x.device):
        call("b200q_amax_axis", x.data_ptr(), outer, axis, inner, dtype_code(x), out.data_ptr(), _stream(x))
    return out


def amax_blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    """fp32 [numel/block] abs-max of each run of ``block`` contiguous elements."""
    x = _prep(x)
    n = x.numel()
    if n % block:
        raise ValueError(f"numel {n} is not divisible by block {block}")
    out = torch.empty(n // block, dtype=torch.float32, device=x.device)
    with _on(x.device):
        call("b200q_amax_blocks", x.data_ptr(), n // block, block, dtype_code(x), out.data_ptr(), _stream(x))
    return out


# --------------------------------------------------------------------------- fake quant --------

def _axis_view(x: torch.Tensor, amax: torch.Tensor):
    """(outer, axis, inner) of the single dimension along which ``amax`` varies."""
    n = amax.numel()
    shape = list(amax.shape)
    if len(shape) == x.dim() and n in shape:
        ax = shape.index(n)
    elif amax.dim() == 1 and n in x.shape:
        ax = list(x.shape).index(n)
    else:
        raise ValueError(f"amax of shape {tuple(amax.shape)} does not select one axis of {tuple(x.shape)}")
    if x.shape[ax] != n:
        raise ValueError(f"amax has {n} elements but input dim {ax} has {x.shape[ax]}")
    outer = 1
    for d in x.shape[:ax]:
        outer *= d
    inner = 1
    for d in x.shape[ax + 1:]:
        inner *= d
    return outer, n, inner


def _kept_dims_first(x: torch.Tensor, amax):
    """``amax`` that broadcasts over ``x`` with two or more kept dimensions (e.g. the [n0, 1, n2, 1] of blocks
    over several dimensions) -> the permutation of ``x`` that brings the kept dimensions to the front, where
    they flatten into the rows of a per-row problem; None for every other amax."""
    if not isinstance(amax, torch.Tensor) or amax.dim() != x.dim():
        return None
    kept = [d for d in range(x.dim()) if amax.shape[d] != 1]
    if len(kept) < 2 or any(amax.shape[d] != x.shape[d] for d in kept):
        return None
    return kept + [d for d in range(x.dim()) if d not in kept]


def _per_row_of_permuted(fn, x, amax, perm, *args):
    xp = x.permute(perm).contiguous()
    rows = amax.numel()
    yp = fn(xp.reshape(rows, -1), amax.permute(perm).reshape(rows, 1), *args)
    inverse = [perm.index(d) for d in range(len(perm))]
    return yp.reshape(xp.shape).permute(inverse).contiguous()


def fake_int(x: torch.Tensor, amax: torch.Tensor, num_bits: int = 8, unsigned: bool = False,
             narrow_range: bool = True) -> torch.Tensor:
    perm = _kept_dims_first(x, amax)
    if perm is not None:
        return _per_row_of_permuted(fake_int, x, amax, perm, num_bits, unsigned, narrow_range)
    x = _prep(x)
    y = torch.empty_like(x)
    if x.numel() == 0:
        return y
    am = _amax_f32(amax, x.device)
    with _on(x.device):
        if am.numel() == 1:
            call("b200q_fake_int_tensor", x.data_ptr(), y.data_ptr(), x.numel(), dtype_code(x),
                 am.data_ptr(), num_bits, int(unsigned), int(narrow_range), _stream(x))
        else:
            outer, axis, inner = _axis_view(x, amax)
            call("b200q_fake_int_axis", x.data_ptr(), y.data_ptr(), outer, axis, inner, dtype_code(x),
                 am.data_ptr(), num_bits, int(unsigned), int(narrow_range), _stream(x))
    return y


def fake_int_rows_dynamic(x: torch.Tensor, num_bits: int = 8, unsigned: bool = False,
                          narrow_range: bool = True, return_amax: bool = False):
    """Per-row dynamic fake quant of a 2-D tensor; the row amax is found in the same pass."""
    x = _prep(x)
    if x.dim() != 2:
        raise ValueError("expected a 2-D tensor [rows, cols]")
    rows, cols = x.shape
    y = torch.empty_like(x)
    am = torch.empty(rows, dtype=torch.float32, device=x.device) if return_amax else None
    with _on(x.device):
        call("b200q_fake_int_rows_dynamic", x.data_ptr(), y.data_ptr(), rows, cols, dtype_code(x),
             am.data_ptr() if am is not None else None, num_bits, int(unsigned), int(narrow_range),
             _stream(x))
    return (y, am) if return_amax else y


def fake_e4m3(x: torch.Tensor, amax: torch.Tensor | None) -> torch.Tensor:
    perm = _kept_dims_first(x, amax)
    if perm is not None:
        return _per_row_of_permuted(fake_e4m3, x, amax, perm)
    x = _prep(x)
    y = torch.empty_like(x)
    if x.numel() == 0:
        return y
    with _on(x.device):
        if amax is None:
            call("b200q_fake_e4m3_tensor", x.data_ptr(), y.data_ptr(), x.numel(), dtype_code(x), None, _stream(x))
            return y
        am = _amax_f32(amax, x.device)
        if am.numel() == 1:
            call("b200q_fake_e4m3_tensor", x.data_ptr(), y.data_ptr(), x.numel(), dtype_code(x),
                 am.data_ptr(), _stream(x))
        else:
            outer, axis, inner = _axis_view(x, amax)
            call("b200q_fake_e4m3_axis", x.data_ptr(), y.data_ptr(), outer, axis, inner, dtype_code(x),
                 am.data_ptr(), _stream(x))
    return y


# --------------------------------------------------------------------------- NVFP4 -------------

def nvfp4_quantize(x: torch.Tensor, amax: torch.Tensor | None = None, scale2: torch.Tensor | None = None,
                   scales_in: torch.Tensor | None = None, block: int = 16, saturate_scales: bool = False):
    """x [..., K] with K % block == 0 -> (packed uint8 [..., K/2], scales float8_e4m3fn [..., K/block],
    scale2 fp32 0-dim).  ``amax`` (any float dtype, 1 element) or ``scale2`` may be given; with
    neither the tensor's own abs-max is used.  block 16 (the format's own) runs the fast kernels.
    ``saturate_scales`` (block 16): a block whose scale exceeds the E4M3 range (data beyond a calibrated
    amax) gets 448, as in the fake-quant path, instead of the NaN code of the tensor cast."""
    x = _prep(x, 32 if block == 16 else 16)
    K = x.shape[-1]
    if K % block or block % 2:
        raise ValueError(f"last dimension must be a multiple of the (even) block size {block} (pad first)")
    nblocks = x.numel() // block
    dev = x.device
    packed = torch.empty((*x.shape[:-1], K // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((*x.shape[:-1], K // block), dtype=torch.uint8, device=dev)
    s2 = torch.empty((), dtype=torch.float32, device=dev)
    flags = 2 if saturate_scales else 0
    if saturate_scales and block != 16:
        raise ValueError("saturate_scales is built for block size 16")
    if scale2 is not None:
        glob = _amax_f32(scale2, dev).reshape(())
        flags |= 1
    elif amax is not None:
        glob = _amax_f32(amax, dev).reshape(())
    else:
        glob = amax_tensor(x)
    sin = None
    if scales_in is not None:
        sin = _cuda(scales_in, "scales_in").contiguous().view(torch.uint8)
        assert sin.numel() == nblocks
    with _on(dev):
        if block == 16:
            call("b200q_nvfp4_quantize", x.data_ptr(), nblocks, dtype_code(x), glob.data_ptr(),
                 sin.data_ptr() if sin is not None else None, packed.data_ptr(), scales.data_ptr(),
                 s2.data_ptr(), flags, _stream(x))
        else:
            call("b200q_nvfp4_quantize_blocks", x.data_ptr(), nblocks, block, dtype_code(x), glob.data_ptr(),
                 sin.data_ptr() if sin is not None else None, packed.data_ptr(), scales.data_ptr(),
                 s2.data_ptr(), flags, _stream(x))
    return packed, scales.view(torch.float8_e4m3fn), s2


def nvfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, scale2: torch.Tensor,
                     dtype: torch.dtype, block: int = 16) -> torch.Tensor:
    packed = _cuda(packed).contiguous()
    scales = _cuda(scales).contiguous().view(torch.uint8)
    s2 = _amax_f32(scale2, packed.device).reshape(())
    y = torch.empty((*packed.shape[:-1], packed.shape[-1] * 2), dtype=dtype, device=packed.device)
    nblocks = y.numel() // block
    assert scales.numel() == nblocks
    with _on(packed.device):
        if block == 16:
            call("b200q_nvfp4_dequantize", packed.data_ptr(), scales.data_ptr(), s2.data_ptr(), y.data_ptr(),
                 nblocks, _DT[dtype], _stream(packed))
        else:
            call("b200q_nvfp4_dequantize_blocks", packed.data_ptr(), scales.data_ptr(), s2.data_ptr(),
                 y.data_ptr(), nblocks, block, _DT[dtype], _stream(packed))
    return y


def nvfp4_fake(x: torch.Tensor, amax: torch.Tensor | None = None, block: int = 16) -> torch.Tensor:
    """NVFP4 fake quant along the last dimension (last dimension % block == 0)."""
    x = _prep(x, 32 if block == 16 else 16)
    if x.shape[-1] % block or block % 2:
        raise ValueError(f"last dimension must be a multiple of the (even) block size {block} (pad first)")
    y = torch.empty_like(x)
    am = amax_tensor(x) if amax is None else _amax_f32(amax, x.device)
    if am.numel() != 1:
        am = am.amax()
    with _on(x.device):
        if block == 16:
            call("b200q_nvfp4_fake", x.data_ptr(), y.data_ptr(), x.numel() // 16, dtype_code(x), am.data_ptr(),
                 _stream(x))
        else:
            call("b200q_nvfp4_fake_blocks", x.data_ptr(), y.data_ptr(), x.numel() // block, block, dtype_code(x),
                 am.data_ptr(), _stream(x))
    return y


class NvFp4Group:
    """A list of same-dtype weight tensors quantised by two grouped launches (amax, quantise).

    The descriptor table lives in device memory and is built once; ``run()`` only zeroes the
    amax slots and launches, so it can be repeated (and timed) without host work per tensor.
    """

    def __init__(self, tensors: list[torch.Tensor], separate_outputs: bool = False):
        """``separate_outputs``: every tensor's packed bytes and block scales get an allocation of their
        own (for results that outlive the group, e.g. module weights) instead of slices of two arenas."""
        if not tensors:
            raise ValueError("empty tensor list")
        self.tensors = [_prep(t, 32) for t in tensors]
        dev, dt = self.tensors[0].device, self.tensors[0].dtype
        tile = call("b200q_nvfp4_group_tile_elems")
        n = len(self.tensors)
        self.device, self.dtype, self.n = dev, dt, n
        total_packed = sum(t.numel() // 2 for t in self.tensors)
        total_scales = sum(t.numel() // 16 for t in self.tensors)
        # one allocation per output kind; 32-byte aligned slices
        if not separate_outputs:
            self._packed = torch.empty(total_packed + 32 * n, dtype=torch.uint8, device=dev)
            self._scales = torch.empty(total_scales + 32 * n, dtype=torch.uint8, device=dev)
        self.amax = torch.zeros(n, dtype=torch.float32, device=dev)
        self.scale2 = torch.empty(n, dtype=torch.float32, device=dev)
        descs = (_cabi.NvFp4Desc * n)()
        self.packed, self.scales = [], []
        po = so = 0
        tiles = 0
        for i, t in enumerate(self.tensors):
            if t.device != dev or t.dtype != dt:
                raise ValueError("all tensors of a group must share device and dtype")
            if t.shape[-1] % 16:
                raise ValueError("last dimension must be a multiple of 16")
            K = t.shape[-1]
            if separate_outputs:
                p = torch.empty((*t.shape[:-1], K // 2), dtype=torch.uint8, device=dev)
                s = torch.empty((*t.shape[:-1], K // 16), dtype=torch.uint8, device=dev)
            else:
                p = self._packed[po:po + t.numel() // 2].view(*t.shape[:-1], K // 2)
                s = self._scales[so:so + t.numel() // 16].view(*t.shape[:-1], K // 16)
            self.packed.append(p)
            self.scales.append(s.view(torch.float8_e4m3fn))
            d = descs[i]
            d.x, d.packed, d.scales = t.data_ptr(), p.data_ptr(), s.data_ptr()
            d.amax = self.amax.data_ptr() + 4 * i
            d.s2 = self.scale2.data_ptr() + 4 * i
            d.nblocks = t.numel() // 16
            d.tile_begin = tiles
            tiles += (t.numel() + tile - 1) // tile
            po += (t.numel() // 2 + 31) // 32 * 32
            so += (t.numel() // 16 + 31) // 32 * 32
        self.total_tiles = tiles
        raw = bytes(descs)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self._descs = host.to(dev)
        self.elements = sum(t.numel() for t in self.tensors)

    def run(self, amax_pass: bool = True, amax_values: dict | None = None):
        """``amax_values`` {index: tensor}: global abs-max to use for those tensors instead of their own (a
        calibrated or clipped weight amax)."""
        dc = _DT[self.dtype]
        with _on(self.device):
            st = torch.cuda.current_stream(self.device).cuda_stream
            if amax_pass:
                self.amax.zero_()
                call("b200q_nvfp4_group_amax", self._descs.data_ptr(), self.n, self.total_tiles, dc, st)
            if amax_values:
                idx = torch.tensor(sorted(amax_values), dtype=torch.int64, device=self.device)
                vals = torch.stack([amax_values[i].detach().to(device=self.device, dtype=torch.float32).reshape(())
                                    for i in sorted(amax_values)])
                self.amax.index_copy_(0, idx, vals)
            call("b200q_nvfp4_group_quantize", self._descs.data_ptr(), self.n, self.total_tiles, dc, st)
        return self.packed, self.scales, self.scale2


# --------------------------------------------------------------------------- INT4 --------------

def int4_quantize(x: torch.Tensor, block: int, scales_in: torch.Tensor | None = None):
    """Flat contiguous x (numel % block == 0) -> (packed uint8 [numel/2], scales T [numel/block, 1])."""
    x = _prep(x)
    n = x.numel()
    if n % block or block % 2:
        raise ValueError("numel must be a multiple of an even block size (pad first)")
    nb = n // block
    packed = torch.empty(n // 2, dtype=torch.uint8, device=x.device)
    if scales_in is not None:
        scales = _cuda(scales_in, "scales").to(x.dtype).contiguous().view(nb, 1)
        sin, sout = scales.data_ptr(), None
    else:
        scales = torch.empty((nb, 1), dtype=x.dtype, device=x.device)
        sin, sout = None, scales.data_ptr()
    with _on(x.device):
        call("b200q_int4_quantize", x.data_ptr(), nb, block, dtype_code(x), sin, sout, packed.data_ptr(),
             _stream(x))
    return packed, scales


def int4_dequantize(packed: torch.Tensor, scales: torch.Tensor, block: int) -> torch.Tensor:
    packed = _cuda(packed).contiguous().view(-1)
    scales = _cuda(scales, "scales").contiguous()
    n = packed.numel() * 2
    y = torch.empty(n, dtype=scales.dtype, device=packed.device)
    with _on(packed.device):
        call("b200q_int4_dequantize", packed.data_ptr(), scales.data_ptr(), y.data_ptr(), n // block, block,
             dtype_code(scales), _stream(packed))
    return y


# --------------------------------------------------------------------------- FP8 / INT8 --------

def _q8(name: str, x: torch.Tensor, scales: torch.Tensor, outer: int, axis: int, inner: int, out_dtype):
    x = _prep(x)
    s = _cuda(scales, "scales").to(x.dtype).contiguous()
    assert s.numel() == axis and x.numel() == outer * axis * inner
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    with _on(x.device):
        call(name, x.data_ptr(), s.data_ptr(), q.data_ptr(), outer, axis, inner, dtype_code(x), _stream(x))
    return q.view(out_dtype)


def fp8_quantize(x, scales, outer, axis, inner):
    return _q8("b200q_fp8_quantize", x, scales, outer, axis, inner, torch.float8_e4m3fn)


def int8_quantize(x, scales, outer, axis, inner):
    return _q8("b200q_int8_quantize", x, scales, outer, axis, inner, torch.int8)


# --------------------------------------------------------------------------- histogram ---------

def hist_collect(x: torch.Tensor, counts: torch.Tensor, nbins: int, range_max: float):
    """counts (int64 [>= nbins], CUDA) += histogram of |x| over [0, range_max] with nbins bins."""
    x = _prep(x)
    assert counts.dtype == torch.int64 and counts.is_cuda and counts.numel() >= nbins
    with _on(x.device):
        call("b200q_hist_collect", x.data_ptr(), x.numel(), dtype_code(x), nbins,
             ctypes.c_float(range_max), counts.data_ptr(), _stream(x))
    return counts


def hist_collect_open(x: torch.Tensor, counts: torch.Tensor, nbins: int, range_max: float,
                      overflow: torch.Tensor):
    """counts (int64 [capacity]) += histogram of |x| with bin width range_max / nbins, open-ended: bins
    run on past nbins - 1 up to counts.numel(); samples beyond that (and NaN / inf) add to overflow."""
    x = _prep(x)
    assert counts.dtype == torch.int64 and counts.is_cuda and counts.numel() >= nbins
    assert overflow.dtype == torch.int64 and overflow.is_cuda and overflow.numel() >= 1
    with _on(x.device):
        call("b200q_hist_collect_open", x.data_ptr(), x.numel(), dtype_code(x), nbins, ctypes.c_float(range_max),
             counts.numel(), counts.data_ptr(), overflow.data_ptr(), _stream(x))
    return counts


def hist_collect_shared(x: torch.Tensor, counts: list, overflow: list, nbins: int, range_dev: torch.Tensor):
    """Bin |x| once and add the counts to every histogram of ``counts`` (1..4 int64 CUDA tensors of one
    capacity, open-ended as in ``hist_collect_open``), the range being the fp32 device scalar ``range_dev``."""
    x = _prep(x)
    n = len(counts)
    assert 1 <= n <= 4 and len(overflow) == n
    cap = counts[0].numel()
    for c, o in zip(counts, overflow):
        assert c.dtype == torch.int64 and c.is_cuda and c.is_contiguous() and c.numel() == cap
        assert o.dtype == torch.int64 and o.is_cuda and o.numel() >= 1
    assert range_dev.dtype == torch.float32 and range_dev.is_cuda and range_dev.numel() >= 1
    cp = (ctypes.c_void_p * n)(*[c.data_ptr() for c in counts])
    op = (ctypes.c_void_p * n)(*[o.data_ptr() for o in overflow])
    with _on(x.device):
        call("b200q_hist_collect_shared", x.data_ptr(), x.numel(), dtype_code(x), nbins, range_dev.data_ptr(), cap,
             ctypes.cast(cp, ctypes.c_void_p), ctypes.cast(op, ctypes.c_void_p), n, _stream(x))


def hist_entropy(counts: torch.Tensor, nbins: int, edges: torch.Tensor, num_levels: int, start_bin: int = 128,
                 stride: int = 1):
    """Entropy-calibrated amax (0-dim fp32 tensor) and the per-candidate divergences (fp64)."""
    ncand = (nbins - start_bin) // stride + 1
    divs = torch.empty(ncand, dtype=torch.float64, device=counts.device)
    out = torch.empty((), dtype=torch.float32, device=counts.device)
    e = edges.to(device=counts.device, dtype=torch.float32).contiguous()
    assert e.numel() >= nbins + 1 and counts.dtype == torch.int64
    with _on(counts.device):
        call("b200q_hist_entropy", counts.data_ptr(), nbins, num_levels, start_bin, stride, e.data_ptr(),
             ctypes.c_float(0.0), divs.data_ptr(), out.data_ptr(), _stream(counts))
    return out, divs


def hist_mse(counts: torch.Tensor, nbins: int, edges: torch.Tensor, bound: float, start_bin: int = 128,
             stride: int = 1):
    """MSE-calibrated amax (0-dim fp32 tensor) and the per-candidate errors (fp64)."""
    ncand = (nbins - 1 - start_bin) // stride + 1
    errs = torch.empty(ncand, dtype=torch.float64, device=counts.device)
    out = torch.empty((), dtype=torch.float32, device=counts.device)
    e = edges.to(device=counts.device, dtype=torch.float32).contiguous()
    assert e.numel() >= nbins + 1 and counts.dtype == torch.int64
    with _on(counts.device):
        call("b200q_hist_mse", counts.data_ptr(), nbins, e.data_ptr(), ctypes.c_double(bound), start_bin, stride,
             errs.data_ptr(), out.data_ptr(), _stream(counts))
    return out, errs


def hist_percentile(counts: torch.Tensor, nbins: int, edges: torch.Tensor | None, width: float,
                    percentile: float) -> torch.Tensor:
    out = torch.empty((), dtype=torch.float32, device=counts.device)
    e = None
    if edges is not None:
        e = edges.to(device=counts.device, dtype=torch.float32).contiguous()
        assert e.numel() >= nbins + 1
    with _on(counts.device):
        call("b200q_hist_percentile", counts.data_ptr(), nbins, e.data_ptr() if e is not None else None,
             ctypes.c_float(width), ctypes.c_double(percentile), out.data_ptr(), _stream(counts))
    return out


def hist_percentile_batch(items, percentile: float) -> torch.Tensor:
    """Percentile read-out of many histograms in one launch.  ``items``: (counts int64 device tensor, nbins,
    edges fp32 device tensor [>= nbins + 1]) per histogram, all on one device.  Returns fp32 [len(items)]."""
    n = len(items)
    dev = items[0][0].device
    descs = (_cabi.HistDesc * n)()
    keep = []
    for d, (counts, nbins, edges) in zip(descs, items):
        e = edges.to(device=dev, dtype=torch.float32).contiguous()
        assert counts.dtype == torch.int64 and counts.is_contiguous() and counts.numel() >= nbins
        assert e.numel() >= nbins + 1
        keep.append(e)
        d.counts, d.edges, d.bin_width, d.nbins = counts.data_ptr(), e.data_ptr(), 0.0, int(nbins)
    table = torch.frombuffer(bytearray(bytes(descs)), dtype=torch.uint8).to(dev)
    out = torch.empty(n, dtype=torch.float32, device=dev)
    with _on(dev):
        call("b200q_hist_percentile_batch", table.data_ptr(), n, ctypes.c_double(percentile), out.data_ptr(),
             torch.cuda.current_stream(dev).cuda_stream)
    return out


# --------------------------------------------------------------------------- MSE search --------

def mse_candidates_supported(x: torch.Tensor, axis) -> bool:
    """Layouts the one-pass candidate kernel covers: per tensor, or one channel axis with at least 32
    sixteen-byte packs of contiguous elements behind it."""
    if not x.is_cuda or x.dtype not in _DT:
        return False
    if axis is None:
        return True
    if not isinstance(axis, int):
        return False
    inner = 1
    for d in x.shape[axis % x.dim() + 1:]:
        inner *= d
    per_pack = 16 // x.element_size()
    return inner % per_pack == 0 and inner >= 32 * per_pack


def mse_candidates(x: torch.Tensor, cand: torch.Tensor, loss: torch.Tensor, axis=None, num_bits=8,
                   unsigned: bool = False, narrow_range: bool = True) -> torch.Tensor:
    """loss[s, c] (float64) += squared fake-quantisation error of x (taken as fp32) under candidate amax
    cand[s, c] (fp32), every candidate in one pass over x.  ``num_bits`` an int, or (4, 3) for FP8 E4M3."""
    x = _prep(x)
    if axis is None:
        outer, channels, inner = 1, 1, x.numel()
    else:
        ax = axis % x.dim()
        outer = inner = 1
        for d in x.shape[:ax]:
            outer *= d
        for d in x.shape[ax + 1:]:
            inner *= d
        channels = x.shape[ax]
    cand = cand.detach().to(device=x.device, dtype=torch.float32).contiguous()
    s = cand.numel() // channels
    assert cand.numel() == s * channels and loss.dtype == torch.float64 and loss.numel() == s * channels
    assert loss.is_cuda and loss.is_contiguous()
    fp8 = not isinstance(num_bits, int)
    if fp8 and tuple(num_bits) != (4, 3):
        raise ValueError("mse_candidates covers integer formats and E4M3")
    with _on(x.device):
        call("b200q_mse_candidates", x.data_ptr(), outer, channels, inner, dtype_code(x), cand.data_ptr(), s,
             1 if fp8 else 0, 8 if fp8 else num_bits, int(unsigned), int(narrow_range), loss.data_ptr(), _stream(x))
    return loss


# --------------------------------------------------------------------------- awq_lite ----------

def awq_scale_fake_int(w: torch.Tensor, s: torch.Tensor, block: int, num_bits: int = 4,
                       unsigned: bool = False, narrow_range: bool = False,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """fake_int over blocks of ``block`` along the last dim of T(w * s), s broadcast over rows."""
    w = _prep(w)
    s = _prep(s.to(w.dtype))
    assert w.dim() == 2 and s.numel() == w.shape[1]
    if out is None:
        y = torch.empty_like(w)
    else:
        assert out.shape == w.shape and out.dtype == w.dtype and out.is_contiguous() and out.device == w.device
        y = out
    with _on(w.device):
        call("b200q_awq_scale_fake_int", w.data_ptr(), s.data_ptr(), y.data_ptr(), w.shape[0], w.shape[1],
             block, dtype_code(w), num_bits, int(unsigned), int(narrow_range), _stream(w))
    return y


def mse_loss(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """mean(float(a - b)^2) with the difference rounded to the tensors' dtype first; fp32 0-dim."""
    a, b = _prep(a), _prep(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    acc = torch.zeros((), dtype=torch.float64, device=a.device)
    with _on(a.device):
        call("b200q_sq_diff_sum", a.data_ptr(), b.data_ptr(), a.numel(), dtype_code(a), acc.data_ptr(), _stream(a))
    return (acc / a.numel()).to(torch.float32)


def awq_gemm_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Shapes / dtype the tensor-core evaluation kernel covers."""
    return (a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
            and a.shape[0] % 128 == 0 and b.shape[0] % 128 == 0 and a.shape[1] % 64 == 0
            and a.shape[1] == b.shape[1])


_SPLITK_SCRATCH: dict = {}


def awq_gemm_splits(m: int, n: int, k: int, device) -> int:
    """How many CTAs share the K extent of one output tile: 1 unless the 128 x 128 tiles leave half of
    the SMs' two CTA slots empty and K is long enough to give every split 16 K blocks or more."""
    tiles = (m // 128) * (n // 128)
    slots = 2 * torch.cuda.get_device_properties(device).multi_processor_count
    return max(1, min(slots // max(tiles, 1), k // 64 // 16, 4))


def awq_gemm_sqerr(a: torch.Tensor, b: torch.Tensor, ref: torch.Tensor, acc: torch.Tensor,
                   status: torch.Tensor, c_out: torch.Tensor | None = None, splits: int | None = None):
    """acc (float64, 1 element) += sum of squared bf16 differences between bf16(a @ b.T) and ref.
    ``status`` is an int32 device word that collects error bits of the kernel's bounded waits.
    ``splits`` (default: ``awq_gemm_splits``) CTAs share the K extent of a tile; their scratch
    (fp32 partial tiles, tile counters) is kept per device, stream and shape and reused in stream
    order."""
    a, b, ref = _prep(a), _prep(b), _prep(ref)
    m, k = a.shape
    n = b.shape[0]
    assert ref.shape == (m, n) and ref.dtype == torch.bfloat16 and acc.dtype == torch.float64
    if splits is None:
        splits = awq_gemm_splits(m, n, k, a.device)
    with _on(a.device):
        if splits <= 1:
            call("b200q_awq_gemm_sqerr", a.data_ptr(), b.data_ptr(), ref.data_ptr(), m, n, k, acc.data_ptr(),
                 c_out.data_ptr() if c_out is not None else None, status.data_ptr(), _stream(a))
        else:
            key = (a.device, _stream(a), splits, m, n)
            scratch = _SPLITK_SCRATCH.get(key)
            if scratch is None:
                scratch = _SPLITK_SCRATCH[key] = (torch.empty(splits * m * n, dtype=torch.float32, device=a.device),
                                                  torch.zeros((m // 128) * (n // 128), dtype=torch.int32, device=a.device))
            call("b200q_awq_gemm_sqerr_splitk", a.data_ptr(), b.data_ptr(), ref.data_ptr(), m, n, k, splits,
                 scratch[0].data_ptr(), scratch[1].data_ptr(), acc.data_ptr(),
                 c_out.data_ptr() if c_out is not None else None, status.data_ptr(), _stream(a))
    return acc


def awq_scale_acts(x2: torch.Tensor, s_all: torch.Tensor) -> torch.Tensor:
    """[n_alpha, rows, cols] = x2[None] * s_all[:, None] in x2's dtype, one pass (``b200q_awq_scale_acts``)."""
    x2, s_all = _prep(x2), _prep(s_all.to(x2.dtype))
    rows, cols = x2.shape
    n_alpha = s_all.shape[0]
    assert s_all.shape == (n_alpha, cols)
    out = torch.empty((n_alpha, rows, cols), dtype=x2.dtype, device=x2.device)
    with _on(x2.device):
        call("b200q_awq_scale_acts", x2.data_ptr(), s_all.data_ptr(), out.data_ptr(), rows, cols, n_alpha,
             dtype_code(x2), _stream(x2))
    return out


def awq_search_fused_supported(x2: torch.Tensor, w: torch.Tensor, block) -> bool:
    """Shapes / dtype the fused all-candidates search kernel covers."""
    return (x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x2.is_cuda and w.is_cuda and x2.dim() == 2
            and w.dim() == 2 and block == 128 and w.shape[1] % 128 == 0 and w.shape[0] % 32 == 0
            and x2.shape[1] == w.shape[1] and x2.shape[0] > 0)


def awq_search_fused(a_all: torch.Tensor, w: torch.Tensor, s_all: torch.Tensor, ref: torch.Tensor,
                     loss: torch.Tensor, status: torch.Tensor, block: int = 128, num_bits: int = 4,
                     unsigned: bool = False, narrow_range: bool = False, c_out: torch.Tensor | None = None):
    """loss[a] (float64) += squared bf16 error of ``a_all[a] @ fq(w * s_all[a]).T`` against ``ref`` for every
    candidate a, in one launch (``b200q_awq_search_fused``).  a_all [n_alpha, m, k], w [n, k], s_all [n_alpha, k],
    ref [m, n], all bf16; ``status`` an int32 device word for the kernel's bounded waits."""
    a_all, w, s_all, ref = _prep(a_all), _prep(w, 32), _prep(s_all), _prep(ref)
    n_alpha, m, k = a_all.shape
    n = w.shape[0]
    assert w.shape == (n, k) and s_all.shape == (n_alpha, k) and ref.shape == (m, n)
    assert a_all.dtype == w.dtype == s_all.dtype == ref.dtype == torch.bfloat16
    assert loss.dtype == torch.float64 and loss.numel() == n_alpha and loss.is_contiguous()
    if c_out is not None:
        assert c_out.dtype == torch.float32 and c_out.shape == (n_alpha, m, n) and c_out.is_contiguous()
    with _on(w.device):
        call("b200q_awq_search_fused", a_all.data_ptr(), w.data_ptr(), s_all.data_ptr(), ref.data_ptr(), n_alpha,
             m, n, k, block, num_bits, int(unsigned), int(narrow_range), loss.data_ptr(),
             c_out.data_ptr() if c_out is not None else None, status.data_ptr(), _stream(w))
    return loss


def awq_search_prequant_supported(x2: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes / dtype the CTA-pair kernel covers when it is handed finished (fake-quantised) weights."""
    return (x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x2.is_cuda and w.is_cuda and x2.dim() == 2
            and w.dim() == 2 and w.shape[1] % 128 == 0 and w.shape[0] % 32 == 0 and x2.shape[1] == w.shape[1]
            and x2.shape[0] > 0)


def awq_search_prequant(a_all: torch.Tensor, wq_all: torch.Tensor, ref: torch.Tensor, loss: torch.Tensor,
                        status: torch.Tensor, c_out: torch.Tensor | None = None):
    """loss[a] (float64) += squared bf16 error of ``a_all[a] @ wq_all[a].T`` against ``ref`` for every candidate
    a, in one launch of the persistent CTA-pair kernel (``b200q_awq_search_prequant``).  a_all [n_alpha, m, k],
    wq_all [n_alpha, n, k] (already scaled and fake-quantised), ref [m, n], all bf16."""
    a_all, wq_all, ref = _prep(a_all), _prep(wq_all, 32), _prep(ref)
    n_alpha, m, k = a_all.shape
    n = wq_all.shape[1]
    assert wq_all.shape == (n_alpha, n, k) and ref.shape == (m, n)
    assert a_all.dtype == wq_all.dtype == ref.dtype == torch.bfloat16
    assert loss.dtype == torch.float64 and loss.numel() == n_alpha and loss.is_contiguous()
    if c_out is not None:
        assert c_out.dtype == torch.float32 and c_out.shape == (n_alpha, m, n) and c_out.is_contiguous()
    with _on(wq_all.device):
        call("b200q_awq_search_prequant", a_all.data_ptr(), wq_all.data_ptr(), ref.data_ptr(), n_alpha, m, n, k,
             loss.data_ptr(), c_out.data_ptr() if c_out is not None else None, status.data_ptr(), _stream(wq_all))
    return loss


def int4_export_pack(w: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """w [rows, cols], scales [rows, cols/block] (fp32 or w.dtype) -> uint8 [rows/2, cols]."""
    w = _prep(w)
    assert w.dim() == 2 and scales.dim() == 2 and scales.shape[0] == w.shape[0]
    rows, cols = w.shape
    block = cols // scales.shape[1]
    sc = _cuda(scales, "scales").contiguous()
    if sc.dtype not in (torch.float32, w.dtype):
        sc = sc.float()
    out = torch.empty((rows // 2, cols), dtype=torch.uint8, device=w.device)
    with _on(w.device):
        call("b200q_int4_export_pack", w.data_ptr(), sc.data_ptr(), int(sc.dtype == torch.float32),
             out.data_ptr(), rows, cols, block, dtype_code(w), _stream(w))
    return out


# --------------------------------------------------------------------------- MX formats --------

MX_FORMATS = {(4, 3): 0, (5, 2): 1, 8: 2, (2, 1): 6, (3, 2): 7, (2, 3): 8}


def mx_fake(x: torch.Tensor, block: int, num_bits) -> torch.Tensor:
    """MX fake quant along the last dim (blocks of ``block``, E8M0 scale); pads like the reference."""
    fmt = MX_FORMATS[tuple(num_bits) if isinstance(num_bits, (tuple, list)) else num_bits]
    shape = x.shape
    pad = (-shape[-1]) % block
    xx = torch.nn.functional.pad(x, (0, pad)) if pad else x
    xx = _prep(xx)
    y = torch.empty_like(xx)
    with _on(xx.device):
        call("b200q_mx_fake", xx.data_ptr(), y.data_ptr(), xx.numel() // block, block, dtype_code(xx), fmt,
             _stream(xx))
    return y[..., : shape[-1]].contiguous() if pad else y


def mxfp4_quantize(x: torch.Tensor, block: int = 32):
    """-> (packed uint8 [..., K/2], e8m0 scale bytes uint8 [numel/block, 1])."""
    x = _prep(x)
    n = x.numel()
    assert n % block == 0
    packed = torch.empty((*x.shape[:-1], x.shape[-1] // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((n // block, 1), dtype=torch.uint8, device=x.device)
    with _on(x.device):
        call("b200q_mxfp4_quantize", x.data_ptr(), n // block, block, dtype_code(x), packed.data_ptr(),
             scales.data_ptr(), _stream(x))
    return packed, scales


# --------------------------------------------------------------------------- awq_clip ----------

def awq_clip_loss(w: torch.Tensor, x: torch.Tensor, w_amax: torch.Tensor, ratios: torch.Tensor,
                  loss: torch.Tensor, block: int, num_bits: int = 4, unsigned: bool = False,
                  narrow_range: bool = False) -> torch.Tensor:
    """loss[r, row, blk] (fp32, CUDA) += block-wise output error of clipping the block amax to
    ``w_amax * ratios[r]`` (see ``b200q_awq_clip_loss``).  w [rows, cols], x [tokens, cols], w_amax
    [rows * cols / block] share one dtype; ratios is an fp32 CUDA tensor."""
    w, x = _prep(w), _prep(x)
    w_amax = _prep(w_amax.to(w.dtype))
    rows, cols = w.shape
    assert x.dim() == 2 and x.shape[1] == cols and x.dtype == w.dtype
    assert w_amax.numel() == rows * (cols // block)
    assert ratios.dtype == torch.float32 and ratios.is_cuda and ratios.is_contiguous()
    assert loss.dtype == torch.float32 and loss.is_cuda and loss.is_contiguous()
    assert loss.numel() == ratios.numel() * rows * (cols // block)
    with _on(w.device):
        call("b200q_awq_clip_loss", w.data_ptr(), x.data_ptr(), w_amax.data_ptr(), ratios.data_ptr(),
             ratios.numel(), loss.data_ptr(), rows, cols, block, x.shape[0], dtype_code(w), num_bits,
             int(unsigned), int(narrow_range), _stream(w))
    return loss


# --------------------------------------------------------------------------- rotation ----------

def hadamard(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Walsh-Hadamard transform along the last dimension (a power of two), times ``scale``."""
    x = _prep(x, 2)
    n = x.shape[-1]
    y = torch.empty_like(x)
    with _on(x.device):
        call("b200q_hadamard", x.data_ptr(), y.data_ptr(), x.numel() // n, n, dtype_code(x), ctypes.c_float(scale),
             _stream(x))
    return y


# --------------------------------------------------------------------------- real-quant GEMMs --

_QGEMM_STATUS: dict = {}


def qgemm_status(device) -> torch.Tensor:
    """The int32 device word that collects error bits of the GEMM kernels' bounded waits on
    ``device`` (0 = every wait completed).  Reading it synchronises; the layers never do."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = _QGEMM_STATUS.get(device)
    if st is None:
        st = _QGEMM_STATUS[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st


def check_qgemm_status(device):
    code = int(qgemm_status(device).item())
    if code:
        qgemm_status(device).zero_()
        raise RuntimeError(f"a bounded wait inside a tensor-core GEMM kernel ran out (status bits {code:#x})")


def _gemm_out(a, n, bias, out_dtype):
    if out_dtype not in _DT:
        raise TypeError(f"unsupported output dtype {out_dtype}")
    if bias is not None:
        bias = _cuda(bias, "bias").to(out_dtype).contiguous()
        assert bias.numel() == n
    return torch.empty((a.shape[0], n), dtype=out_dtype, device=a.device), bias


def fp8_gemm(a8: torch.Tensor, b8: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor | None = None,
             bias: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """a8 [m, k], b8 [n, k] float8_e4m3fn (or their bytes), fp32 device scalars scale_a / scale_b ->
    out_dtype [m, n] = a8 @ b8.T * scale_a * scale_b + bias, on the tensor cores."""
    a8 = _cuda(a8, "a").contiguous().view(torch.uint8)
    b8 = _cuda(b8, "b").contiguous().view(torch.uint8)
    assert a8.dim() == 2 and b8.dim() == 2 and a8.shape[1] == b8.shape[1]
    (m, k), n = a8.shape, b8.shape[0]
    sa = _amax_f32(scale_a, a8.device).reshape(())
    sb = _amax_f32(scale_b, a8.device).reshape(()) if scale_b is not None else None
    out, bias = _gemm_out(a8, n, bias, out_dtype)
    with _on(a8.device):
        call("b200q_fp8_gemm", a8.data_ptr(), b8.data_ptr(), sa.data_ptr(), sb.data_ptr() if sb is not None else None,
             bias.data_ptr() if bias is not None else None, out.data_ptr(), m, n, k, _DT[out_dtype],
             qgemm_status(a8.device).data_ptr(), _stream(a8))
    return out


def fp8_gemm_operand(x: torch.Tensor, scale: torch.Tensor, fused: bool = False) -> torch.Tensor:
    """e4m3(clamp(x / scale, -448, 448)), ``scale`` one fp32 element.  The quotient is rounded to x's
    dtype before the clamp (the eager arithmetic of the expression) unless ``fused`` (the quotient
    stays in fp32, as in a compiled graph)."""
    x = _prep(x)
    s = _amax_f32(scale, x.device).reshape(1)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    with _on(x.device):
        call("b200q_fp8_gemm_operand", x.data_ptr(), s.data_ptr(), q.data_ptr(), x.numel(), dtype_code(x),
             0 if fused else 1, _stream(x))
    return q.view(torch.float8_e4m3fn)


def nvfp4_swizzled_scale_bytes(rows: int, cols: int) -> int:
    return -(-rows // 128) * (-(-cols // 16) * 4) * 512


def nvfp4_swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """Block scales [rows, K/16] (float8_e4m3fn or bytes, row-major) -> flat uint8 in the 128 x 4 tile
    order the block-scaled GEMM reads (rows padded to 128, K to 256, with zeros)."""
    s = _cuda(scales, "scales").contiguous().view(torch.uint8)
    s = s.reshape(-1, s.shape[-1])
    rows, cols = s.shape
    out = torch.empty(nvfp4_swizzled_scale_bytes(rows, cols), dtype=torch.uint8, device=s.device)
    with _on(s.device):
        call("b200q_nvfp4_swizzle_scales", s.data_ptr(), out.data_ptr(), rows, cols, _stream(s))
    return out


def nvfp4_gemm(a4: torch.Tensor, sfa: torch.Tensor, b4: torch.Tensor, sfb: torch.Tensor, alpha: torch.Tensor,
               bias: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """a4 [m, k/2], b4 [n, k/2] packed E2M1; sfa, sfb the block scales as ``nvfp4_swizzle_scales``
    returns them; alpha fp32 device scalar -> out_dtype [m, n], on the tensor cores."""
    a4 = _cuda(a4, "a").contiguous().view(torch.uint8)
    b4 = _cuda(b4, "b").contiguous().view(torch.uint8)
    assert a4.dim() == 2 and b4.dim() == 2 and a4.shape[1] == b4.shape[1]
    m, n, k = a4.shape[0], b4.shape[0], a4.shape[1] * 2
    sfa, sfb = _cuda(sfa, "sfa").view(torch.uint8), _cuda(sfb, "sfb").view(torch.uint8)
    assert sfa.numel() == nvfp4_swizzled_scale_bytes(m, k // 16), "sfa is not in the tiled order for this shape"
    assert sfb.numel() == nvfp4_swizzled_scale_bytes(n, k // 16), "sfb is not in the tiled order for this shape"
    al = _amax_f32(alpha, a4.device).reshape(())
    out, bias = _gemm_out(a4, n, bias, out_dtype)
    with _on(a4.device):
        call("b200q_nvfp4_gemm", a4.data_ptr(), b4.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), al.data_ptr(),
             bias.data_ptr() if bias is not None else None, out.data_ptr(), m, n, k, _DT[out_dtype],
             qgemm_status(a4.device).data_ptr(), _stream(a4))
    return out
