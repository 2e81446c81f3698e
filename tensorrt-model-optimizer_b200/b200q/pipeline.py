"""Host-to-host NVFP4 packing of a list of weight tensors that live in (pinned) host memory.

This is the call a user makes when the checkpoint is on the host: weights are streamed to the
GPU group by group, quantised there by the grouped kernels, and the packed bytes, block scales and
per-tensor scales are streamed back, with the three phases of consecutive groups overlapping on
separate CUDA streams (copy-in, compute, copy-out) over double-buffered device staging.
Stands in for the per-weight loop of ``pack_real_quantize_weight``
(modelopt/torch/quantization/qtensor/base_qtensor.py:196-229) run on a model that sits on the CPU.
"""
from __future__ import annotations

import torch

from .ops import NvFp4Group


class HostNvFp4Packer:
    """Pack groups of host tensors to NVFP4.

    Args:
        group_shapes: shapes of the tensors of one group (e.g. the seven linears of a layer);
            every group passed to :meth:`pack` must have exactly these shapes.
        dtype: element type of the weights.
        device: CUDA device that does the work.
    """

    def __init__(self, group_shapes, dtype=torch.bfloat16, device="cuda", depth: int = 2):
        self.device = torch.device(device)
        self.dtype = dtype
        self.shapes = [tuple(s) for s in group_shapes]
        self.depth = depth
        with torch.cuda.device(self.device):
            self.s_in = torch.cuda.Stream()
            self.s_run = torch.cuda.Stream()
            self.s_out = torch.cuda.Stream()
        self.slots = []
        for _ in range(depth):
            staging = [torch.empty(s, dtype=dtype, device=self.device) for s in self.shapes]
            grp = NvFp4Group(staging)
            self.slots.append({
                "staging": staging, "group": grp,
                "loaded": torch.cuda.Event(), "done": torch.cuda.Event(), "drained": torch.cuda.Event(),
            })
        g0 = self.slots[0]["group"]
        self.packed_bytes = sum(p.numel() for p in g0.packed)
        self.scale_bytes = sum(s.numel() for s in g0.scales)
        self.in_bytes = sum(t.numel() * t.element_size() for t in g0.tensors)

    def alloc_host_outputs(self, ngroups: int):
        """Pinned host buffers for the results of ``ngroups`` groups."""
        out = []
        for _ in range(ngroups):
            out.append({
                "packed": [torch.empty((*s[:-1], s[-1] // 2), dtype=torch.uint8, pin_memory=True) for s in self.shapes],
                "scales": [torch.empty((*s[:-1], s[-1] // 16), dtype=torch.uint8, pin_memory=True) for s in self.shapes],
                "scale2": torch.empty(len(self.shapes), dtype=torch.float32, pin_memory=True),
            })
        return out

    def pack(self, host_groups, host_out, amax_values=None):
        """Quantise every group of ``host_groups`` (lists of pinned host tensors) into
        ``host_out`` (from :meth:`alloc_host_outputs`).  ``amax_values[i]`` ({index in group: tensor}) gives
        calibrated global abs-max values for group i.  Returns after everything has landed."""
        with torch.cuda.device(self.device):
            for i, tensors in enumerate(host_groups):
                slot = self.slots[i % self.depth]
                grp = slot["group"]
                # staging of this slot is free once the previous user's compute has finished
                if i >= self.depth:
                    self.s_in.wait_event(slot["done"])
                with torch.cuda.stream(self.s_in):
                    for dst, src in zip(slot["staging"], tensors):
                        dst.copy_(src, non_blocking=True)
                    slot["loaded"].record(self.s_in)
                self.s_run.wait_event(slot["loaded"])
                if i >= self.depth:
                    self.s_run.wait_event(slot["drained"])  # outputs of the previous user were read out
                with torch.cuda.stream(self.s_run):
                    grp.run(amax_values=amax_values[i] if amax_values else None)
                    slot["done"].record(self.s_run)
                self.s_out.wait_event(slot["done"])
                with torch.cuda.stream(self.s_out):
                    ho = host_out[i]
                    for k in range(len(self.shapes)):
                        ho["packed"][k].copy_(grp.packed[k], non_blocking=True)
                        ho["scales"][k].copy_(grp.scales[k].view(torch.uint8), non_blocking=True)
                    ho["scale2"].copy_(grp.scale2, non_blocking=True)
                    slot["drained"].record(self.s_out)
            self.s_out.synchronize()
        return host_out


def _repeating_unit(keys):
    """Smallest p such that ``keys`` is a whole number (>= 2) of repetitions of its first p entries (the
    linears of one transformer layer, in model order), or None."""
    n = len(keys)
    for p in range(1, n // 2 + 1):
        if n % p == 0 and all(keys[i] == keys[i - p] for i in range(p, n)):
            return p
    return None


def _plan_groups(keys, sizes, group_bytes):
    """Split tensor indices into groups for the packer; groups with the same signature (shapes and dtype
    in order) are streamed through one packer without draining its pipeline.  A model made of repeated
    layers becomes groups of whole layers (several small layers per group, or a large layer cut at the
    same places every time); anything else is bucketed by shape."""
    n = len(keys)
    p = _repeating_unit(keys)
    groups = []
    if p is not None:
        unit_bytes = sum(sizes[:p])
        if unit_bytes <= group_bytes:
            per = max(1, group_bytes // max(unit_bytes, 1)) * p
            groups = [list(range(i, min(i + per, n))) for i in range(0, n, per)]
        else:
            cuts, acc = [0], 0
            for j in range(p):
                if acc and acc + sizes[j] > group_bytes:
                    cuts.append(j)
                    acc = 0
                acc += sizes[j]
            cuts.append(p)
            for base in range(0, n, p):
                groups += [list(range(base + lo, base + hi)) for lo, hi in zip(cuts[:-1], cuts[1:])]
        return groups
    buckets = {}
    for i, k in enumerate(keys):
        buckets.setdefault(k, []).append(i)
    for k, idxs in buckets.items():
        per = max(1, min(len(idxs), group_bytes // max(sizes[idxs[0]], 1)))
        groups += [idxs[i:i + per] for i in range(0, len(idxs), per)]
    return groups


def pack_host_tensors(tensors, device="cuda", amax=None, group_bytes: int = 512 << 20):
    """NVFP4-pack a list of host (CPU) weight tensors of any shapes through the GPU.  The tensors are
    split into groups of about ``group_bytes`` (``_plan_groups``) and all groups of one signature are
    streamed through one :class:`HostNvFp4Packer`, whose three streams overlap the copies and kernels of
    consecutive groups.  ``amax[i]`` (or None) is a calibrated global abs-max for tensor i.  Returns, in
    the order of ``tensors``, tuples (packed uint8, block scales float8_e4m3fn, scale2 fp32 0-dim), all on
    the host."""
    results = [None] * len(tensors)
    keys = [(tuple(t.shape), t.dtype) for t in tensors]
    sizes = [t.numel() * t.element_size() for t in tensors]
    by_signature = {}
    for ids in _plan_groups(keys, sizes, group_bytes):
        by_signature.setdefault(tuple(keys[i] for i in ids), []).append(ids)
    for signature, id_groups in by_signature.items():
        packer = HostNvFp4Packer([shape for shape, _ in signature], signature[0][1], device)
        groups = [[tensors[j] for j in ids] for ids in id_groups]
        out = packer.alloc_host_outputs(len(groups))
        av = None
        if amax is not None:
            av = [{k: amax[j] for k, j in enumerate(ids) if amax[j] is not None} for ids in id_groups]
        packer.pack(groups, out, av)
        for b, ids in enumerate(id_groups):
            for k, j in enumerate(ids):
                results[j] = (out[b]["packed"][k], out[b]["scales"][k].view(torch.float8_e4m3fn),
                              out[b]["scale2"][k].clone())
    return results
