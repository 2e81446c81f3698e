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
                "packed": [torch.empty((*s[:-1], s[-1] // 2), dtype=torch.uint8).pin_memory() for s in self.shapes],
                "scales": [torch.empty((*s[:-1], s[-1] // 16), dtype=torch.uint8).pin_memory() for s in self.shapes],
                "scale2": torch.empty(len(self.shapes), dtype=torch.float32).pin_memory(),
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


def pack_host_tensors(tensors, device="cuda", amax=None, group_bytes: int = 256 << 20):
    """NVFP4-pack a list of host (CPU) weight tensors of any shapes through the GPU: tensors are
    bucketed by (shape, dtype), every bucket is streamed through a :class:`HostNvFp4Packer` in groups of
    about ``group_bytes``.  ``amax[i]`` (or None) is a calibrated global abs-max for tensor i.  Returns, in
    the order of ``tensors``, tuples (packed uint8, block scales float8_e4m3fn, scale2 fp32 0-dim), all on
    the host."""
    results = [None] * len(tensors)
    buckets = {}
    for i, t in enumerate(tensors):
        buckets.setdefault((tuple(t.shape), t.dtype), []).append(i)
    for (shape, dtype), idxs in buckets.items():
        nbytes = 1
        for d in shape:
            nbytes *= d
        nbytes *= torch.empty((), dtype=dtype).element_size()
        per = max(1, min(len(idxs), group_bytes // max(nbytes, 1)))
        full = len(idxs) // per * per
        # groups of `per` tensors, then one smaller group for what is left
        for ids, g in ((idxs[:full], per), (idxs[full:], len(idxs) - full)):
            if not ids:
                continue
            packer = HostNvFp4Packer([shape] * g, dtype, device)
            groups = [[tensors[j] for j in ids[k:k + g]] for k in range(0, len(ids), g)]
            out = packer.alloc_host_outputs(len(groups))
            av = None
            if amax is not None:
                av = [{k: amax[j] for k, j in enumerate(ids[b:b + g]) if amax[j] is not None}
                      for b in range(0, len(ids), g)]
            packer.pack(groups, out, av)
            for b in range(len(groups)):
                for k in range(g):
                    results[ids[b * g + k]] = (out[b]["packed"][k], out[b]["scales"][k].view(torch.float8_e4m3fn),
                                               out[b]["scale2"][k].clone())
    return results
