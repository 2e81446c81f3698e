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

    def pack(self, host_groups, host_out):
        """Quantise every group of ``host_groups`` (lists of pinned host tensors) into
        ``host_out`` (from :meth:`alloc_host_outputs`).  Returns after everything has landed."""
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
                    grp.run()
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
