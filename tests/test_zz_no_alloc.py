"""The allocation-free grouped NVFP4 entry point, called through the C ABI.

Some callers of this library cannot allocate device memory at the point where they quantise (a
plugin inside an engine's enqueue call, a server whose memory was handed out once at start-up),
so `b200q_nvfp4_group_quantize_noalloc` keeps its scratch inside the library.  Here it is given
only inputs and outputs and must produce exactly what the ordinary grouped entry points produce,
on two calls in a row with different tensor lists (the second call finds the first call's
descriptors and abs-max values still in the shared scratch and must not be disturbed by them).
The file name keeps this test last in collection order.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(shapes, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [(torch.randn(s, generator=g, device="cuda") * (0.02 * (i + 1))).to(torch.bfloat16)
            for i, s in enumerate(shapes)]


def _run_noalloc(cabi, tensors):
    """Quantise `tensors` with the allocation-free entry point: the test owns every buffer."""
    n = len(tensors)
    packed = [torch.full((t.numel() // 2,), 0xAA, dtype=torch.uint8, device="cuda") for t in tensors]
    scales = [torch.full((t.numel() // 16,), 0xAA, dtype=torch.uint8, device="cuda") for t in tensors]
    s2 = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
    descs = (cabi.NvFp4Desc * n)()
    for i, t in enumerate(tensors):
        descs[i].x, descs[i].packed, descs[i].scales = t.data_ptr(), packed[i].data_ptr(), scales[i].data_ptr()
        descs[i].amax = None                      # ignored by this entry point
        descs[i].s2 = s2.data_ptr() + 4 * i
        descs[i].nblocks = t.numel() // 16
        descs[i].tile_begin = -123                # ignored as well
    stream = torch.cuda.current_stream().cuda_stream
    cabi.call("b200q_nvfp4_group_quantize_noalloc", ctypes.cast(descs, ctypes.c_void_p), n, cabi.BF16, stream)
    torch.cuda.synchronize()
    return packed, scales, s2


def test_noalloc_group_matches_grouped_entry_points_twice_in_a_row():
    from b200q import _cabi as cabi
    from b200q.ops import NvFp4Group

    assert cabi.call("b200q_nvfp4_group_max_tensors_noalloc") == 1024
    first = _weights([(256, 4096), (64, 1024), (1000, 48), (3, 16)], seed=1)
    second = _weights([(128, 2048), (4096, 1440)], seed=2)        # fewer tensors, other sizes
    for tensors in (first, second):
        ref_packed, ref_scales, ref_s2 = NvFp4Group(tensors).run()
        torch.cuda.synchronize()
        packed, scales, s2 = _run_noalloc(cabi, tensors)
        for i, t in enumerate(tensors):
            assert torch.equal(packed[i], ref_packed[i].reshape(-1)), i
            assert torch.equal(scales[i], ref_scales[i].view(torch.uint8).reshape(-1)), i
            assert s2[i].item() == ref_s2[i].item(), i
            assert s2[i].item() == t.float().abs().max().item() / 2688.0 or np.isclose(
                s2[i].item(), t.float().abs().max().item() / 2688.0, rtol=1e-6)


def test_noalloc_group_rejects_oversized_and_bad_requests():
    from b200q import _cabi as cabi

    t = _weights([(16, 16)], seed=3)[0]
    out = torch.empty(128, dtype=torch.uint8, device="cuda")
    n = 1025
    descs = (cabi.NvFp4Desc * n)()
    for d in descs:
        d.x, d.packed, d.scales, d.nblocks = t.data_ptr(), out.data_ptr(), None, 16
    p = ctypes.cast(descs, ctypes.c_void_p)
    assert cabi.lib.b200q_nvfp4_group_quantize_noalloc(p, n, cabi.BF16, None) == -9
    assert b"capacity" in cabi.lib.b200q_strerror(-9)
    with pytest.raises(cabi.B200QError, match="capacity"):
        cabi.call("b200q_nvfp4_group_quantize_noalloc", p, n, cabi.BF16, None)
    assert cabi.lib.b200q_nvfp4_group_quantize_noalloc(None, 1, cabi.BF16, None) == -1
    assert cabi.lib.b200q_nvfp4_group_quantize_noalloc(p, 0, cabi.BF16, None) == -4
    descs[0].nblocks = 0
    assert cabi.lib.b200q_nvfp4_group_quantize_noalloc(p, 1, cabi.BF16, None) == -4
