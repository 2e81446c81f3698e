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


def _run_noalloc(cabi, tensors, stream=None, with_scales=True, with_s2=True):
    """Quantise `tensors` with the allocation-free entry point: the test owns every buffer."""
    from b200q.ops import dtype_code

    n = len(tensors)
    packed = [torch.full((t.numel() // 2,), 0xAA, dtype=torch.uint8, device="cuda") for t in tensors]
    scales = [torch.full((t.numel() // 16,), 0xAA, dtype=torch.uint8, device="cuda") for t in tensors]
    s2 = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
    descs = (cabi.NvFp4Desc * n)()
    for i, t in enumerate(tensors):
        descs[i].x, descs[i].packed = t.data_ptr(), packed[i].data_ptr()
        descs[i].scales = scales[i].data_ptr() if with_scales else None
        descs[i].amax = None                      # ignored by this entry point
        descs[i].s2 = s2.data_ptr() + 4 * i if with_s2 else None
        descs[i].nblocks = t.numel() // 16
        descs[i].tile_begin = -123                # ignored as well
    torch.cuda.synchronize()                      # the buffers above were filled on torch's stream
    handle = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
    cabi.call("b200q_nvfp4_group_quantize_noalloc", ctypes.cast(descs, ctypes.c_void_p), n,
              dtype_code(tensors[0]), handle)
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


def test_noalloc_group_at_its_capacity_on_a_side_stream_against_the_oracle():
    """Exactly 1024 tensors (the limit, 16 chunks of the staged table) of one block each, on a stream
    other than torch's current one; every tensor is checked against the CPU oracle directly."""
    from b200q import _cabi as cabi
    from oracle import quant_oracle as qo

    n = cabi.call("b200q_nvfp4_group_max_tensors_noalloc")
    g = torch.Generator(device="cuda").manual_seed(11)
    # one 32-byte aligned input per tensor (row stride 16 bf16 = 32 bytes)
    pool = (torch.randn((n, 16), generator=g, device="cuda") * torch.linspace(0.01, 3.0, n, device="cuda")[:, None]
            ).to(torch.bfloat16)
    tensors = [pool[i] for i in range(n)]
    side = torch.cuda.Stream()
    packed, scales, s2 = _run_noalloc(cabi, tensors, stream=side)
    host = pool.float().cpu().numpy()
    for i in (0, 1, 63, 64, 65, 511, 1022, 1023):       # chunk boundaries and both ends
        wp, ws, ws2 = qo.nvfp4_quantize(host[i:i + 1], 16)
        assert s2[i].item() == float(ws2), i
        assert np.array_equal(scales[i].cpu().numpy(), ws.reshape(-1)), i
        assert np.array_equal(packed[i].cpu().numpy(), wp.reshape(-1)), i
    # all of them against the ordinary single-tensor entry point
    from b200q import ops
    for i in range(0, n, 97):
        rp, rs, r2 = ops.nvfp4_quantize(tensors[i].reshape(1, 16))
        assert torch.equal(packed[i], rp.reshape(-1)) and torch.equal(scales[i], rs.view(torch.uint8).reshape(-1))
        assert s2[i].item() == r2.item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_noalloc_group_other_dtypes_and_absent_optional_outputs(dtype):
    """fp16 / fp32 inputs, and descriptors without block-scale and global-scale outputs (both are
    optional in the grouped kernels): codes must still equal the ordinary grouped entry's."""
    from b200q import _cabi as cabi
    from b200q.ops import NvFp4Group

    g = torch.Generator(device="cuda").manual_seed(5)
    tensors = [(torch.randn(s, generator=g, device="cuda") * 0.05).to(dtype) for s in [(96, 256), (7, 32)]]
    ref_packed, ref_scales, ref_s2 = NvFp4Group(tensors).run()
    torch.cuda.synchronize()
    packed, scales, s2 = _run_noalloc(cabi, tensors)
    for i in range(len(tensors)):
        assert torch.equal(packed[i], ref_packed[i].reshape(-1))
        assert torch.equal(scales[i], ref_scales[i].view(torch.uint8).reshape(-1))
        assert s2[i].item() == ref_s2[i].item()
    packed, scales, s2 = _run_noalloc(cabi, tensors, with_scales=False, with_s2=False)
    for i in range(len(tensors)):
        assert torch.equal(packed[i], ref_packed[i].reshape(-1))
        assert bool((scales[i] == 0xAA).all()) and s2[i].item() == -1.0     # untouched


def test_noalloc_group_refuses_a_capturing_stream():
    """The table is copied from the callee's stack frame, so a stream that is being captured into a
    graph is refused before anything is enqueued; the capture itself stays valid and empty."""
    from b200q import _cabi as cabi

    t = _weights([(16, 64)], seed=4)[0]
    ref = _run_noalloc(cabi, [t])                 # first use of the device happens outside any capture
    out = torch.full((t.numel() // 2,), 0x55, dtype=torch.uint8, device="cuda")
    descs = (cabi.NvFp4Desc * 1)()
    descs[0].x, descs[0].packed, descs[0].nblocks = t.data_ptr(), out.data_ptr(), t.numel() // 16
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graph.capture_begin(capture_error_mode="thread_local")
        try:
            rc = cabi.lib.b200q_nvfp4_group_quantize_noalloc(ctypes.cast(descs, ctypes.c_void_p), 1, cabi.BF16,
                                                             side.cuda_stream)
        finally:
            graph.capture_end()
    assert rc == -7
    torch.cuda.synchronize()
    assert bool((out == 0x55).all())              # nothing ran, then or at capture end
    again = _run_noalloc(cabi, [t])               # and the entry point still works afterwards
    assert torch.equal(again[0][0], ref[0][0])
