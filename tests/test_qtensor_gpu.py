"""The real-quantisation cases of the reference's own test file
(tests/gpu/torch/quantization/test_qtensor_cuda.py: known dequantised values for INT4 / INT8 / FP8 per
tensor, per channel and per 1-D / 2-D block with and without padding, MXFP4, quantised data shapes,
scales taken from a quantiser's amax, FP8 with an amax and block sizes together, NVFP4 quantise /
dequantise on the E2M1 grid and on random data), on CUDA tensors through ``TensorQuantizer`` with
``fake_quant=False``.  NF4 (double-quantised INT4) is not part of this library and its cases are absent."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _quantizer(fake=False, **kw):
    import b200q as mtq

    return mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(fake_quant=fake, **kw)).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, BF])
@pytest.mark.parametrize(("shape", "check_memory"), [((256, 64), True), ((256, 32), False)])
def test_int4_blocks_save_memory_and_round_trip(dtype, shape, check_memory):
    """Reference :32-68 (the INT4 arm).  32 columns with a block of 64 pads every row."""
    q = _quantizer(num_bits=4, block_sizes={-1: 64})
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.rand(shape, generator=g, device="cuda").to(dtype)
    base = torch.cuda.memory_allocated()
    qx = q(x)
    used = torch.cuda.memory_allocated() - base
    if check_memory and dtype == BF:
        assert used / (x.numel() * x.element_size()) < 0.3
    assert torch.allclose(q(qx), x, rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize(("num_bits", "block_sizes", "scale_of", "name"), [
    ((2, 1), {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, lambda a: a / 448.0 / 6.0, "_double_scale"),
    ((4, 3), None, lambda a: a / 448.0, "_scale"),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, BF])
def test_scales_come_from_the_quantisers_amax(num_bits, block_sizes, scale_of, name, dtype):
    """Reference :70-105."""
    q = _quantizer(num_bits=num_bits, block_sizes=block_sizes)
    amax = torch.tensor(1.1, device="cuda")
    q.amax = amax
    g = torch.Generator(device="cuda").manual_seed(1)
    q(torch.rand(32, 32, generator=g, device="cuda").to(dtype))
    assert hasattr(q, name)
    assert torch.allclose(getattr(q, name).float().reshape(()), scale_of(amax))


_ACCURACY = [
    # INT4 blocks of 4 (the scale is 7 / amax in the input dtype; dequantisation divides by it)
    (4, {-1: 4}, None, [[0, 1, 2, 3, 4, 5, 6, 7]],
     [[0.0000, 0.8516, 2.1406, 2.9844, 4.0000, 5.0000, 6.0000, 7.0000]]),
    # INT4 with padding of the flattened input
    (4, {-1: 4}, None, [[0, 1, 2, 3, 4, 5, 6, 7, 3, 3]],
     [[0.0000, 0.8516, 2.1406, 2.9844, 4.0000, 5.0000, 6.0000, 7.0000, 2.9844, 2.9844]]),
    # INT8 per channel
    (8, None, 0, [[0, 1, 2, 3, 4, 5, 6, 7]],
     [[0.0000, 0.9922, 1.9844, 2.9844, 3.9688, 4.9688, 5.9688, 7.0000]]),
    # INT8 2-D blocks
    (8, {-1: 2, -2: 2}, None, [[0, 1, 2, 3], [4, 5, 6, 7]],
     [[0.0000, 1.0234, 1.9844, 2.9844], [4.0000, 5.0000, 5.9688, 7.0000]]),
    # FP8 2-D blocks
    ((4, 3), {-1: 2, -2: 2}, None, [[0, 1, 2, 3], [4, 5, 6, 7]],
     [[0.0000, 0.9844, 2.0000, 3.0000], [3.9375, 5.0000, 6.0000, 7.0000]]),
    # FP8 2-D blocks with padding
    ((4, 3), {-1: 2, -2: 2}, None, [[0, 1, 3], [4, 5, 7]],
     [[0.0000, 0.9844, 3.0000], [3.9375, 5.0000, 7.0000]]),
    # FP8 1-D blocks
    ((4, 3), {-1: 2}, None, [[0, 1, 2, 3], [4, 5, 6, 7]],
     [[0.0000, 1.0000, 1.9219, 3.0000], [3.9375, 5.0000, 6.0000, 7.0000]]),
    # FP8 per channel
    ((4, 3), None, 0, [[0, 1, 2, 3], [4, 5, 6, 7]],
     [[0.0000, 0.9609, 1.9219, 3.0000], [4.0000, 5.0000, 6.0000, 7.0000]]),
    # FP8 per tensor
    ((4, 3), None, None, [[0, 1, 2, 3], [4, 5, 6, 7]], [[0, 1, 2, 3], [4, 5, 6, 7]]),
]


@pytest.mark.parametrize(("num_bits", "block_sizes", "axis", "values", "expected"), _ACCURACY)
def test_known_dequantised_values(num_bits, block_sizes, axis, values, expected):
    """Reference :108-275: quantise, dequantise, compare with the listed bf16 values; the fake-quant
    result of the same configuration stays within the reference's tolerance of it."""
    x = torch.tensor(values, dtype=BF, device="cuda")
    q = _quantizer(num_bits=num_bits, block_sizes=block_sizes, axis=axis)
    deq = q(q(x))
    assert deq.shape == x.shape and deq.dtype == BF
    assert torch.allclose(deq, torch.tensor(expected, dtype=BF, device="cuda")), deq
    fake = _quantizer(fake=True, num_bits=num_bits, block_sizes=block_sizes, axis=axis)(x)
    assert torch.allclose(fake, deq, rtol=1e-1, atol=1e-1)


def test_mxfp4_round_trip_against_fake_quant():
    """Reference :262-268 (no listed values: the dequantised tensor is compared with fake quant)."""
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(512, 512, generator=g, device="cuda")
    cfg = dict(num_bits=(2, 1), block_sizes={-1: 32, "type": "dynamic", "scale_bits": (8, 0)})
    q = _quantizer(**cfg)
    deq = q(q(x))
    assert torch.allclose(_quantizer(fake=True, **cfg)(x), deq, rtol=1e-1, atol=1e-1)


_E2M1 = [0, 0.5, 1, 1.5, 2, 3, 4, 6, 0, -0.5, -1, -1.5, -2, -3, -4, -6]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, BF])
@pytest.mark.parametrize("shift", [0.0, -0.25, 0.25, 0.5])
def test_nvfp4_quantize_on_the_grid_and_between_grid_points(dtype, shift):
    """Reference :277-388: the sixteen E2M1 values themselves and the same values moved by a quarter or a
    half step, in blocks of 8; unpack (low nibble first), multiply by the scales, compare."""
    from b200q.qtensor import NVFP4QTensor

    x = (torch.tensor(_E2M1, device="cuda") + shift).unsqueeze(0).to(dtype)
    packed = NVFP4QTensor.quantize(x, 8)[0]._quantized_data
    scales, _ = NVFP4QTensor.get_weights_scaling_factor(x, 8)
    unscale = scales.to(torch.float32).unsqueeze(-1) * NVFP4QTensor.get_weights_scaling_factor_2(x)
    lut = torch.tensor(_E2M1, device="cuda")
    codes = torch.stack([packed & 0x0F, packed >> 4], dim=-1).reshape(1, -1).long()
    deq = (lut[codes].view(1, 2, 8) * unscale).view(1, -1).to(dtype)
    assert torch.allclose(deq, x, rtol=2e-1, atol=2e-1)


@pytest.mark.parametrize(("num_bits", "block_sizes", "shape"), [
    ((4, 3), {-1: 128, -2: 128}, (128, 576)),
    ((4, 3), {-1: 128, -2: 128}, (576, 128)),
])
def test_quantized_data_shape(num_bits, block_sizes, shape):
    """Reference :468-500: padding to whole 2-D blocks does not leak into the stored data's shape."""
    q = _quantizer(num_bits=num_bits, block_sizes=block_sizes)
    g = torch.Generator(device="cuda").manual_seed(3)
    qx = q(torch.rand(shape, generator=g, device="cuda"))
    assert tuple(qx._quantized_data.shape) == shape


@pytest.mark.parametrize("shape", [(128, 64), (64, 128, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, BF])
def test_nvfp4_quantize_dequantize(shape, dtype):
    """Reference :502-562: both dequantisation entries (``fast`` or not) return the same values, close to
    the input."""
    from b200q.qtensor import NVFP4QTensor

    bs = {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(shape, generator=g, device="cuda").to(dtype)
    qt, scale, double_scale = NVFP4QTensor.quantize(x, 16, try_tensorrt=False)
    std = qt.dequantize(dtype=dtype, fast=False, scale=scale, double_scale=double_scale, block_sizes=bs)
    fast = qt.dequantize(dtype=dtype, fast=True, scale=scale, double_scale=double_scale, block_sizes=bs)
    assert std.shape == x.shape and std.dtype == dtype
    assert torch.allclose(std, x, atol=0.5, rtol=0.1)
    assert torch.equal(std, fast)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, BF])
@pytest.mark.parametrize(("shape", "block_sizes"), [((128, 1152), {-1: 128}), ((256, 256), {-1: 64, -2: 64})])
def test_fp8_with_an_amax_and_block_sizes(dtype, shape, block_sizes):
    """Reference :564-594: a scalar amax on a block-quantised FP8 quantiser is ignored in favour of
    per-block scales."""
    q = _quantizer(num_bits=(4, 3), block_sizes=block_sizes)
    q.amax = torch.tensor(1.5, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(shape, generator=g, device="cuda").to(dtype)
    deq = q(q(x))
    assert torch.allclose(deq, x, rtol=1e-1, atol=1e-1)
    assert q._scale.numel() > 1


@pytest.mark.parametrize("values", [
    None,
    [[0.25, 0.75, 1.25], [1.75, 2.5, 3.5]],
    [[0.1, 2.5, 1.0, 4.8], [1.5, 1.25, 3.25, 5.0]],
    [[0, 0.75, 1.25], [1.75, 2.5, 5.5]],
    [[-0.25, -0.75, -1.25], [-1.75, -2.5, -3.5]],
    [[-0.1, -2.5, -1.0, -4.8], [-1.5, -1.25, -3.25, -5.0]],
    [[0, -0.75, -1.25], [-1.75, -2.5, -5.5]]])
def test_cast_fp4_equivalence(values):
    """Reference tests/gpu/torch/quantization/test_qtensor_cuda.py:398-445: the 4-bit code of each value
    equals the definition by the E2M1 midpoints, values on a midpoint going to the even code."""
    from b200q.qtensor import NVFP4QTensor

    x = (torch.randn(32, 16, generator=torch.Generator().manual_seed(0)) if values is None
         else torch.tensor(values, dtype=torch.float32)).cuda()
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5], device="cuda")
    up_on_tie = torch.tensor([0, 1, 0, 1, 0, 1, 0], device="cuda")
    magnitude = (x.abs().unsqueeze(-1) > bounds).sum(-1) + ((x.abs().unsqueeze(-1) == bounds) * up_on_tie).sum(-1)
    want = ((x < 0).to(torch.uint8) * 8 + magnitude.to(torch.uint8)).to(torch.uint8)
    got = NVFP4QTensor._cast_fp4(x)
    assert got.dtype == torch.uint8 and got.shape == x.shape
    # the sign of a value that rounds to zero is kept by the definition above and by the kernel alike
    assert torch.equal(got, want)


@pytest.mark.parametrize("shape", [(128, 64), (64, 128, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_nvfp4_dequantize_fast_equals_the_standard_one(shape, dtype):
    """Reference tests/gpu/torch/quantization/test_qtensor_cuda.py:534-572: ``fast=True`` changes nothing
    here (one kernel serves both), and the result stays close to the input."""
    from b200q.qtensor import NVFP4QTensor

    block_sizes = {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}
    x = torch.randn(shape, dtype=dtype, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    q, scale, double_scale = NVFP4QTensor.quantize(x, 16)
    standard = q.dequantize(dtype=dtype, fast=False, scale=scale, double_scale=double_scale, block_sizes=block_sizes)
    fast = q.dequantize(dtype=dtype, fast=True, scale=scale, double_scale=double_scale, block_sizes=block_sizes)
    assert torch.equal(fast, standard)
    assert torch.allclose(standard, x, atol=0.5, rtol=0.1)
