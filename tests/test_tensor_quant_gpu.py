"""The autograd-level quantisation functions, after the reference's own test files
(tests/gpu/torch/quantization/test_tensor_quant_cuda.py and the shared cases of
tests/_test_utils/torch/quantization/tensor_quant_common.py): ``fake_tensor_quant`` per tensor / per
channel / unsigned / full range / every bit width / fp16 overflow / double input, clipped straight-through
gradients, ``scaled_e4m3`` with and without an amax, per channel, on a transposed view, and NVFP4
``dynamic_block_quant`` on the E2M1 grid and its rounding boundaries for blocks of 8, 16 and 32.
The expected values are the reference's torch formula ``clamp(round(x * (bound / amax))) / (bound / amax)``
(tests/_test_utils/torch/quantization/quant_utils.py:19-30)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tq():
    from b200q import tensor_quant

    return tensor_quant


def _rand(*shape, seed=0, dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda").to(dtype)


def quant(x, amax, num_bits=8, narrow_range=True):
    intmax = 2.0 ** (num_bits - 1) - 1.0
    intmin = -intmax if narrow_range else -intmax - 1
    scale = intmax / amax
    return torch.clamp((x * scale).round_(), intmin, intmax) / scale


def fp8_eager(x, amax):
    """Scale to the E4M3 range, cast, scale back (reference tensor_quant.py:49-61)."""
    dtype = x.dtype
    scale = 448.0 / amax.float()
    return (x.float() * scale).to(torch.float8_e4m3fn).float().div(scale).to(dtype)


# ---- fake_tensor_quant (shared cases :32-135) -----------------------------------------------------------

def test_double_input_runs(tq):
    x = _rand(2, 3).double() * 100
    y = tq.fake_tensor_quant(x, x.abs().max(), None, 7)
    assert y.dtype == torch.float64 and y.shape == x.shape
    assert torch.allclose(y.float(), quant(x.float(), x.abs().max().float(), 7), rtol=1e-6, atol=0)


def test_per_tensor_scale(tq):
    x = _rand(31, seed=1)
    assert torch.allclose(tq.fake_tensor_quant(x, x.abs().max()), quant(x, x.abs().max()))


def test_per_channel_scale_with_clipping(tq):
    x = _rand(3, 3, 6, 8, seed=123)
    amax = 0.7 * torch.amax(x.abs(), dim=(1, 2, 3), keepdim=True)
    assert torch.allclose(tq.fake_tensor_quant(x, amax), quant(x, amax))


def test_backward_is_straight_through(tq):
    x = _rand(3, 7, seed=2).requires_grad_(True)
    labels = torch.tensor([1, 5, 0], device="cuda")
    y = tq.fake_tensor_quant(x, x.abs().max(), None, 7)
    y.retain_grad()
    torch.nn.CrossEntropyLoss()(y, labels).backward()
    assert torch.allclose(y.grad, x.grad)


def test_unsigned(tq):
    x = _rand(31, seed=3).abs()
    assert torch.allclose(tq.fake_tensor_quant(x, x.abs().max(), None, 8, True), quant(x, x.abs().max(), num_bits=9))


def test_gradient_is_clipped_outside_amax(tq):
    x = _rand(3, 7, seed=4).requires_grad_(True)
    amax = x.detach().abs().max() / 2
    y = tq.fake_tensor_quant(x, amax, None, 8)
    torch.sum((y - 0.5) ** 2).backward()
    inside = (-amax <= x.detach()) & (x.detach() <= amax)
    assert torch.equal(x.grad != 0, inside)


def test_full_range(tq):
    x = _rand(31, seed=5).abs()
    want = quant(x, x.max(), num_bits=9, narrow_range=False)
    assert torch.allclose(tq.fake_tensor_quant(x, x.max(), None, 8, True, False), want)


def test_fp16_does_not_overflow_with_a_tiny_amax(tq):
    x = _rand(31, seed=6, dtype=torch.float16)
    y = tq.fake_tensor_quant(x, torch.tensor(1e-4, device="cuda").half(), None, 8, False)
    assert torch.isfinite(y).all()


# ---- the kernel entry itself (:42-108) ------------------------------------------------------------------

@pytest.mark.parametrize("num_bits", [3, 4, 5, 7, 8, 11])
@pytest.mark.parametrize("unsigned", [True, False])
def test_every_bit_width(tq, num_bits, unsigned):
    x = _rand(31, seed=7)
    if unsigned:
        x = x.abs()
    got = tq.fake_tensor_quant(x, x.abs().max(), None, num_bits, unsigned)
    want = quant(x, x.abs().max(), num_bits + int(unsigned))
    assert torch.allclose(got, want, rtol=0, atol=2e-7 * float(x.abs().max()) * 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("num_bits", [3, 4, 5, 7, 8, 11])
@pytest.mark.parametrize("unsigned", [True, False])
def test_amax_along_an_axis(tq, dtype, num_bits, unsigned):
    """amax along axis 1 of a 4-D tensor: the axis kernel and the broadcast form agree to the bit, and both
    equal the formula evaluated in fp32 and rounded to the tensor's dtype."""
    from b200q import ops

    x = _rand(3, 4, 5, 6, seed=8, dtype=dtype)
    if unsigned:
        x = x.abs()
    amax = torch.tensor([0.8, 0.9, 0.7, 0.6], device="cuda")
    got = tq.fake_tensor_quant(x, amax.view(1, -1, 1, 1), None, num_bits, unsigned)
    assert torch.equal(got, ops.fake_int(x, amax.view(1, -1, 1, 1), num_bits, unsigned))
    bound = 2.0 ** (num_bits - 1 + int(unsigned)) - 1.0
    # a tensor numerator: torch evaluates ``number / cuda_tensor`` as reciprocal times number, one rounding more
    scale = torch.full((), bound, device="cuda") / amax.view(1, -1, 1, 1)
    want = (torch.clamp(torch.round(x.float() * scale), 0.0 if unsigned else -bound, bound) / scale).to(dtype)
    assert (got != want).float().mean() <= 0.02
    assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_low_precision_inputs(tq, dtype):
    x = _rand(31, seed=1234, dtype=dtype)
    got = tq.fake_tensor_quant(x, x.abs().max())
    want = quant(x.float(), x.abs().max().float())
    atol = {torch.bfloat16: 1e-1, torch.float16: 1e-3, torch.float32: 1e-6}[dtype]
    assert got.dtype == dtype and torch.allclose(got.float(), want, atol=atol)


def test_a_tiny_amax_zeroes_its_channel(tq):
    x = torch.rand(2, 3, 4, device="cuda")
    amax = torch.tensor([1.0, 1.0e-26, 1.0], device="cuda").view(1, 3, 1)
    y = tq.fake_tensor_quant(x, amax)
    assert y[:, 1, :].sum() == 0 and y[:, 0, :].abs().sum() > 0


# ---- scaled_e4m3 (:110-165) -----------------------------------------------------------------------------

def test_e4m3_without_a_scale(tq):
    x = _rand(4, 4, seed=9)
    assert torch.allclose(tq.scaled_e4m3(x, None, None, 4, 3), fp8_eager(x, torch.tensor(448.0, device="cuda")),
                          atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_e4m3_with_an_amax(tq, dtype):
    x = _rand(4, 4, seed=10, dtype=dtype)
    amax = x.abs().amax().reshape(1, 1)
    assert torch.allclose(tq.scaled_e4m3(x, amax, None, 4, 3), fp8_eager(x, amax))


def test_e4m3_on_a_transposed_view(tq):
    x = _rand(4, 4, seed=11).transpose(1, 0)
    assert not x.is_contiguous()
    got = tq.scaled_e4m3(x, None, None, 4, 3)
    assert torch.allclose(got, fp8_eager(x, torch.tensor(448.0, device="cuda")), atol=1e-4, rtol=1e-4)


def test_e4m3_backward(tq):
    x = _rand(3, 7, seed=12).requires_grad_(True)
    labels = torch.tensor([2, 0, 4], device="cuda")
    y = tq.scaled_e4m3(x, None, None, 4, 3)
    y.retain_grad()
    torch.nn.CrossEntropyLoss()(y, labels).backward()
    assert torch.allclose(y.grad, x.grad)


@pytest.mark.parametrize("axis", [0, 1, 2])
def test_e4m3_per_channel(tq, axis):
    x = _rand(4, 4, 4, seed=13)
    amax = x.abs().amax(dim=[a for a in range(3) if a != axis], keepdim=True)
    assert torch.allclose(tq.scaled_e4m3(x, amax, None, 4, 3), fp8_eager(x, amax))


def test_e4m3_other_formats_are_refused(tq):
    with pytest.raises(NotImplementedError):
        tq.scaled_e4m3(_rand(4, 4), None, None, 5, 2)


# ---- NVFP4 on its grid (:167-215) -----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_fp4_grid_points_and_rounding_boundaries(tq, dtype, block_size):
    """Inputs of one 16-element block (the reference passes 16 to its kernel for every width): grid values
    stay, exact mid-points go to the even code, values just below a mid-point go down."""
    g = torch.Generator(device="cuda").manual_seed(block_size)
    sign = (torch.randint(0, 2, (1, 8), generator=g, device="cuda") * 2 - 1).to(dtype)

    def check(test_in, test_out):
        reps = block_size // 8
        x = torch.cat((test_in,) * reps, dim=-1).to(dtype)
        want = torch.cat((test_out,) * reps, dim=-1).to(dtype)
        got = tq.dynamic_block_quant(x, 16, x.abs().amax().float(), None, (2, 1), (4, 3))
        assert torch.allclose(got, want), (got, want)

    grid = torch.tensor([[0, 0.5, 1, 1.5, 2, 3, 4, 6]], device="cuda")
    check(grid * sign, grid * sign)
    mid = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5, 6]], device="cuda")
    check(mid * sign, torch.tensor([[0.0, 1, 1, 2, 2, 4, 4, 6]], device="cuda") * sign)
    below = mid.clone()
    below[:, :-1] -= 0.1
    check(below * sign, grid * sign)


# ---- an amax kept along several dimensions (the reference's eager broadcast, tensor_quant.py:574-612) -----

@pytest.mark.parametrize("amax_shape", [(2, 2, 1, 2, 1), (2, 2, 1, 1, 1), (1, 2, 3, 1, 2)])
def test_amax_kept_along_several_dimensions(tq, amax_shape):
    x = _rand(2, 2, 3, 2, 2, seed=30)
    reduce = [d for d, n in enumerate(amax_shape) if n == 1]
    amax = x.abs().amax(dim=reduce, keepdim=True) * 0.8
    assert tuple(amax.shape) == amax_shape
    scale = torch.full((), 127.0, device="cuda") / amax
    want = torch.clamp(torch.round(x * scale), -128, 127) / scale
    assert torch.equal(tq.fake_tensor_quant(x, amax, None, 8, False, False), want)
    assert torch.allclose(tq.scaled_e4m3(x, amax, None, 4, 3), fp8_eager(x.clamp(-amax, amax), amax))


# ---- a tensor on a GPU that is not the current one (test_tensor_quant_cuda.py:33-41,148-155) --------------

@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensors_on_a_gpu_that_is_not_current(tq):
    from b200q import ops

    torch.cuda.set_device(0)
    other = torch.device("cuda", torch.cuda.device_count() - 1)
    x0 = _rand(3, 4, seed=50)
    x = x0.to(other)
    assert torch.cuda.current_device() == 0
    got = tq.fake_tensor_quant(x, x.abs().max(), None)
    assert got.device == other and torch.equal(got.cpu(), tq.fake_tensor_quant(x0, x0.abs().max(), None).cpu())
    e = tq.scaled_e4m3(x, None, None, 4, 3)
    assert e.device == other and torch.equal(e.cpu(), tq.scaled_e4m3(x0, None, None, 4, 3).cpu())
    w = _rand(64, 256, seed=51, dtype=torch.bfloat16)
    p0, s0, g0 = ops.nvfp4_quantize(w)
    p1, s1, g1 = ops.nvfp4_quantize(w.to(other))
    assert p1.device == other and torch.equal(p0.cpu(), p1.cpu()) and torch.equal(s0.cpu(), s1.cpu()) and g0.item() == g1.item()
    assert torch.cuda.current_device() == 0
