"""The reference's own GPU kernels, compiled unmodified from its checkout by ``oracle/build_ref.py``
(``oracle/_ref/``), as a second oracle beside the numpy restatement:

  fake_tensor_quant / _with_axis      modelopt/torch/quantization/src/tensor_quant_gpu.cu:41-140
  INT4_quantize / INT4_dequantize     .../src/tensor_quant_gpu.cu:262-366
  fake_e4m3fy / _with_axis            .../src/tensor_quant_gpu_fp8.cu:35-101
  fused_amax_convert                  .../src/tensor_quant_mx.cu:239-391
  fp4_fake_quant_block, fp4_dequantize  .../triton/fp4_kernel.py:45-383

Bit-exact where the arithmetic is IEEE on both sides (integer fake quant, the INT4 pack in the tensor's
own type with roundf, FP8 fake quant, the MX formats with power-of-two scales, NVFP4 dequantise to
16-bit types).  The reference's two NVFP4 fake-quant kernels replace the division ``|x| / scale`` of its
torch path by an approximate division (Triton) or a multiply by a rounded reciprocal (fast-math CUDA):
they differ from the torch path — the parity target — only at elements whose quotient sits on a rounding
boundary of E2M1, which the tests assert element by element together with the mismatch fraction.

Skipped when the modules were not built (no checkout of the reference on the build machine)."""
import pytest
import torch

from oracle import ref_ext

pytestmark = pytest.mark.gpu

TS = [torch.float32, torch.float16, torch.bfloat16]


def _need(mod):
    if mod is None:
        pytest.skip("the reference's extension was not built into oracle/_ref")
    return mod


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


@pytest.mark.parametrize("T", TS)
def test_int4_pack_kernel_of_the_reference(T):
    """b200q_int4_quantize against INT4_quantize: the multiply and the +8 in the tensor's type, roundf
    (half away from zero), first element in the high nibble — with every .5 tie, the clamp at both ends
    and an all-zero block (scale = inf: the reference's kernel turns the NaN products into code 15)."""
    from b200q import ops

    ext = _need(ref_ext.cuda_ext())
    x = (torch.randn(4096 * 128, generator=_gen(1), device="cuda") * 0.05).to(T)
    xb = x.view(-1, 128)
    ties = [7, -7, .5, -.5, 1.5, 2.5, -2.5, 6.5, -6.5, -7.5, 3.5, -3.5, 4.5, 5.5, -5.5, 0.]
    xb[0, :16] = torch.tensor(ties, device="cuda").to(T)       # block amax 7.5 -> scale 7 / 7.5
    xb[0, 16:] = 0
    xb[1] = 0
    xb[2, :16] = torch.tensor(ties, device="cuda").to(T)
    xb[2, 9] = 0                                                 # block amax 7 -> scale exactly 1: true ties
    xb[2, 16:] = 0
    scales = 7 / torch.maximum(xb.amax(-1, keepdim=True).abs(), xb.amin(-1, keepdim=True).abs())   # int4_tensor.py:62
    want = ext.INT4_quantize(x, scales, 128)
    got, got_scales = ops.int4_quantize(x, 128)
    assert torch.equal(got_scales.view(-1).float(), scales.view(-1).float())
    assert torch.equal(got, want)
    # scale 1 block: code = roundf(x + 8), half away from zero: 0.5 -> 9, -0.5 -> 8, 2.5 -> 11, -2.5 -> 6, -6.5 -> 2
    codes = torch.stack([want[128:136] >> 4, want[128:136] & 15], -1).reshape(-1).tolist()
    assert codes[:9] == [15, 1, 9, 8, 10, 11, 6, 15, 2], codes
    back_ref = ext.INT4_dequantize(want, scales, 128)
    back = ops.int4_dequantize(got, got_scales, 128).view(back_ref.shape)
    live = torch.isfinite(back_ref.float())
    assert torch.equal(back[live], back_ref[live]) and live.float().mean() > 0.99


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("bits,unsigned,narrow", [(8, False, True), (8, False, False), (4, False, False), (8, True, False), (3, False, True)])
def test_integer_fake_quant_kernels_of_the_reference(T, bits, unsigned, narrow):
    from b200q import ops

    ext = _need(ref_ext.cuda_ext())
    x = (torch.randn(1024, 4096, generator=_gen(2), device="cuda") * 3).to(T)
    if unsigned:
        x = x.abs()
    amax = x.abs().amax().float() * 0.7                       # values beyond amax clamp
    assert torch.equal(ops.fake_int(x, amax, bits, unsigned, narrow), ext.fake_tensor_quant(x, amax, bits, unsigned, narrow))
    rows = x.abs().amax(dim=1, keepdim=True).float() * 0.7
    assert torch.equal(ops.fake_int(x, rows, bits, unsigned, narrow),
                       ext.fake_tensor_quant_with_axis(x, rows.squeeze(), 0, bits, unsigned, narrow))
    cols = x.abs().amax(dim=0, keepdim=True).float() * 0.7
    assert torch.equal(ops.fake_int(x, cols, bits, unsigned, narrow),
                       ext.fake_tensor_quant_with_axis(x, cols.squeeze(), 1, bits, unsigned, narrow))


@pytest.mark.parametrize("T", TS)
def test_fp8_fake_quant_kernels_of_the_reference_on_out_of_range_data(T):
    """Values up to three times the amax: the kernel saturates to +-448 (the CPU eager cast of the
    reference would give NaN there), and so does ours."""
    from b200q import ops

    ext = _need(ref_ext.cuda_ext_fp8())
    x = (torch.randn(1024, 4096, generator=_gen(3), device="cuda") * 3).to(T)
    amax = (x.abs().amax() / 3).float()
    want = ext.fake_e4m3fy(x, amax)
    assert not want.isnan().any() and float(want.abs().max()) <= float(amax) * 1.01
    assert torch.equal(ops.fake_e4m3(x, amax), want)
    rows = (x.abs().amax(dim=1, keepdim=True) / 2).float()
    assert torch.equal(ops.fake_e4m3(x, rows), ext.fake_e4m3fy_with_axis(x, rows.squeeze(), 0))


def _nvfp4_case(T, seed=4):
    g = _gen(seed)
    x = (torch.randn(2048, 4096, generator=g, device="cuda") * torch.exp(torch.randn(2048, 1, generator=g, device="cuda"))).to(T)
    return x, x.abs().amax().float()


def _on_a_rounding_boundary(x, where):
    """For the elements selected by ``where``: is the torch path's quotient |x| / (e4m3 scale * scale2)
    within 4e-7 (three fp32 ulps) of one of E2M1's rounding boundaries?"""
    from b200q import ops

    _, scales, s2 = ops.nvfp4_quantize(x)
    scale = (scales.float() * s2).repeat_interleave(16, dim=-1)
    quot = (x.float().abs() / scale)[where]
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    rel = ((quot[:, None] - bounds[None, :]).abs() / bounds[None, :]).amin(dim=1)
    return rel <= 4e-7


# one ulp of a 16-bit type; fp32: a block scale one ulp apart moves the rounded product by up to two
_ULP = {torch.float32: 2.0 ** -22, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def _split_differences(mine, ref, T):
    """(different E2M1 code, beyond the last-bit allowance of T without being a code difference).  Neighbouring E2M1
    values are at least 20 % apart, so 1 % separates a different code from a last-bit difference."""
    a, b = mine.float(), ref.float()
    gap = (a - b).abs()
    big = torch.maximum(a.abs(), b.abs())
    code = gap > 0.01 * big
    return code, (gap > 1.01 * _ULP[T] * big) & ~code


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("seed", [4, 7])
def test_nvfp4_fake_quant_against_the_triton_kernel_of_the_reference(T, seed):
    """Where the Triton kernel and the torch path (= ours) disagree.
    (1) Different codes: the kernel's approximate division lands just beside exact ties of
    |x| / scale.  fp32 inputs: below 1e-6 of the elements; 16-bit inputs, where exact ties are common
    (8- and 11-bit significands over a 4-bit scale): up to 2e-3.  Every one sits on a rounding boundary.
    (2) Last-bit differences of whole tensors: the kernel's wrapper forms scale2 = amax / 2688 on the
    GPU, where torch multiplies by the rounded reciprocal of a host scalar; the torch path on the CPU —
    the golden vectors, and our kernel — divides.  The two differ by one ulp for about a quarter of all
    amax values (seed 4 is one), which shows in fp32 outputs only.  Nothing else differs by more than
    the last bit of the tensor's type."""
    from b200q import ops

    tri = _need(ref_ext.triton_fp4())
    x, amax = _nvfp4_case(T, seed)
    mine = ops.nvfp4_fake(x, amax)
    ref = tri.fp4_fake_quant_block(x, amax)
    code, beyond = _split_differences(mine, ref, T)
    assert not beyond.any()
    frac = code.float().mean().item()
    same_scale2 = (amax / 2688.0).item() == (amax.cpu() / 2688.0).item()      # GPU: amax * (1 / 2688)
    if same_scale2:
        assert frac <= (1e-6 if T == torch.float32 else 2e-3), frac
        if code.any():
            assert _on_a_rounding_boundary(x, code).all()
    else:
        # a scale2 one ulp apart also moves a few block scales across an E4M3 rounding boundary
        assert T == torch.float32 and seed == 4
        assert frac <= 1e-4, frac
        assert (mine != ref).float().mean().item() > 0.5


@pytest.mark.parametrize("T", TS)
def test_nvfp4_fake_quant_against_the_cuda_kernel_of_the_reference(T):
    """The fast-math CUDA kernel forms the block scale as e4m3(.) / (448 * 6 / amax) in double and
    multiplies by its reciprocal: its block scale can differ from e4m3(.) * (amax / 2688) in the last
    fp32 bit (whole blocks of an fp32 output one ulp apart), and its codes differ at rounding
    boundaries: at most 3e-3 of the elements, each of them on a boundary."""
    from b200q import ops

    ext = _need(ref_ext.cuda_ext_mx())
    x, amax = _nvfp4_case(T)
    mine = ops.nvfp4_fake(x, amax)
    ref = ext.fused_amax_convert(x, 16, ext.Types.E2M1, ext.Types.E4M3, amax)
    code, beyond = _split_differences(mine, ref, T)
    assert not beyond.any()
    frac = code.float().mean().item()
    assert frac <= 3e-3, frac
    if code.any():
        assert _on_a_rounding_boundary(x, code).all()


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("fmt,bits", [("E2M1", (2, 1)), ("E4M3", (4, 3)), ("INT8", 8)])
def test_mx_formats_against_the_cuda_kernel_of_the_reference(T, fmt, bits):
    from b200q import ops

    ext = _need(ref_ext.cuda_ext_mx())
    x, _ = _nvfp4_case(T, seed=5)
    want = ext.fused_amax_convert(x, 32, getattr(ext.Types, fmt), ext.Types.E8M0, None)
    assert torch.equal(ops.mx_fake(x, 32, bits), want)


@pytest.mark.parametrize("T", TS)
def test_nvfp4_dequantize_against_the_triton_kernel_of_the_reference(T):
    """16-bit outputs: bit-exact.  fp32: the Triton kernel multiplies (value * block scale) * scale2, the
    torch path value * (block scale * scale2): one fp32 rounding apart."""
    from b200q import ops

    tri = _need(ref_ext.triton_fp4())
    x, _ = _nvfp4_case(torch.bfloat16, seed=6)
    packed, scales, s2 = ops.nvfp4_quantize(x)
    want = tri.fp4_dequantize(packed, scales, s2, 16, 128, T)
    got = ops.nvfp4_dequantize(packed, scales, s2, T)
    if T == torch.float32:
        assert torch.allclose(got, want, rtol=1.2e-7, atol=0)
    else:
        assert torch.equal(got, want)
