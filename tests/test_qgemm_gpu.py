"""Real-quant GEMM consumers (tcgen05 kind::f8f6f4 and kind::mxf4nvf4) against the float64 oracle.

Tolerance: the kernels accumulate in fp32 inside the tensor cores in an order the hardware chooses,
so results are compared with the float64 sum at |err| <= 2^-7 * |y| + 2e-3 * sum_k |a_k b_k| * scale
(one bf16 ulp of the result plus an fp32-accumulation allowance); layouts and scale plumbing are
bit-exact (swizzle kernel)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import quant_oracle as qo  # noqa: E402

pytestmark = pytest.mark.gpu


_TILE_CODES = {"128": 128, "256": 256, "big": 512, "k2": 2}


def _force_tile(monkeypatch, tile):
    """Force one CTA tile shape of the real-quant GEMMs (process-wide switch of the library)."""
    from b200q import _cabi

    _cabi.lib.b200q_qgemm_tile_override(_TILE_CODES[tile])


@pytest.fixture(autouse=True)
def _automatic_tile_choice_after_each_test():
    yield
    from b200q import _cabi

    _cabi.lib.b200q_qgemm_tile_override(0)


def _ops():
    from b200q import ops
    return ops


def _check(got: torch.Tensor, want: np.ndarray, absdot: np.ndarray, what):
    g = got.float().cpu().numpy().astype(np.float64)
    tol = np.abs(want) * 2.0 ** -7 + 2e-3 * absdot + 1e-30
    bad = np.abs(g - want) > tol
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, worst " \
                          f"{np.max(np.abs(g - want) / tol):.2f}x"


@pytest.mark.parametrize("rows,cols", [(128, 16), (256, 32), (137, 21), (1, 4), (300, 16), (512, 512)])
def test_swizzle_scales_matches_oracle(rows, cols):
    ops = _ops()
    rng = np.random.default_rng(rows * 1000 + cols)
    s = rng.integers(0, 127, size=(rows, cols), dtype=np.uint8)
    got = ops.nvfp4_swizzle_scales(torch.from_numpy(s).cuda()).cpu().numpy()
    assert np.array_equal(got, qo.nvfp4_swizzle_scales(s))


def _fp8_case(m, n, k, seed, dtype, with_bias):
    rng = np.random.default_rng(seed)
    a8 = qo.e4m3_encode(rng.standard_normal((m, k)).astype(np.float32) * 2, "torch")
    b8 = qo.e4m3_encode(rng.standard_normal((n, k)).astype(np.float32) * 2, "torch")
    sa, sb = np.float32(0.013), np.float32(0.37)
    bias = rng.standard_normal(n).astype(np.float32) if with_bias else None
    if bias is not None:
        bias = torch.from_numpy(bias).to(dtype).float().numpy()
    return a8, b8, sa, sb, bias


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 256, 512), (256, 512, 1024), (100, 136, 80),
                                   (1, 128, 256), (333, 1000, 4096), (512, 4096, 512), (2048, 2048, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fp8_gemm_matches_float64_sum(m, n, k, dtype):
    if dtype is not torch.bfloat16 and m * n * k > 256 * 512 * 1024:
        pytest.skip("large shapes run in bf16 only")
    ops = _ops()
    T = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype]
    a8, b8, sa, sb, bias = _fp8_case(m, n, k, m + n + k, dtype, with_bias=(m % 2 == 0))
    got = ops.fp8_gemm(torch.from_numpy(a8).cuda(), torch.from_numpy(b8).cuda(), torch.tensor(sa), torch.tensor(sb),
                       None if bias is None else torch.from_numpy(bias).cuda(), dtype)
    ops.check_qgemm_status("cuda")
    af, bf = qo.e4m3_decode(a8).astype(np.float64), qo.e4m3_decode(b8).astype(np.float64)
    want = af @ bf.T * float(sa) * float(sb) + (0 if bias is None else bias.astype(np.float64))
    absdot = np.abs(af) @ np.abs(bf).T * float(sa) * float(sb)
    _check(got, want, absdot, f"fp8 {m}x{n}x{k}")
    # and the rounded oracle itself within one ulp of T
    ref = qo.fp8_gemm(a8, b8, sa, sb, bias, T).astype(np.float64)
    _check(got, ref, absdot, f"fp8 oracle {m}x{n}x{k}")


def test_fp8_gemm_tile_choices_agree(monkeypatch):
    ops = _ops()
    a8, b8, sa, sb, _ = _fp8_case(300, 520, 768, 5, torch.bfloat16, False)
    outs = []
    for tile in ("128", "256", "big", "k2"):
        _force_tile(monkeypatch, tile)
        outs.append(ops.fp8_gemm(torch.from_numpy(a8).cuda(), torch.from_numpy(b8).cuda(), torch.tensor(sa),
                                 torch.tensor(sb), None, torch.float32))
    ops.check_qgemm_status("cuda")
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])     # same K order: identical sums
    # two half sums added once: equal to fp32 rounding of the different summation order
    assert torch.allclose(outs[3], outs[0], rtol=1e-5, atol=1e-5 * float(outs[0].abs().max()))


def test_fp8_gemm_integer_inputs_are_exact():
    """Small integers: every product and partial sum is exact in fp32, so the result is too."""
    ops = _ops()
    rng = np.random.default_rng(0)
    a = rng.integers(-4, 5, size=(256, 512)).astype(np.float32)
    b = rng.integers(-4, 5, size=(384, 512)).astype(np.float32)
    got = ops.fp8_gemm(torch.from_numpy(a).cuda().to(torch.float8_e4m3fn), torch.from_numpy(b).cuda().to(torch.float8_e4m3fn),
                       torch.tensor(1.0), torch.tensor(1.0), None, torch.float32)
    ops.check_qgemm_status("cuda")
    assert np.array_equal(got.cpu().numpy(), a @ b.T)


def _nvfp4_operand(rng, rows, k):
    x = (rng.standard_normal((rows, k)) * np.exp(rng.standard_normal((rows, 1)))).astype(np.float32)
    packed, scales, s2 = qo.nvfp4_quantize(x, 16)
    return x, packed, scales, s2


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (128, 256, 512), (256, 512, 1024), (100, 136, 320),
                                   (1, 128, 64), (333, 1000, 4096), (512, 4096, 512), (2048, 2048, 2048)])
def test_nvfp4_gemm_matches_float64_sum(m, n, k):
    ops = _ops()
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    _, a4, sfa, s2a = _nvfp4_operand(rng, m, k)
    _, b4, sfb, s2b = _nvfp4_operand(rng, n, k)
    alpha = np.float32(s2a) * np.float32(s2b)
    bias = rng.standard_normal(n).astype(np.float32) if m % 2 == 0 else None
    if bias is not None:
        bias = torch.from_numpy(bias).to(torch.bfloat16).float().numpy()
    dev = lambda t: torch.from_numpy(t).cuda()  # noqa: E731
    got = ops.nvfp4_gemm(dev(a4), ops.nvfp4_swizzle_scales(dev(sfa)), dev(b4), ops.nvfp4_swizzle_scales(dev(sfb)),
                         torch.tensor(alpha), None if bias is None else dev(bias), torch.bfloat16)
    ops.check_qgemm_status("cuda")
    af = qo.nvfp4_dequantize(a4, sfa, 1.0).astype(np.float64)
    bf = qo.nvfp4_dequantize(b4, sfb, 1.0).astype(np.float64)
    want = af @ bf.T * float(alpha) + (0 if bias is None else bias.astype(np.float64))
    absdot = np.abs(af) @ np.abs(bf).T * float(alpha)
    _check(got, want, absdot, f"nvfp4 {m}x{n}x{k}")
    ref = qo.nvfp4_gemm(a4, sfa, b4, sfb, alpha, bias, "bf16").astype(np.float64)
    _check(got, ref, absdot, f"nvfp4 oracle {m}x{n}x{k}")


@pytest.mark.parametrize("tile", ["128", "256", "big", "k2"])
def test_nvfp4_gemm_exact_on_exactly_representable_products(tile, monkeypatch):
    """Codes in {0, +-1, +-2} with power-of-two block scales: every partial sum is an integer multiple
    of a power of two well inside fp32, so the kernel must reproduce the sum exactly; this pins the
    nibble order, the block-to-scale mapping and the row/column order of the scale tiles."""
    ops = _ops()
    _force_tile(monkeypatch, tile)
    rng = np.random.default_rng(1)
    m, n, k = 300, 1000, 512                       # ragged row and column tiles for every tile shape
    codes = np.array([0, 2, 4, 10, 12], dtype=np.uint8)          # 0, 1, 2, -1, -2
    qa, qb = rng.choice(codes, size=(m, k)), rng.choice(codes, size=(n, k))
    a4 = ((qa[:, 1::2] << 4) | qa[:, 0::2]).astype(np.uint8)
    b4 = ((qb[:, 1::2] << 4) | qb[:, 0::2]).astype(np.uint8)
    pow2 = np.array([0x28, 0x30, 0x38, 0x40, 0x48], dtype=np.uint8)   # E4M3 0.25, 0.5, 1, 2, 4
    sfa, sfb = rng.choice(pow2, size=(m, k // 16)), rng.choice(pow2, size=(n, k // 16))
    dev = lambda t: torch.from_numpy(t).cuda()  # noqa: E731
    got = ops.nvfp4_gemm(dev(a4), ops.nvfp4_swizzle_scales(dev(sfa)), dev(b4), ops.nvfp4_swizzle_scales(dev(sfb)),
                         torch.tensor(1.0), None, torch.float32)
    ops.check_qgemm_status("cuda")
    want = qo.nvfp4_dequantize(a4, sfa, 1.0).astype(np.float64) @ qo.nvfp4_dequantize(b4, sfb, 1.0).astype(np.float64).T
    assert np.array_equal(got.cpu().numpy().astype(np.float64), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fp8_gemm_operand_matches_oracle_bytes(dtype):
    ops = _ops()
    T = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype]
    rng = np.random.default_rng(3)
    x = torch.from_numpy((rng.standard_normal((64, 1000)) * 3).astype(np.float32)).to(dtype)
    x[0, :4] = torch.tensor([1e4, -1e4, float("nan"), 0.0], dtype=dtype)      # beyond the range: saturate
    x[1, :6] = torch.tensor([-0.0, float("inf"), -float("inf"), 1e-30, -1e-30, 6e-8], dtype=dtype)   # signed zero, infinities, tiny
    scale = torch.tensor(0.0123)
    for fused in (False, True):
        got = ops.fp8_gemm_operand(x.cuda(), scale.cuda(), fused=fused).view(torch.uint8).cpu().numpy()
        want = qo.fp8_to_gemm_operand(x.float().numpy(), np.float32(scale.item()), T, fused=fused)
        assert np.array_equal(got, want)
        assert got[0, 0] == 0x7E and got[0, 1] == 0xFE and (got[0, 2] & 0x7F) == 0x7F
    odd = x.flatten()[3:3 + 4099].cuda()                                   # unaligned start, ragged tail
    assert np.array_equal(ops.fp8_gemm_operand(odd, scale.cuda()).view(torch.uint8).cpu().numpy(),
                          qo.fp8_to_gemm_operand(odd.float().cpu().numpy(), np.float32(scale.item()), T))


# ------------------------------------------------------------------ layer level ---------------------

def _one_layer(cfg_name, k=512, n=384, bias=True, tokens=(4, 48)):
    import copy

    import b200q as mtq
    from torch import nn
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(k, n, bias=bias)).to(torch.bfloat16).cuda()
    x = torch.randn(*tokens, k, device="cuda", dtype=torch.bfloat16)
    mtq.quantize(model, copy.deepcopy(getattr(mtq, cfg_name)), lambda m: m(x))
    with torch.no_grad():
        fake = model(x)
    mtq.compress(model, config={"quant_gemm": False})       # first the dequantise-then-GEMM path
    with torch.no_grad():
        dequant = model(x)
    return mtq, model, x, fake, dequant


@pytest.mark.parametrize("cfg_name,impl", [("FP8_DEFAULT_CFG", "Fp8PerTensorLinear"), ("NVFP4_DEFAULT_CFG", "Nvfp4Linear")])
@pytest.mark.parametrize("bias", [True, False])
def test_real_quant_linear_runs_registered_gemm(cfg_name, impl, bias):
    """enable_real_quant_gemm switches the compressed layer to the tensor-core GEMM; the result
    agrees with the dequantise-then-bf16-GEMM path to bf16 rounding of the two different sums."""
    mtq, model, x, fake, dequant = _one_layer(cfg_name, bias=bias)
    from b200q import backends, ops
    from b200q.nn import RealQuantLinear
    assert isinstance(model[0], RealQuantLinear)
    backends.enable_real_quant_gemm(model)
    assert backends.is_real_quant_gemm_enabled(model)
    with torch.no_grad():
        out = model(x)
    ops.check_qgemm_status("cuda")
    assert model[0]._real_quant_gemm_impl == getattr(backends, impl).apply
    assert out.shape == dequant.shape and out.dtype == dequant.dtype
    err = (out.float() - dequant.float()).abs().max() / dequant.float().abs().max()
    assert err < 2e-2, err
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), dequant.float().flatten(), dim=0)
    assert cos > 0.9995, cos
    backends.disable_real_quant_gemm(model)
    with torch.no_grad():
        assert torch.equal(model(x), dequant)


def test_real_quant_gemm_not_used_when_shapes_do_not_qualify():
    mtq, model, x, fake, dequant = _one_layer("NVFP4_DEFAULT_CFG", k=544, n=384)     # k % 64 != 0
    from b200q import backends
    backends.enable_real_quant_gemm(model)
    with pytest.warns(UserWarning, match="no real-quant GEMM"):
        with torch.no_grad():
            out = model(x)
    assert torch.equal(out, dequant)


@pytest.mark.parametrize("cfg_name", ["FP8_DEFAULT_CFG", "NVFP4_DEFAULT_CFG"])
def test_real_quant_gemm_backward_uses_high_precision(cfg_name):
    mtq, model, x, fake, dequant = _one_layer(cfg_name, bias=True)
    from b200q import backends
    backends.enable_real_quant_gemm(model)
    xg = x.clone().requires_grad_(True)
    out = model(xg)
    out.float().sum().backward()
    w = model[0].weight_quantizer(model[0].weight)            # dequantised weight
    want = torch.ones_like(out) @ w
    assert torch.allclose(xg.grad.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert model[0].bias.grad is not None and torch.allclose(
        model[0].bias.grad.float(), torch.full_like(model[0].bias, x.shape[0] * x.shape[1]).float())


def test_fp8_layer_matches_oracle_end_to_end():
    """Uncompressed weight: both operands are cast by ops.fp8_gemm_operand; compare with the oracle
    restatement of _to_fp8 + _scaled_mm on the same tensors."""
    import b200q as mtq
    from b200q import backends, ops
    from b200q.nn import RealQuantLinear
    from torch import nn
    torch.manual_seed(1)
    model = nn.Sequential(nn.Linear(256, 128, bias=True)).to(torch.bfloat16).cuda()
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    mtq.quantize(model, mtq.FP8_DEFAULT_CFG, lambda m: m(x))
    model[0].__class__ = RealQuantLinear
    backends.enable_real_quant_gemm(model)
    with torch.no_grad():
        out = model(x)
    ops.check_qgemm_status("cuda")
    lin = model[0]
    sa = float(lin.input_quantizer.amax.float() / 448.0)
    sb = float(lin.weight_quantizer.amax.float() / 448.0)
    a8 = qo.fp8_to_gemm_operand(x.float().cpu().numpy(), np.float32(sa), "bf16")
    b8 = qo.fp8_to_gemm_operand(lin.weight.detach().float().cpu().numpy(), np.float32(sb), "bf16")
    want = qo.fp8_gemm(a8, b8, np.float32(sa), np.float32(sb), lin.bias.detach().float().cpu().numpy(), "bf16")
    af, bfm = qo.e4m3_decode(a8).astype(np.float64), qo.e4m3_decode(b8).astype(np.float64)
    _check(out, want.astype(np.float64), np.abs(af) @ np.abs(bfm).T * sa * sb, "fp8 layer")


def _golden_fp8_cases():
    from _util import load, to_f32 as unbits
    d = load("fp8_gemm")
    for i in range(4):
        m, n, k, t, wb = (int(v) for v in d[f"case{i}_meta"])
        T = ["f32", "f16", "bf16"][t]
        yield i, T, {key: d[f"case{i}_{key}"] for key in ("x", "w", "y", "a8", "b8", "scale_a", "scale_b")}, \
            (d[f"case{i}_bias"] if wb else None), unbits


def test_fp8_linear_matches_reference_fixture():
    """The reference's fp8_per_tensor_gemm run on the CPU (tests/golden/make_golden.py): operand bytes
    bit-exact, output within the accumulation tolerance."""
    ops = _ops()
    TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    for i, T, c, bias, unbits in _golden_fp8_cases():
        x = torch.from_numpy(unbits(c["x"], T)).to(TD[T]).cuda()
        w = torch.from_numpy(unbits(c["w"], T)).to(TD[T]).cuda()
        sa, sb = torch.from_numpy(c["scale_a"]).cuda(), torch.from_numpy(c["scale_b"]).cuda()
        a8, b8 = ops.fp8_gemm_operand(x, sa), ops.fp8_gemm_operand(w, sb)
        assert np.array_equal(a8.view(torch.uint8).cpu().numpy(), c["a8"]), f"case {i} activation bytes"
        assert np.array_equal(b8.view(torch.uint8).cpu().numpy(), c["b8"]), f"case {i} weight bytes"
        b = None if bias is None else torch.from_numpy(unbits(bias, T)).to(TD[T]).cuda()
        got = ops.fp8_gemm(a8, b8, sa, sb, b, TD[T])
        ops.check_qgemm_status("cuda")
        af, bf = qo.e4m3_decode(c["a8"]).astype(np.float64), qo.e4m3_decode(c["b8"]).astype(np.float64)
        absdot = np.abs(af) @ np.abs(bf).T * float(c["scale_a"]) * float(c["scale_b"])
        _check(got, unbits(c["y"], T).astype(np.float64), absdot, f"fixture case {i}")


def test_nvfp4_quantize_saturating_scales_for_data_beyond_the_amax():
    """Activations above a calibrated amax: with saturate_scales the block scale stops at 448 (oracle
    cast "sat"), without it the tensor cast's NaN code appears (oracle cast "torch"); both bit-exact."""
    ops = _ops()
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    x[3, 32:48] *= 40.0                                  # one block far beyond the amax below
    xt = torch.from_numpy(x).to(torch.bfloat16)
    xf = xt.float().numpy()
    amax = np.float32(3.0)
    for sat, cast in ((True, "sat"), (False, "torch")):
        packed, scales, s2 = ops.nvfp4_quantize(xt.cuda(), amax=torch.tensor(amax), saturate_scales=sat)
        want_p, want_s, want_s2 = qo.nvfp4_quantize(xf, 16, amax=amax, cast=cast)
        assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), want_s)
        assert np.float32(s2.item()) == want_s2
        ok = (want_s & 0x7F) != 0x7F                     # codes of a NaN-scaled block are unspecified
        assert np.array_equal(packed.cpu().numpy().reshape(64, 16, 8)[ok], want_p.reshape(64, 16, 8)[ok])
    assert ((want_s & 0x7F) == 0x7F).sum() >= 1          # the torch cast did produce the NaN code


@pytest.mark.parametrize("m,n,k", [(256, 1024, 4096 + 256), (100, 520, 2048), (128, 128, 256)])
def test_gemm_k_split_over_a_cluster_matches(m, n, k, monkeypatch):
    """The cluster K-split (two CTAs per tile, partner's tile through distributed shared memory)
    against the single-CTA result, FP8 and NVFP4, ragged tiles and an odd number of K blocks; exact
    integer data must come out exactly."""
    ops = _ops()
    rng = np.random.default_rng(k)
    a8 = qo.e4m3_encode(rng.standard_normal((m, k)).astype(np.float32), "torch")
    b8 = qo.e4m3_encode(rng.standard_normal((n, k)).astype(np.float32), "torch")
    _, a4, sfa, _ = _nvfp4_operand(rng, m, k)
    _, b4, sfb, _ = _nvfp4_operand(rng, n, k)
    dev = lambda t: torch.from_numpy(t).cuda()  # noqa: E731
    one = torch.tensor(1.0)
    res = {}
    for tile in ("128", "k2"):
        _force_tile(monkeypatch, tile)
        res[tile] = (ops.fp8_gemm(dev(a8), dev(b8), one, one, None, torch.float32),
                     ops.nvfp4_gemm(dev(a4), ops.nvfp4_swizzle_scales(dev(sfa)), dev(b4),
                                    ops.nvfp4_swizzle_scales(dev(sfb)), one, None, torch.float32))
    ops.check_qgemm_status("cuda")
    for i in range(2):
        ref, got = res["128"][i], res["k2"][i]
        assert torch.allclose(got, ref, rtol=2e-5, atol=2e-5 * float(ref.abs().max()))
    ai = rng.integers(-3, 4, size=(m, k)).astype(np.float32)
    bi = rng.integers(-3, 4, size=(n, k)).astype(np.float32)
    got = ops.fp8_gemm(torch.from_numpy(ai).cuda().to(torch.float8_e4m3fn), torch.from_numpy(bi).cuda().to(torch.float8_e4m3fn),
                       one, one, None, torch.float32)
    ops.check_qgemm_status("cuda")
    assert np.array_equal(got.cpu().numpy(), ai @ bi.T)


def test_a_reported_wait_run_out_reaches_the_caller():
    """Host side of the bounded waits: a kernel that gives up a wait ORs an error bit into the device
    status word; ``check_qgemm_status`` turns a non-zero word into an exception and clears it.  The word
    is written from the host here — no kernel is made to time out."""
    from b200q import ops

    word = ops.qgemm_status("cuda")
    ops.check_qgemm_status("cuda")            # clean
    word.fill_(0x400)
    with pytest.raises(RuntimeError, match="0x400"):
        ops.check_qgemm_status("cuda")
    assert int(word.item()) == 0
    ops.check_qgemm_status("cuda")
