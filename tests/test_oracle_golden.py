"""The CPU oracle against golden vectors produced by the reference itself (CPU, no GPU needed)."""
import numpy as np
import pytest

from oracle import quant_oracle as qo
from _util import load, same_bits, same_values, to_f32

TS = ("f32", "f16", "bf16")


def test_fake_int_matches_reference_cpu_path():
    g = load("fake_int")
    n = 0
    for T in TS:
        for bits in (3, 4, 5, 7, 8, 11):
            for u in (0, 1):
                for nr in (0, 1):
                    for axis in (None, 0, 1):
                        k = f"{T}_b{bits}_u{u}_n{nr}_a{axis}"
                        x = to_f32(g[k + "_x"], T)
                        amax = g[k + "_amax"]
                        y = qo.fake_int(x, amax, bits, bool(u), bool(nr), T, cpu_flavour=True)
                        assert same_values(y, to_f32(g[k + "_y"], T)), k
                        # kernel flavour differs only in the epsilon rule and the unsigned floor
                        y2 = qo.fake_int(x, amax, bits, bool(u), bool(nr), T)
                        assert same_values(y2, y), k
                        n += 1
    assert n == 216
    y = qo.fake_int(g["tiny_x"], g["tiny_amax"], 8, False, True, "f32", cpu_flavour=True)
    assert same_values(y, g["tiny_y"])
    assert np.all(y[3] == 0)


def test_fake_e4m3_matches_reference_eager():
    g = load("fake_e4m3")
    for T in TS:
        x = to_f32(g[f"{T}_x"], T)
        assert same_bits(qo.fake_e4m3(x, g[f"{T}_amax"], T, eager=True), to_f32(g[f"{T}_y"], T)), T
        assert same_bits(qo.fake_e4m3(x, None, T), to_f32(g[f"{T}_y_noamax"], T)), T
        for axis in (0, 1):
            y = qo.fake_e4m3(x, g[f"{T}_amax_a{axis}"], T, eager=True)
            assert same_bits(y, to_f32(g[f"{T}_y_a{axis}"], T)), (T, axis)


def test_e4m3_encode_edges():
    v = np.array([448, 463, 464, 465, 480, 1000, np.nan, -465, -448, 0, -0.0, 2 ** -9, 2 ** -10,
                  1.5 * 2 ** -10, 0.0009765625 * 3], dtype=np.float32)
    t = qo.e4m3_encode(v, "torch")
    assert list(t[:9]) == [126, 126, 126, 127, 127, 127, 127, 255, 254]
    s = qo.e4m3_encode(v, "sat")
    assert list(s[:9]) == [126, 126, 126, 126, 126, 126, 127, 254, 254]
    # smallest subnormal 2^-9; half of it ties to even (0); 1.5*2^-10 rounds up
    assert list(s[9:14]) == [0, 0x80, 1, 0, 1]
    # round trip of every code
    codes = np.arange(256, dtype=np.uint8)
    vals = qo.e4m3_decode(codes)
    ok = ~np.isnan(vals)
    back = qo.e4m3_encode(vals[ok], "sat")
    assert np.array_equal(back, codes[ok])


def test_nvfp4_matches_reference():
    g = load("nvfp4")
    assert np.array_equal(qo.e2m1_encode(g["cast_v"]), g["cast_code"])
    for T in TS:
        for j in range(3):
            k = f"{T}_{j}"
            x = to_f32(g[k + "_x"], T)
            packed, scales, s2 = qo.nvfp4_quantize(x, 16)
            assert np.array_equal(packed, g[k + "_packed"]), k
            assert np.array_equal(scales, g[k + "_scales"]), k
            assert same_bits(np.array([s2]), g[k + "_s2"]), k
            if k + "_deq" in g:
                d = qo.nvfp4_dequantize(packed, scales, s2, 16, T)
                assert same_bits(d, to_f32(g[k + "_deq"], T)), k
            p2, sc2, _ = qo.nvfp4_quantize(x, 16, s2=g[k + "_clip_s2"][0])
            assert np.array_equal(sc2, g[k + "_clip_scales"]), k
            assert np.array_equal(p2, g[k + "_clip_packed"]), k
    # the clipped case really exercises the overflowing block-scale cast
    assert any((g[f"{T}_{j}_clip_scales"] == 0x7F).any() for T in TS for j in range(3))


def test_int4_cpu_flavour_matches_reference_and_kernel_flavour_differs_only_at_ties():
    g = load("int4")
    for T in TS:
        for j in range(3):
            k = f"{T}_{j}"
            x = to_f32(g[k + "_x"], T)
            block = int(g[k + "_block"])
            packed, scales = qo.int4_quantize(x, block, T, flavour="cpu")
            assert same_bits(scales.reshape(-1), to_f32(g[k + "_scales"], T).reshape(-1)), k
            assert np.array_equal(packed, g[k + "_packed"].reshape(-1)), k
            deq = qo.int4_dequantize(packed, scales, block, T)[: x.size]
            assert same_values(deq, to_f32(g[k + "_deq"], T).reshape(-1)), k
            pk, _ = qo.int4_quantize(x, block, T, flavour="kernel")
            hi = lambda p: (p >> 4).astype(int)  # noqa: E731
            lo = lambda p: (p & 15).astype(int)  # noqa: E731
            assert np.abs(hi(pk) - hi(packed)).max() <= 1 and np.abs(lo(pk) - lo(packed)).max() <= 1
            assert (pk != packed).mean() < (0.2 if T == "bf16" else 0.02), k


def test_int4_kernel_flavour_known_answers():
    # scale 1: values straight onto the grid; .5 ties round away from zero; bf16 rounds y+8 first
    x = np.zeros(16, dtype=np.float32)
    x[:8] = [7, -7, 0.5, -0.5, 1.5, 2.5, -2.5, 6.5]
    pk, sc = qo.int4_quantize(x, 16, "f32", flavour="kernel")
    assert sc[0, 0] == 1.0
    codes = np.stack([pk >> 4, pk & 15], -1).reshape(-1)[:8]
    assert list(codes) == [15, 1, 9, 8, 10, 11, 6, 15]
    # bf16: 0.484375 + 8 = 8.484375 -> bf16 spacing 1/16 -> 8.5 -> roundf -> 9 (exact math gives 8)
    x2 = np.zeros(16, dtype=np.float32)
    x2[0], x2[1] = 7.0, 0.484375
    pk2, _ = qo.int4_quantize(x2, 16, "bf16", flavour="kernel")
    assert pk2[0] == ((15 << 4) | 9)
    pk3, _ = qo.int4_quantize(x2, 16, "f32", flavour="kernel")
    assert pk3[0] == ((15 << 4) | 8)


def test_q8_matches_reference():
    g = load("q8")
    for T in TS:
        x = to_f32(g[f"{T}_x"], T)
        for name, fn in (("fp8", qo.fp8_quantize), ("int8", qo.int8_quantize)):
            s = to_f32(g[f"{T}_{name}_t_s"], T)
            q = fn(x, s.reshape(()), T)
            assert np.array_equal(q.view(np.uint8), g[f"{T}_{name}_t_q"].view(np.uint8)), (T, name)
            s = to_f32(g[f"{T}_{name}_a0_s"], T)
            q = fn(x, s.reshape(-1, 1), T)
            assert np.array_equal(q.view(np.uint8), g[f"{T}_{name}_a0_q"].view(np.uint8)), (T, name)
            s = to_f32(g[f"{T}_{name}_blk_s"], T)
            q = fn(x.reshape(16, 3, 32), s.reshape(16, 3, 1), T).reshape(16, 96)
            assert np.array_equal(q.view(np.uint8), g[f"{T}_{name}_blk_q"].view(np.uint8)), (T, name)


def test_amax_matches_reference():
    g = load("amax")
    for T in TS:
        x = to_f32(g[f"{T}_x"], T)
        assert same_bits(qo.reduce_amax(x).reshape(1), to_f32(g[f"{T}_all"], T))
        for axis in (0, 1, 2, -1):
            red = qo.quant_axis_to_reduce_axis(3, axis)
            assert same_bits(qo.reduce_amax(x, red).reshape(-1), to_f32(g[f"{T}_ax{axis}"], T))
        for blk in (16, 32):
            assert same_bits(qo.reduce_block_amax(x, blk).reshape(-1), to_f32(g[f"{T}_blk{blk}"], T))


def test_histogram_matches_reference_within_tolerance():
    """Counts are tolerance-compared: the reference ran torch's CPU histc here, whose edge
    placement differs from the CUDA formula the oracle restates by a few samples per edge."""
    g = load("hist")
    h = qo.HistogramOracle(2048)
    for b in range(3):
        x = to_f32(g[f"x{b}"], "bf16")
        h.collect(x)
        ref = g[f"hist{b}"]
        assert h.hist.size == ref.size, b
        assert h.hist.sum() == ref.sum(), b
        assert np.abs(h.hist - ref).sum() <= 2e-3 * ref.sum(), b
        assert np.allclose(h.edges, g[f"edges{b}"], rtol=1e-5, atol=0), b
    for p in (99.0, 99.9, 99.99, 100.0):
        amax, _ = qo.percentile_amax(h.hist, h.edges, p)
        assert abs(amax - g[f"pct_{p}"]) <= 1e-3 * g[f"pct_{p}"], p
    # entropy on the reference's own histogram: exact same algorithm -> same edge
    amax = qo.entropy_amax(g["hist2"], g["edges2"], 8, False)
    assert abs(amax - g["entropy"]) <= 1e-3 * g["entropy"]


def test_c_restatement_matches_numpy_oracle_and_golden():
    """oracle/nvfp4_ref.c (the CPU baseline that bench.py times) gives the reference's bytes."""
    from oracle import cref

    lib = cref.load()
    g = load("nvfp4")
    for j in (0, 1):
        x = g[f"bf16_{j}_x"]
        packed, scales, s2 = cref.nvfp4_quantize_bf16(lib, x.reshape(-1))
        assert np.array_equal(packed, g[f"bf16_{j}_packed"].reshape(-1))
        assert np.array_equal(scales, g[f"bf16_{j}_scales"].reshape(-1))
        assert same_bits(np.array([s2]), g[f"bf16_{j}_s2"])
    rng = np.random.default_rng(0)
    x = qo.round_bf16((rng.standard_t(4, size=(256, 512)) * 0.02).astype(np.float32))
    x[3, :16] = 0
    bits = (x.view(np.uint32) >> 16).astype(np.uint16)
    for amax in (-1.0, float(np.abs(x).max()) / 3):     # own amax, and a clipped one (NaN scale codes)
        packed, scales, s2 = cref.nvfp4_quantize_bf16(lib, bits.reshape(-1), amax, threads=3)
        wp, ws, ws2 = qo.nvfp4_quantize(x, 16, amax=None if amax < 0 else np.float32(amax))
        assert np.array_equal(packed, wp.reshape(-1)) and np.array_equal(scales, ws.reshape(-1)) and s2 == ws2


def test_export_packers_match_reference():
    g = load("export")
    for T in TS:
        w = to_f32(g[f"{T}_w"], T)
        s4 = qo.export_scaling_factor(w, 128)
        assert same_bits(s4, g[f"{T}_int4_scale"]), T
        assert np.array_equal(qo.pack_int4_export(w, s4, T), g[f"{T}_int4_packed"]), T
        s8 = qo.export_scaling_factor(w, 0)
        assert same_bits(s8, g[f"{T}_int8_scale"]), T
        assert np.array_equal(qo.int8_quantize(w, s8[:, None], "f32"), g[f"{T}_int8_q"]), T
        # a 0-dim fp32 scale does not promote a 16-bit weight: the quotient is rounded to T
        assert np.array_equal(qo.fp8_quantize(w, g[f"{T}_fp8_scale"].reshape(()), T), g[f"{T}_fp8_q"]), T
        p, _, _ = qo.nvfp4_quantize(w, 16, s2=g[f"{T}_nvfp4_wsf2"][0], scales=g[f"{T}_nvfp4_wsf"])
        assert np.array_equal(p, g[f"{T}_nvfp4_packed"]), T


# ------------------------------------------------------------------------------- MX formats ----
MX_FMTS = ("e2m1", "e3m2", "e2m3", "e4m3", "e5m2", "int8")


def test_mx_fake_matches_reference_known_answers():
    """The tables of the reference's own MX tests (same tolerances as those tests use)."""
    g = load("mx_known_answers")
    for fmt in MX_FMTS:
        x, want, block = g[fmt + "_in"], g[fmt + "_out"], int(g[fmt + "_block"])
        for sign in (1.0, -1.0):
            y = qo.mx_fake(x * np.float32(sign), block, fmt)
            atol = 1e-8 if fmt == "e2m1" else 1e-3
            assert np.allclose(y, want * np.float32(sign), rtol=1e-5, atol=atol), fmt
        if fmt == "e2m1":  # the reference runs this table at blocks 8, 16 and 32
            for b in (16, 32):
                y = qo.mx_fake(np.tile(x, (1, b // 8)), b, fmt)
                assert np.allclose(y, np.tile(want, (1, b // 8)), rtol=1e-5, atol=1e-8), b


def test_minifloat_round_against_value_tables():
    """Round-to-nearest-even against tables built from the format definitions: every value is a
    fixed point, every midpoint goes to the neighbour with an even mantissa."""
    for fmt in ("e2m1", "e3m2", "e2m3"):
        ebits, mbits, bias, fmax = qo.MX_FORMATS[fmt]
        vals = []
        for e in range(1 << ebits):
            for m in range(1 << mbits):
                vals.append((m / (1 << mbits)) * 2.0 ** (1 - bias) if e == 0
                            else (1 + m / (1 << mbits)) * 2.0 ** (e - bias))
        vals = np.array(vals, np.float32)
        assert vals[-1] == fmax and np.all(np.diff(vals) > 0)
        assert np.array_equal(qo.minifloat_round(vals, fmt), vals)
        mid = (vals[:-1] + vals[1:]) / 2
        want = np.where(np.arange(len(mid)) % 2 == 0, vals[:-1], vals[1:])
        assert np.array_equal(qo.minifloat_round(mid, fmt), want)
        assert np.array_equal(qo.minifloat_round(np.nextafter(mid, np.float32(0)), fmt), vals[:-1])
        assert np.array_equal(qo.minifloat_round(np.nextafter(mid, np.float32(1e9)), fmt), vals[1:])
        assert qo.minifloat_round(np.float32([fmax * 4, np.inf, np.nan]), fmt).tolist() == [fmax] * 3


def test_mx_scale_exponent_edges():
    # exact powers of two keep their exponent, anything above moves up, 2^127 is the clamp
    e = qo.mx_unscale_exponent(np.float32([6, 6.0000005, 12, 3, 0.75, 6 * 2.0 ** -126, 3.0e38]), "e2m1")
    assert e.tolist() == [0, 1, 1, -1, -3, -126, 126]
    y = qo.mx_fake(np.zeros((1, 32), np.float32), 32, "e4m3")
    assert np.all(y == 0)
    y = qo.mx_fake(np.float32([[np.inf] + [1.0] * 7]), 8, "e2m1")   # invalid amax: unscaled
    assert y[0, 1:].tolist() == [1.0] * 7 and y[0, 0] == 6.0


def test_mxfp4_qtensor_matches_reference_cpu_path():
    g = load("mxfp4")
    for T in TS:
        for j in range(3):
            k = f"{T}_{j}"
            x, block = to_f32(g[k + "_x"], T), int(g[k + "_block"])
            packed, scales = qo.mxfp4_quantize(x, block)
            assert np.array_equal(packed, g[k + "_packed"]), k
            assert np.array_equal(scales, g[k + "_scales"]), k
            deq = qo.mxfp4_dequantize(packed, scales, block, T)
            assert same_bits(deq, to_f32(g[k + "_deq"], T)), k


def test_torch_path_restatement_matches_reference_bytes():
    """oracle/torch_path.py (what `bench.py --impl reference` times) against the reference's bytes."""
    import torch

    from oracle import torch_path

    g = load("nvfp4")
    n = 0
    for T, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        for k in [k[: -len("_x")] for k in g.files if k.startswith(T + "_") and k.endswith("_x")]:
            if k + "_packed" not in g.files or k + "_amax" in g.files:
                continue
            x = torch.from_numpy(to_f32(g[k + "_x"], T)).to(dt)
            if x.shape[-1] % 16:
                continue
            packed, scales, s2 = torch_path.nvfp4_quantize(x, 16)
            assert np.array_equal(packed.numpy(), g[k + "_packed"]), k
            assert np.array_equal(scales.view(torch.uint8).numpy(), g[k + "_scales"]), k
            n += 1
    assert n >= 3


def test_fp8_gemm_operand_and_product_match_reference_cpu_run():
    """Fixture: the reference's fp8_per_tensor_gemm on the CPU.  The operand cast is bit-exact; the
    product (torch._scaled_mm there, a float64 sum here) agrees to one ulp of T plus an
    accumulation allowance."""
    d = load("fp8_gemm")
    for i in range(4):
        m, n, k, t, wb = (int(v) for v in d[f"case{i}_meta"])
        T = ["f32", "f16", "bf16"][t]
        x, w = to_f32(d[f"case{i}_x"], T), to_f32(d[f"case{i}_w"], T)
        sa, sb = np.float32(d[f"case{i}_scale_a"]), np.float32(d[f"case{i}_scale_b"])
        a8, b8 = qo.fp8_to_gemm_operand(x, sa, T), qo.fp8_to_gemm_operand(w, sb, T)
        assert np.array_equal(a8, d[f"case{i}_a8"]) and np.array_equal(b8, d[f"case{i}_b8"])
        bias = to_f32(d[f"case{i}_bias"], T) if wb else None
        y = qo.fp8_gemm(a8, b8, sa, sb, bias, T).astype(np.float64)
        want = to_f32(d[f"case{i}_y"], T).astype(np.float64)
        absdot = np.abs(qo.e4m3_decode(a8)).astype(np.float64) @ np.abs(qo.e4m3_decode(b8)).astype(np.float64).T
        tol = np.abs(want) * 2.0 ** -7 + 2e-3 * absdot * float(sa) * float(sb)
        assert np.all(np.abs(y - want) <= tol)
        assert np.mean(y == want) > (0.99 if T != "f32" else 0.1)


def test_nvfp4_scale_tiling_roundtrip():
    rng = np.random.default_rng(0)
    s = rng.integers(0, 127, size=(300, 40), dtype=np.uint8)
    t = qo.nvfp4_swizzle_scales(s)
    assert t.size == 3 * 12 * 512
    for r, c in [(0, 0), (31, 3), (32, 0), (137, 21), (299, 39)]:
        assert t[((r // 128) * 12 + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4] == s[r, c]
    assert t.sum() == s.sum()          # padding is zero


@pytest.mark.parametrize("fixture", ["awq", "awq128"])
@pytest.mark.parametrize("T", ["bf16", "f32"])
def test_awq_lite_restatement_matches_the_reference(fixture, T):
    """The oracle's awq_lite search (statistics, scale function, loss per alpha, selection) against what
    the reference computed on the CPU: bf16 statistics bit for bit, fp32 ones to the summation order of a
    mean, losses to 1e-4 (5e-4 behind this test's silu), the selected alpha exactly and its scale to 1e-5."""
    g = load(fixture)
    p = T + "_"
    w_up, w_down = to_f32(g[p + "w_up"], T), to_f32(g[p + "w_down"], T)
    xs = [to_f32(g[f"{p}x{i}"], T) for i in range(2)]

    def silu(v):
        return (v.astype(np.float64) / (1.0 + np.exp(-v.astype(np.float64)))).astype(np.float32)

    hs = [qo.round_to(silu(qo.awq_linear(x, w_up, T)), T) for x in xs]
    for name, w, inputs in (("up_proj", w_up, xs), ("down_proj", w_down, hs)):
        k = f"{p}{name}_"
        alphas = [float(a) for a in g[k + "alphas"]]
        wsc, asc, losses, best, scale = qo.awq_lite_search(w, inputs, 128, alphas, T)
        if T == "bf16":
            assert np.array_equal(wsc, g[k + "weight_scale"]) and np.array_equal(asc, g[k + "act_scale"])
        else:
            assert np.allclose(wsc, g[k + "weight_scale"], rtol=5e-6) and np.allclose(asc, g[k + "act_scale"], rtol=5e-6)
        # (the down projection's inputs pass through this test's own silu, whose last bit can differ from
        # torch's: in fp32 that moves single quantisation ties, a few 1e-4 of a loss)
        assert np.allclose(np.array(list(losses.values())), g[k + "losses"], rtol=1e-4 if name == "up_proj" else 5e-4)
        assert best == float(g[k + "best_alpha"])
        assert np.allclose(scale, g[k + "best_scale"], rtol=1e-5)
