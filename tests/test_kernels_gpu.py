"""CUDA kernels (through the C ABI) against the CPU oracle and the reference's golden vectors."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from _util import f32_from_tensor, load, same_bits, same_values, tensor_from_f32, to_f32, torch_dtype

pytestmark = pytest.mark.gpu
TS = ("f32", "f16", "bf16")


@pytest.fixture(scope="module")
def ops():
    from b200q import ops as _ops

    return _ops


def rnd(shape, T, seed, scale=1.0, heavy=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape).astype(np.float32)
    if heavy:
        x = x / np.sqrt(rng.chisquare(4, shape) / 4).astype(np.float32)
    return qo.round_to((x * np.float32(scale)).astype(np.float32), T)


# ----------------------------------------------------------------------------- amax ------------

@pytest.mark.parametrize("T", TS)
def test_amax_tensor_axis_blocks_golden(ops, T):
    g = load("amax")
    x = to_f32(g[f"{T}_x"], T)
    xt = tensor_from_f32(x, T)
    assert same_bits(f32_from_tensor(ops.amax_tensor(xt)).reshape(1), to_f32(g[f"{T}_all"], T))
    shape = x.shape
    for axis in (0, 1, 2):
        outer = int(np.prod(shape[:axis])); inner = int(np.prod(shape[axis + 1:]))
        got = f32_from_tensor(ops.amax_axis3(xt, outer, shape[axis], inner))
        assert same_bits(got, to_f32(g[f"{T}_ax{axis}"], T)), axis
    for blk in (16, 32):
        assert same_bits(f32_from_tensor(ops.amax_blocks(xt, blk)), to_f32(g[f"{T}_blk{blk}"], T))


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4096 * 33 + 5, 1 << 22])
def test_amax_tensor_sizes(ops, T, n):
    x = rnd((n,), T, n)
    got = f32_from_tensor(ops.amax_tensor(tensor_from_f32(x, T)))
    assert got == np.abs(x).max()


def test_amax_running_and_nan(ops):
    a = tensor_from_f32(rnd((4096,), "bf16", 1), "bf16")
    b = tensor_from_f32(rnd((4096,), "bf16", 2, scale=3.0), "bf16")
    out = ops.amax_tensor(a)
    ops.amax_tensor(b, out=out)
    assert out.item() == max(a.abs().max().item(), b.abs().max().item())
    c = a.clone(); c[17] = float("nan")
    assert torch.isnan(ops.amax_tensor(c))


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8192, 512, 1), (3, 40, 24), (2, 5, 7), (300, 1024, 1),
                                   (1, 3, 100000)])
def test_amax_axis_shapes(ops, T, shape):
    x = rnd(shape, T, sum(shape))
    got = f32_from_tensor(ops.amax_axis3(tensor_from_f32(x, T), *shape))
    assert same_bits(got, np.abs(x).max(axis=(0, 2)))


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("block", [8, 16, 32, 128, 256, 24, 4096])
def test_amax_blocks(ops, T, block):
    x = rnd((37 * block,), T, block)
    got = f32_from_tensor(ops.amax_blocks(tensor_from_f32(x, T), block))
    assert same_bits(got, np.abs(x.reshape(-1, block)).max(-1))


# ----------------------------------------------------------------------------- int fake quant --

def test_fake_int_golden_grid(ops):
    """Reference grid: bits x signed/unsigned x narrow x dtype x {per tensor, axis 0, axis 1}."""
    g = load("fake_int")
    for T in TS:
        for bits in (3, 4, 5, 7, 8, 11):
            for u in (0, 1):
                for nr in (0, 1):
                    for axis in (None, 0, 1):
                        k = f"{T}_b{bits}_u{u}_n{nr}_a{axis}"
                        x = to_f32(g[k + "_x"], T)
                        amax = torch.from_numpy(g[k + "_amax"]).cuda()
                        y = ops.fake_int(tensor_from_f32(x, T), amax, bits, bool(u), bool(nr))
                        assert same_values(f32_from_tensor(y), to_f32(g[k + "_y"], T)), k
                        want = qo.fake_int(x, g[k + "_amax"], bits, bool(u), bool(nr), T)
                        assert same_bits(f32_from_tensor(y), want), k


def test_fake_int_tiny_amax_is_zero(ops):
    g = load("fake_int")
    y = ops.fake_int(torch.from_numpy(g["tiny_x"]).cuda(), torch.from_numpy(g["tiny_amax"]).cuda(), 8, False, True)
    assert same_values(f32_from_tensor(y), g["tiny_y"])
    x = torch.randn(1000, device="cuda")
    assert torch.all(ops.fake_int(x, torch.tensor(1e-9, device="cuda")) == 0)


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("shape,axis", [((1024, 4096), 0), ((512, 1024), 1), ((33, 100), 0), ((33, 100), 1),
                                        ((4, 64, 24), 1), ((1, 5, 3), 2), ((7, 1037), None)])
def test_fake_int_layouts(ops, T, shape, axis):
    x = rnd(shape, T, 11 + len(shape), scale=0.02)
    if axis is None:
        amax = np.float32(np.abs(x).max() * 0.9).reshape(())
    else:
        red = tuple(d for d in range(len(shape)) if d != axis)
        amax = (np.abs(x).max(axis=red, keepdims=True) * np.float32(0.9)).astype(np.float32)
    y = ops.fake_int(tensor_from_f32(x, T), torch.from_numpy(np.asarray(amax)).cuda(), 8, False, True)
    assert same_bits(f32_from_tensor(y), qo.fake_int(x, amax, 8, False, True, T))


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("rows,cols,bits,narrow", [(4096, 4096, 8, True), (1000, 128, 4, False), (77, 16, 4, False),
                                                   (5, 1024, 8, True), (9, 8200, 8, True), (3, 32768, 8, True),
                                                   (64, 24, 4, False)])
def test_fake_int_rows_dynamic(ops, T, rows, cols, bits, narrow):
    x = rnd((rows, cols), T, rows + cols, scale=0.02)
    if T == "f32" and cols > 32768 // 1:
        pytest.skip("row too long for the fused kernel")
    y, am = ops.fake_int_rows_dynamic(tensor_from_f32(x, T), bits, False, narrow, return_amax=True)
    amax = np.abs(x).max(-1, keepdims=True)
    assert same_bits(f32_from_tensor(am), amax.reshape(-1))
    assert same_bits(f32_from_tensor(y), qo.fake_int(x, amax, bits, False, narrow, T))


# ----------------------------------------------------------------------------- FP8 fake --------

@pytest.mark.parametrize("T", TS)
def test_fake_e4m3_golden(ops, T):
    """In-range data: the reference's eager path and the saturating kernel agree except for the
    last-bit difference of reciprocal-times-448 vs 448/amax, which the oracle models both ways."""
    g = load("fake_e4m3")
    x = to_f32(g[f"{T}_x"], T)
    xt = tensor_from_f32(x, T)
    y = ops.fake_e4m3(xt, None)
    assert same_bits(f32_from_tensor(y), to_f32(g[f"{T}_y_noamax"], T))
    amax = g[f"{T}_amax"]
    y = ops.fake_e4m3(xt, torch.from_numpy(amax).cuda())
    assert same_bits(f32_from_tensor(y), qo.fake_e4m3(x, amax, T))
    for axis in (0, 1):
        am = g[f"{T}_amax_a{axis}"]
        y = ops.fake_e4m3(xt, torch.from_numpy(am).cuda())
        assert same_bits(f32_from_tensor(y), qo.fake_e4m3(x, am, T)), axis


@pytest.mark.parametrize("T", TS)
def test_fake_e4m3_saturates_and_all_codes(ops, T):
    # every E4M3 value and every midpoint between neighbours, both signs, plus out-of-range values
    vals = qo.e4m3_decode(np.arange(0, 127, dtype=np.uint8)).astype(np.float64)
    mids = (vals[1:] + vals[:-1]) / 2
    pts = np.concatenate([vals, mids, mids * (1 + 2 ** -12), mids * (1 - 2 ** -12), [470, 1000, 3e38, 0]])
    pts = np.concatenate([pts, -pts]).astype(np.float32)
    x = qo.round_to(pts, T)
    pad = (-x.size) % 16
    x = np.concatenate([x, np.zeros(pad, np.float32)])
    y = ops.fake_e4m3(tensor_from_f32(x, T), None)
    assert same_bits(f32_from_tensor(y), qo.fake_e4m3(x, None, T))
    amax = np.float32(300.0)  # calibrated amax below the data: the kernel saturates at +-amax-ish
    y = ops.fake_e4m3(tensor_from_f32(x, T), torch.tensor(300.0, device="cuda"))
    want = qo.fake_e4m3(x, amax, T)
    assert same_bits(f32_from_tensor(y), want)
    assert np.isfinite(want[np.isfinite(x)]).all()


def test_fake_e4m3_config2_shape_bf16(ops):
    g = torch.Generator().manual_seed(1000)
    x = torch.randn(8192, 4096, generator=g)
    idx = torch.randperm(4096, generator=torch.Generator().manual_seed(7))[:4]
    x[:, idx] *= 50
    x = x.bfloat16()
    xt = x.cuda()
    amax = ops.amax_tensor(xt)
    assert amax.item() == x.float().abs().max().item()
    y = ops.fake_e4m3(xt, amax)
    want = qo.fake_e4m3(x.float().numpy(), np.float32(amax.item()), "bf16")
    assert same_bits(f32_from_tensor(y), want)


# ----------------------------------------------------------------------------- NVFP4 -----------

@pytest.mark.parametrize("T", TS)
def test_nvfp4_golden(ops, T):
    g = load("nvfp4")
    for j in range(3):
        k = f"{T}_{j}"
        x = to_f32(g[k + "_x"], T)
        x = qo.pad_last(x, 16)
        xt = tensor_from_f32(x, T)
        packed, scales, s2 = ops.nvfp4_quantize(xt)
        assert np.array_equal(packed.cpu().numpy(), g[k + "_packed"]), k
        assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), g[k + "_scales"]), k
        assert same_bits(f32_from_tensor(s2).reshape(1), g[k + "_s2"]), k
        if k + "_deq" in g:
            d = ops.nvfp4_dequantize(packed, scales, s2, torch_dtype(T))
            assert same_bits(f32_from_tensor(d), to_f32(g[k + "_deq"], T)), k
        s2c = torch.from_numpy(g[k + "_clip_s2"]).cuda()
        p2, sc2, _ = ops.nvfp4_quantize(xt, scale2=s2c)
        assert np.array_equal(sc2.view(torch.uint8).cpu().numpy(), g[k + "_clip_scales"]), k
        assert np.array_equal(p2.cpu().numpy(), g[k + "_clip_packed"]), k


def test_nvfp4_every_rounding_boundary(ops):
    """_cast_fp4 golden points: with amax = 2688 the global scale is 1 and a block whose max is 6
    gets block scale 1, so the codes are those of the raw values."""
    g = load("nvfp4")
    v = g["cast_v"]
    v = v[np.isfinite(v) & (np.abs(v) <= 6)]
    code = qo.e2m1_encode(v)
    blocks = []
    for i in range(0, v.size, 15):
        chunk = v[i:i + 15]
        blocks.append(np.concatenate([chunk, np.zeros(15 - chunk.size, np.float32), [6.0]]))
    x = np.stack(blocks).astype(np.float32)
    packed, scales, s2 = ops.nvfp4_quantize(torch.from_numpy(x).cuda(), amax=torch.tensor(2688.0))
    assert s2.item() == 1.0 and (scales.float() == 1).all()
    p = packed.cpu().numpy()
    got = np.stack([p & 15, p >> 4], -1).reshape(x.shape)
    want = qo.e2m1_encode(x)
    assert np.array_equal(got, want)
    assert np.array_equal(got[:, :15].reshape(-1)[: v.size], code)


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("shape,scale,heavy", [((1024, 4096), 0.02, True), ((333, 48), 1.0, False),
                                               ((1, 16), 3.0, False), ((4096, 14336), 0.02, True)])
def test_nvfp4_quantize_vs_oracle(ops, T, shape, scale, heavy):
    if shape[0] * shape[1] > 2 ** 24 and T != "bf16":
        pytest.skip("large case only in bf16")
    x = rnd(shape, T, shape[1], scale, heavy)
    packed, scales, s2 = ops.nvfp4_quantize(tensor_from_f32(x, T))
    wp, ws, ws2 = qo.nvfp4_quantize(x, 16)
    assert s2.item() == ws2
    assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), ws)
    assert np.array_equal(packed.cpu().numpy(), wp)
    d = ops.nvfp4_dequantize(packed, scales, s2, torch_dtype(T))
    assert same_bits(f32_from_tensor(d), qo.nvfp4_dequantize(wp, ws, ws2, 16, T))


@pytest.mark.parametrize("T", TS)
def test_nvfp4_fake_vs_oracle(ops, T):
    x = rnd((512, 1024), T, 5, 1.0)
    x[0, :16] = 0
    x[1, :16] = 1e-9  # tiny block: keeps its (tiny) scale in the canonical definition
    x[2, 5] = -0.0
    xt = tensor_from_f32(x, T)
    amax = np.float32(np.abs(x).max())
    y = ops.nvfp4_fake(xt, torch.tensor(float(amax)))
    assert same_bits(f32_from_tensor(y), qo.nvfp4_fake(x, amax, 16, T))
    # calibrated amax below the data: block scales saturate at 448 instead of becoming NaN
    y = ops.nvfp4_fake(xt, torch.tensor(float(amax) / 4))
    want = qo.nvfp4_fake(x, amax / 4, 16, T)
    assert np.isfinite(want).all()
    assert same_bits(f32_from_tensor(y), want)


def test_nvfp4_supplied_block_scales(ops):
    x = rnd((64, 256), "bf16", 9, 0.02, True)
    xt = tensor_from_f32(x, "bf16")
    _, scales, s2 = ops.nvfp4_quantize(xt)
    sc = scales.view(torch.uint8).clone()
    sc[:, ::2] = torch.clamp(sc[:, ::2].int() - 3, min=1).to(torch.uint8)  # perturb: forces saturation
    packed, sc_out, _ = ops.nvfp4_quantize(xt, scale2=s2, scales_in=sc)
    wp, _, _ = qo.nvfp4_quantize(x, 16, s2=np.float32(s2.item()), scales=sc.cpu().numpy())
    assert np.array_equal(packed.cpu().numpy(), wp)
    assert torch.equal(sc_out.view(torch.uint8), sc)


def test_nvfp4_group_matches_single(ops):
    shapes = [(256, 4096), (64, 4096), (1024, 1024), (48, 16), (4096, 1440)]
    ts = [tensor_from_f32(rnd(s, "bf16", i + 40, 0.02, True), "bf16") for i, s in enumerate(shapes)]
    grp = ops.NvFp4Group(ts)
    packed, scales, s2 = grp.run()
    torch.cuda.synchronize()
    for i, t in enumerate(ts):
        p1, sc1, s21 = ops.nvfp4_quantize(t)
        assert torch.equal(packed[i], p1), i
        assert torch.equal(scales[i].view(torch.uint8), sc1.view(torch.uint8)), i
        assert s2[i].item() == s21.item(), i
        assert grp.amax[i].item() == t.abs().max().item()
    # a second run gives the same bytes (amax slots are reset, nothing accumulates)
    before = [p.clone() for p in packed]
    grp.run()
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(before, grp.packed))


# ----------------------------------------------------------------------------- INT4 ------------

@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("n,block", [(4096 * 128, 128), (77 * 16, 16), (13 * 32, 32), (5 * 24, 24), (3 * 1024, 1024)])
def test_int4_quantize_vs_oracle(ops, T, n, block):
    x = rnd((n,), T, n % 1000, 0.05)
    packed, scales = ops.int4_quantize(tensor_from_f32(x, T), block)
    wp, ws = qo.int4_quantize(x, block, T, flavour="kernel")
    assert same_bits(f32_from_tensor(scales), ws)
    assert np.array_equal(packed.cpu().numpy(), wp)
    d = ops.int4_dequantize(packed, scales, block)
    assert same_bits(f32_from_tensor(d), qo.int4_dequantize(wp, ws, block, T))


def test_int4_known_answers(ops):
    x = np.zeros(16, dtype=np.float32)
    x[:8] = [7, -7, 0.5, -0.5, 1.5, 2.5, -2.5, 6.5]
    p, s = ops.int4_quantize(torch.from_numpy(x).cuda(), 16)
    codes = np.stack([p.cpu().numpy() >> 4, p.cpu().numpy() & 15], -1).reshape(-1)[:8]
    assert list(codes) == [15, 1, 9, 8, 10, 11, 6, 15]
    x2 = np.zeros(16, dtype=np.float32); x2[0], x2[1] = 7.0, 0.484375
    p2, _ = ops.int4_quantize(torch.from_numpy(x2).cuda().bfloat16(), 16)
    assert p2[0].item() == ((15 << 4) | 9)


@pytest.mark.parametrize("T", TS)
def test_int4_golden_where_kernel_and_cpu_branch_agree(ops, T):
    """The reference's CPU branch pins scales exactly and codes wherever no .5 tie / T rounding of
    y+8 is involved (the oracle's two flavours mark those positions)."""
    g = load("int4")
    for j in range(3):
        k = f"{T}_{j}"
        x = to_f32(g[k + "_x"], T)
        block = int(g[k + "_block"])
        xp = qo.pad_last(x.reshape(-1), block)
        packed, scales = ops.int4_quantize(tensor_from_f32(xp, T), block)
        assert same_bits(f32_from_tensor(scales).reshape(-1), to_f32(g[k + "_scales"], T).reshape(-1)), k
        pk, _ = qo.int4_quantize(x, block, T, flavour="kernel")
        pc, _ = qo.int4_quantize(x, block, T, flavour="cpu")
        got = packed.cpu().numpy()
        assert np.array_equal(got, pk), k
        agree = pk == pc
        assert np.array_equal(got[agree], g[k + "_packed"].reshape(-1)[agree]), k


# ----------------------------------------------------------------------------- FP8 / INT8 ------

@pytest.mark.parametrize("T", TS)
def test_q8_golden(ops, T):
    g = load("q8")
    x = to_f32(g[f"{T}_x"], T)
    xt = tensor_from_f32(x, T)
    for name, fn in (("fp8", ops.fp8_quantize), ("int8", ops.int8_quantize)):
        for tag, (outer, axis, inner) in (("t", (1, 1, x.size)), ("a0", (1, 16, 96)), ("blk", (1, 48, 32))):
            s = tensor_from_f32(to_f32(g[f"{T}_{name}_{tag}_s"], T), T)
            q = fn(xt, s, outer, axis, inner)
            assert np.array_equal(q.view(torch.uint8).cpu().numpy().reshape(-1),
                                  g[f"{T}_{name}_{tag}_q"].view(np.uint8).reshape(-1)), (name, tag)


# ----------------------------------------------------------------------------- histogram -------

@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("nbins", [128, 2048, 5000, 20000])
def test_hist_collect_vs_oracle(ops, T, nbins):
    x = rnd((1 << 20,), T, nbins, 1.0, heavy=True)
    xt = tensor_from_f32(x, T)
    rmax = float(np.abs(x).max()) * 0.7  # some samples fall outside and are dropped
    counts = torch.zeros(nbins, dtype=torch.int64, device="cuda")
    ops.hist_collect(xt, counts, nbins, rmax)
    want = qo.hist_bins(x, nbins, rmax)
    assert np.array_equal(counts.cpu().numpy(), want)
    ops.hist_collect(xt, counts, nbins, rmax)  # accumulates
    assert np.array_equal(counts.cpu().numpy(), 2 * want)


@pytest.mark.parametrize("nbins", [2048, 1500, 30000, 120000])
def test_hist_bin_edges_and_specials(ops, nbins):
    """Samples on and one ulp around every bin edge, the range end, NaN, inf and every finite bf16
    value: the bracketed bin index must fall back to the exact division wherever it matters."""
    rng = np.random.default_rng(nbins)
    for rmax in (np.float32(1.0), np.float32(7.3125), np.float32(rng.uniform(0.01, 300.0)), np.float32(3.0e-3)):
        k = np.arange(nbins + 2, dtype=np.float64)
        edges = (k * float(rmax) / nbins).astype(np.float32)
        x = np.concatenate([edges, np.nextafter(edges, np.float32(0)), np.nextafter(edges, np.float32(1e30)),
                            -edges, np.float32([rmax, -rmax, np.nan, np.inf, -np.inf, 0.0, -0.0, 1e-45, 1e38]),
                            rng.uniform(0, float(rmax), 100003).astype(np.float32)])
        counts = torch.zeros(nbins, dtype=torch.int64, device="cuda")
        ops.hist_collect(tensor_from_f32(x, "f32"), counts, nbins, float(rmax))
        assert np.array_equal(counts.cpu().numpy(), qo.hist_bins(x, nbins, rmax)), float(rmax)
    pat = np.arange(65536, dtype=np.uint32)
    vals = (pat << 16).view(np.float32)
    h16 = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    for rmax in (np.float32(2.0), np.float32(448.0), np.float32(rng.uniform(0.5, 50.0)), np.float32(1e-3),
                 np.float32(7e4), np.float32(3e30)):
        for T, v in (("bf16", vals), ("f16", h16)):
            v = np.concatenate([v, v[: 12345]])  # a ragged length and repeated values
            counts = torch.zeros(nbins, dtype=torch.int64, device="cuda")
            ops.hist_collect(tensor_from_f32(v, T), counts, nbins, float(rmax))
            assert np.array_equal(counts.cpu().numpy(), qo.hist_bins(v, nbins, rmax)), (T, float(rmax))


@pytest.mark.parametrize("T", TS)
def test_hist_collect_open_vs_oracle(ops, T):
    """Open-ended collection: later, larger batches land in bins past the first range; what is
    beyond the capacity, NaN and inf are counted apart."""
    nbins, cap = 2048, 2048 * 16
    x0 = rnd((1 << 18,), T, 11, 1.0, heavy=True)
    rmax = float(np.abs(x0).max())
    counts = torch.zeros(cap, dtype=torch.int64, device="cuda")
    over = torch.zeros(1, dtype=torch.int64, device="cuda")
    want = np.zeros(cap, np.int64)
    beyond = 0
    for i, scale in enumerate((1.0, 3.0, 12.0, 40.0)):
        x = rnd((1 << 18,) if i else x0.shape, T, 11 + i, scale, heavy=True) if i else x0
        x = x.copy()
        x[5] = np.nan; x[77] = np.inf; x[78] = -np.inf
        ops.hist_collect_open(tensor_from_f32(x, T), counts, nbins, rmax, over)
        w, b = qo.hist_bins_open(x, nbins, np.float32(rmax), cap)
        want += w; beyond += b
        assert np.array_equal(counts.cpu().numpy(), want), scale
        assert int(over) == beyond
    assert beyond > 3 * 4 and want[nbins:].sum() > 0


def test_hist_golden_and_percentile(ops):
    g = load("hist")
    x = to_f32(g["x0"], "bf16")
    counts = torch.zeros(2048, dtype=torch.int64, device="cuda")
    rmax = float(np.abs(x).max())
    ops.hist_collect(tensor_from_f32(x, "bf16"), counts, 2048, rmax)
    ref = g["hist0"]
    got = counts.cpu().numpy()
    assert got.sum() == ref.sum()
    assert np.abs(got - ref).sum() <= 2e-3 * ref.sum()
    for p in (99.0, 99.9, 99.99, 100.0):
        want, _ = qo.percentile_amax(got, g["edges0"], p)
        a = ops.hist_percentile(counts, 2048, torch.from_numpy(g["edges0"]), 0.0, p)
        assert a.item() == want


def test_nvfp4_every_bf16_value_under_many_divisors(ops):
    """All finite bf16 bit patterns quantised under 160 per-tensor scales spread over 12 decades:
    the reciprocal-and-correct quotient of the kernel must give the codes of the IEEE division."""
    pat = np.arange(65536, dtype=np.uint32)
    vals = (pat << 16).view(np.float32)
    vals = vals[np.isfinite(vals)]
    rng = np.random.default_rng(123)
    for i in range(160):
        x = rng.permutation(vals)[: (vals.size // 16) * 16].reshape(-1, 16)
        s2 = np.float32(10.0 ** rng.uniform(-8, 4))
        packed, scales, s2o = ops.nvfp4_quantize(tensor_from_f32(x, "bf16"), scale2=torch.tensor(float(s2)))
        wp, ws, _ = qo.nvfp4_quantize(x, 16, s2=s2)
        assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), ws), i
        assert np.array_equal(packed.cpu().numpy(), wp), i


@pytest.mark.parametrize("num_bits,unsigned", [(8, False), (8, True), (4, False)])
def test_hist_entropy_kernel_vs_host_search(ops, num_bits, unsigned):
    """The device KL search against the numpy restatement of the reference's host loop: same
    divergences (fp64 sums in another order) and the same chosen clip point."""
    from b200q.calib.histogram import _entropy_amax

    rng = np.random.default_rng(7 + num_bits)
    for nbins, start, stride in ((2048, 128, 1), (2048, 128, 3), (700, 128, 1), (4600, 256, 7)):
        x = np.abs(rng.standard_normal(400_000)).astype(np.float32)
        x[:50] *= 30.0                                          # outliers: a long, mostly empty tail
        counts, edges = np.histogram(x, bins=nbins, range=(0, float(x.max())))
        c = torch.from_numpy(counts.astype(np.int64)).cuda()
        e = torch.from_numpy(edges.astype(np.float32)).cuda()
        levels = 1 << (num_bits - 1 + int(unsigned))
        amax, divs = ops.hist_entropy(c, nbins, e, levels, start, stride)
        want = _entropy_amax(counts, edges.astype(np.float32), num_bits, unsigned, stride, start)
        assert amax.item() == np.float32(want), (nbins, start, stride)
        assert torch.isfinite(divs).any()


def test_hist_mse_kernel_vs_host_search(ops):
    from b200q.calib.histogram import _mse_amax

    rng = np.random.default_rng(21)
    for nbins, start, stride, bits, unsigned in ((2048, 128, 1, 8, False), (2048, 128, 5, 8, True), (300, 16, 1, 4, False)):
        x = np.abs(rng.standard_normal(300_000)).astype(np.float32)
        x[:20] *= 25.0
        counts, edges = np.histogram(x, bins=nbins, range=(0, float(x.max())))
        edges = edges.astype(np.float32)
        bound = 2.0 ** (bits - 1 + int(unsigned)) - 1
        amax, errs = ops.hist_mse(torch.from_numpy(counts.astype(np.int64)).cuda(), nbins,
                                  torch.from_numpy(edges).cuda(), bound, start, stride)
        want = _mse_amax(counts, edges, bits, unsigned, stride, start)
        assert abs(amax.item() - want) <= 1e-6 * want, (nbins, amax.item(), want)
        assert torch.isfinite(errs).all()


def test_back_to_back_dependent_launches_keep_stream_order(ops):
    """The kernels overlap their launch with the previous kernel's tail; a kernel must still see
    everything its predecessor wrote.  Chains of dependent launches (abs-max -> fake quant that
    reads it -> abs-max of the result -> histogram of the result) with nothing in between, many
    times over, against results computed step by step with synchronisation in between."""
    torch.manual_seed(11)
    xs = [(torch.randn(1 << 20, device="cuda") * (1 + i)).bfloat16() for i in range(6)]
    want = []
    for x in xs:                                   # reference: every step synchronised
        a = ops.amax_tensor(x); torch.cuda.synchronize()
        y = ops.fake_e4m3(x, a); torch.cuda.synchronize()
        b = ops.amax_tensor(y); torch.cuda.synchronize()
        z = ops.nvfp4_fake(y, b); torch.cuda.synchronize()
        c = torch.zeros(2048, dtype=torch.int64, device="cuda")
        ops.hist_collect(z, c, 2048, float(b)); torch.cuda.synchronize()
        want.append((a.clone(), y.clone(), b.clone(), z.clone(), c.clone()))
    for rep in range(20):                          # the same chains, enqueued without any host wait
        got = []
        rmax = [float(w[2]) for w in want]
        for x, r in zip(xs, rmax):
            a = ops.amax_tensor(x)
            y = ops.fake_e4m3(x, a)
            b = ops.amax_tensor(y)
            z = ops.nvfp4_fake(y, b)
            c = torch.zeros(2048, dtype=torch.int64, device="cuda")
            ops.hist_collect(z, c, 2048, r)
            got.append((a, y, b, z, c))
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            for u, v in zip(g, w):
                assert torch.equal(u, v), rep


def test_plain_c_host_program_through_the_c_abi(tmp_path):
    """tests/c/cabi_host.c: a C program (gcc, CUDA runtime, no Python objects) quantises through the
    shared library and checks the result and the status codes itself."""
    import os
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    lib_dir = root / "tensorrt-model-optimizer_b200" / "b200q" / "_lib"
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    exe = tmp_path / "cabi_host"
    subprocess.run(["gcc", "-std=c99", "-O1", str(root / "tests" / "c" / "cabi_host.c"), "-I", str(root / "include"),
                    "-I", str(cuda / "include"), "-L", str(lib_dir), "-lb200q", "-L", str(cuda / "lib64"), "-lcudart",
                    "-lm", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda / 'lib64'}", "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "cabi_host ok" in r.stdout


def test_tensors_beyond_2_31_elements(ops):
    """64-bit indexing: one bf16 tensor of 2^31 + 2^20 elements (4.3 GB) through the abs-max, NVFP4
    quantise / dequantise and histogram kernels, checked by size-independent properties."""
    n = (1 << 31) + (1 << 20)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    step = 1 << 28
    for i in range(0, n, step):
        m = min(step, n - i)
        x[i:i + m] = (torch.randn(m, generator=g, device="cuda") * 0.02).bfloat16()
    x[-1] = 3.0                                  # the maximum sits in the very last element
    x[(1 << 31) + 5] = -2.5
    amax = ops.amax_tensor(x)
    assert float(amax) == 3.0
    xv = x.view(-1, 4096)
    packed, scales, s2 = ops.nvfp4_quantize(xv, amax=amax)
    assert float(s2) == float(torch.tensor(3.0) / torch.tensor(2688.0))
    deq = ops.nvfp4_dequantize(packed, scales, s2, torch.bfloat16)
    assert deq.shape == xv.shape
    assert float(deq.view(-1)[-1]) == 3.0 and abs(float(deq.view(-1)[(1 << 31) + 5]) + 2.5) < 0.1
    # slices at the start, across the 2^31 boundary and at the very end against the oracle
    for lo in (0, (1 << 31) - (1 << 15), n - (1 << 16)):
        sl = slice(lo, lo + (1 << 16))
        xs = f32_from_tensor(x[sl]).reshape(-1, 4096)
        wp, ws, _ = qo.nvfp4_quantize(xs, 16, amax=np.float32(3.0))
        assert np.array_equal(packed.view(-1)[lo // 2: lo // 2 + (1 << 15)].cpu().numpy(), wp.reshape(-1)), lo
        assert np.array_equal(scales.view(torch.uint8).view(-1)[lo // 16: lo // 16 + (1 << 12)].cpu().numpy(),
                              ws.reshape(-1)), lo
        want = qo.nvfp4_dequantize(wp, ws, np.float32(3.0) / np.float32(2688.0), 16, "bf16")
        assert same_bits(f32_from_tensor(deq.view(-1)[sl]), want.reshape(-1)), lo
    del packed, scales
    # every element lands in exactly one bin
    counts = torch.zeros(2048, dtype=torch.int64, device="cuda")
    ops.hist_collect(deq.view(-1), counts, 2048, 3.0)
    assert int(counts.sum()) == n and int(counts[-1]) >= 1


def test_kernels_capture_into_a_cuda_graph(ops):
    """A chain of dependent launches captured once and replayed on new data in the same buffers."""
    x = torch.zeros(1 << 20, dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros((), device="cuda")
    ops.amax_tensor(x, out=amax); ops.nvfp4_fake(x, amax)          # load everything before capture
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            amax.zero_()
            ops.amax_tensor(x, out=amax)
            y = ops.fake_e4m3(x, amax)
            z = ops.nvfp4_fake(y, amax)
    torch.cuda.current_stream().wait_stream(s)
    for i in range(3):
        new = (torch.randn(1 << 20, device="cuda") * (i + 1)).bfloat16()
        x.copy_(new)
        graph.replay()
        torch.cuda.synchronize()
        a = ops.amax_tensor(new)
        want = ops.nvfp4_fake(ops.fake_e4m3(new, a), a)
        assert torch.equal(amax, a) and torch.equal(z, want), i


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("n", [2, 16, 32, 64, 128, 512, 1024, 4096])
def test_hadamard_transform(ops, T, n):
    """Against the Sylvester matrix: exact for small-integer inputs (every sum and the 1/sqrt(n)
    scaling for n a power of 4 are exact in T), within rounding for random inputs; H(H(x)) = n x."""
    import scipy.linalg

    H = scipy.linalg.hadamard(n).astype(np.float64)
    rng = np.random.default_rng(n)
    xi = rng.integers(-1, 2, (37, n)).astype(np.float32)           # entries in {-1, 0, 1}
    yi = f32_from_tensor(ops.hadamard(tensor_from_f32(xi, T), 1.0))
    want = xi.astype(np.float64) @ H
    exact = np.abs(want).max() <= (256 if T == "bf16" else 2048)   # sums representable in T
    if exact:
        assert np.array_equal(yi, want.astype(np.float32))
        back = f32_from_tensor(ops.hadamard(tensor_from_f32(yi, T), 1.0 / n))
        assert np.array_equal(back, xi)
    x = rnd((64, n), T, n + 1)
    y = f32_from_tensor(ops.hadamard(tensor_from_f32(x, T), 1.0 / np.sqrt(n)))
    want = qo.round_to((qo.round_to((x.astype(np.float64) @ H).astype(np.float32), T) * np.float32(1.0 / np.sqrt(n))
                        ).astype(np.float32), T)
    tol = {"f32": 1e-5, "f16": 2e-3, "bf16": 1.6e-2}[T]
    assert np.allclose(y, want, rtol=tol, atol=tol * np.abs(want).max())
    if T != "f32":   # 16-bit outputs: the rounding to T hides the order of the fp32 sums almost everywhere
        assert np.mean(y != want) < 0.05


def test_rotating_quantizer(ops):
    import b200q as mtq

    x = tensor_from_f32(rnd((4, 8, 128), "bf16", 3), "bf16")
    q = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(enable=False, rotate=True)).cuda()
    assert torch.equal(q(x), ops.hadamard(x, 1.0 / 128 ** 0.5))     # a disabled quantiser still rotates
    k = mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(
        num_bits=(2, 1), block_sizes={-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, axis=None, rotate=True)).cuda()
    r = ops.hadamard(x, 1.0 / 128 ** 0.5)
    assert torch.equal(k(x), ops.nvfp4_fake(r, r.abs().amax().float()))
    xg = x.float().requires_grad_(True)
    q(xg).sum().backward()
    assert torch.allclose(xg.grad, ops.hadamard(torch.ones_like(xg), 1.0 / 128 ** 0.5))


@pytest.mark.parametrize(("block_sizes", "rows", "expected"), [
    ({-1: 2, -2: 2}, 2, [[5.0, 7.0]]),
    ({-1: 4, -2: 2}, 4, [[7.0], [15.0]]),
    ({-2: 4}, 4, [[12.0, 13.0, 14.0, 15.0]])])
def test_reduce_block_amax_over_several_dimensions_like_the_reference_test(block_sizes, rows, expected):
    """Reference tests/unit/torch/quantization/test_utils.py:26-59 (its comparison is not asserted there; the
    values are what its ``reduce_block_amax`` returns: one dimension after the other)."""
    from b200q.utils import reduce_block_amax

    x = torch.arange(rows * 4, dtype=torch.bfloat16, device="cuda").reshape(rows, 4)
    got = reduce_block_amax(x, block_sizes)
    want = torch.tensor(expected, dtype=torch.bfloat16, device="cuda")
    assert got.dtype == torch.bfloat16 and got.shape == want.shape and torch.equal(got, want)
