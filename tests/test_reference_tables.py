"""Known answers held by the reference's own GPU tests (tests/golden/reference_test_tables.npz, taken
from the test sources as data): the oracle on CPU, the kernels and the TensorQuantizer on the GPU."""
import numpy as np
import pytest

from oracle import quant_oracle as qo
from _util import f32_from_tensor, load, same_bits, tensor_from_f32, to_f32

TS = ("f32", "f16", "bf16")


def _expand(scales, shape, blocks):
    """Per-block values [ceil(shape/blocks)] -> one value per element of `shape`."""
    out = scales
    for ax, b in enumerate(blocks):
        out = np.repeat(out, b, axis=ax)
    return out[tuple(slice(0, n) for n in shape)]


def _block_amax(x, blocks):
    """abs-max over blocks of size `blocks` (one entry per dim; ragged edges padded with zeros)."""
    pad = [(0, (-n) % b) for n, b in zip(x.shape, blocks)]
    xp = np.pad(np.abs(x), pad)
    shp = []
    for n, b in zip(xp.shape, blocks):
        shp += [n // b, b]
    return xp.reshape(shp).max(axis=tuple(range(1, 2 * x.ndim, 2)))


def _row(g, i):
    nb = g[f"acc{i}_num_bits"]
    num_bits = int(nb) if nb.ndim == 0 else tuple(int(v) for v in nb)
    blocks = {int(k): int(v) for k, v in g[f"acc{i}_blocks"]}
    axis = int(g[f"acc{i}_axis"])
    return num_bits, blocks, (None if axis == -99 else axis), to_f32(g[f"acc{i}_x"], "bf16"), to_f32(g[f"acc{i}_y"], "bf16")


def test_oracle_real_quant_rows_of_the_reference_tests():
    g = load("reference_test_tables")
    assert int(g["acc_count"]) == 9
    for i in range(9):
        num_bits, blocks, axis, x, want = _row(g, i)
        if num_bits == 4:   # INT4QTensor: blocks along the last dim, CPU flavour of the reference
            b = blocks[-1]
            xp = qo.pad_last(x, b)
            packed, scales = qo.int4_quantize(xp.reshape(-1), b, "bf16", flavour="cpu")
            y = qo.int4_dequantize(packed, scales, b, "bf16").reshape(xp.shape)[..., : x.shape[-1]]
        else:
            if blocks:
                bl = [blocks.get(d - x.ndim, 1) for d in range(x.ndim)]
                amax = _expand(_block_amax(x, bl), x.shape, bl)
            elif axis is not None:
                amax = np.abs(x).max(axis=tuple(d for d in range(x.ndim) if d != axis), keepdims=True) + 0 * x
            else:
                amax = np.full_like(x, np.abs(x).max())
            bound = 448.0 if num_bits == (4, 3) else 127.0
            scales = qo.round_to((amax / np.float32(bound)).astype(np.float32), "bf16")
            if num_bits == (4, 3):
                q = qo.e4m3_decode(qo.fp8_quantize(x, scales, "bf16"))
            else:
                q = qo.int8_quantize(x, scales, "bf16").astype(np.float32)
            y = qo.round_to((q * scales).astype(np.float32), "bf16")
        assert np.allclose(y, want, rtol=1e-5, atol=1e-8), (i, y, want)


def test_oracle_fp4_tables_of_the_reference_tests():
    g = load("reference_test_tables")
    for i in range(int(g["cast_count"])):
        assert np.array_equal(qo.e2m1_encode(g[f"cast{i}_x"]), g[f"cast{i}_codes"]), i
    for i in range(int(g["nvq_count"])):
        for T in TS:
            k = f"nvq{i}_{T}_"
            x = to_f32(g[k + "x"], T)
            packed, scales, s2 = qo.nvfp4_quantize(x, 8)
            assert np.array_equal(packed, g[k + "packed"]) and np.array_equal(scales, g[k + "scales"]), k
            assert same_bits(np.float32([s2]), g[k + "scale2"]), k
    rng = np.random.default_rng(0)
    for i in range(4):
        sign = (rng.integers(0, 2, (1, 8)) * 2 - 1).astype(np.float32)
        for T in TS:
            x = qo.round_to(np.tile(g[f"fp4fake{i}_x"] * sign, (1, 2)), T)
            y = qo.nvfp4_fake(x, np.abs(x).max(), 16, T)
            want = qo.round_to(np.tile(g[f"fp4fake{i}_y"] * sign, (1, 2)), T)
            assert np.allclose(y, want, rtol=1e-5, atol=1e-8), (i, T)


@pytest.mark.gpu
def test_tensor_quantizer_real_quant_rows_of_the_reference_tests():
    import b200q as mtq
    from b200q.nn import TensorQuantizer

    g = load("reference_test_tables")
    for i in range(9):
        num_bits, blocks, axis, x, want = _row(g, i)
        cfg = mtq.QuantizerAttributeConfig(num_bits=num_bits, block_sizes=blocks or None, fake_quant=False, axis=axis)
        q = TensorQuantizer(cfg).cuda()
        xt = tensor_from_f32(x, "bf16")
        deq = q(q(xt))
        assert deq.shape == xt.shape
        assert np.allclose(f32_from_tensor(deq), want, rtol=1e-5, atol=1e-8), (i, f32_from_tensor(deq), want)
        fq = TensorQuantizer(mtq.QuantizerAttributeConfig(num_bits=num_bits, block_sizes=blocks or None,
                                                          fake_quant=True, axis=axis)).cuda()
        assert np.allclose(f32_from_tensor(fq(xt)), f32_from_tensor(deq), rtol=1e-1, atol=1e-1), i


@pytest.mark.gpu
def test_nvfp4_tables_of_the_reference_tests_on_gpu():
    import torch

    from b200q.qtensor import NVFP4QTensor
    from b200q.tensor_quant import dynamic_block_quant

    g = load("reference_test_tables")
    for i in range(int(g["nvq_count"])):
        for T in TS:
            k = f"nvq{i}_{T}_"
            q, s, s2 = NVFP4QTensor.quantize(tensor_from_f32(to_f32(g[k + "x"], T), T), 8)
            assert np.array_equal(q._quantized_data.cpu().numpy(), g[k + "packed"]), k
            assert np.array_equal(s.view(torch.uint8).cpu().numpy(), g[k + "scales"]), k
            assert same_bits(s2.float().cpu().numpy().reshape(1), g[k + "scale2"]), k
    rng = np.random.default_rng(0)
    for i in range(4):
        sign = (rng.integers(0, 2, (1, 8)) * 2 - 1).astype(np.float32)
        for T in TS:
            x = qo.round_to(np.tile(g[f"fp4fake{i}_x"] * sign, (1, 2)), T)
            xt = tensor_from_f32(x, T)
            y = dynamic_block_quant(xt, 16, xt.abs().amax().float(), None, (2, 1), (4, 3))
            want = qo.round_to(np.tile(g[f"fp4fake{i}_y"] * sign, (1, 2)), T)
            assert np.allclose(f32_from_tensor(y), want, rtol=1e-5, atol=1e-8), (i, T)
