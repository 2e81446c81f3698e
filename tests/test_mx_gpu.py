"""MX (E8M0-scaled) format kernels against the oracle, the reference's known-answer tables and the
MXFP4QTensor golden vectors."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from _util import f32_from_tensor, load, same_bits, same_values, tensor_from_f32, to_f32

pytestmark = pytest.mark.gpu
TS = ("f32", "f16", "bf16")
FMT_BITS = {"e2m1": (2, 1), "e3m2": (3, 2), "e2m3": (2, 3), "e4m3": (4, 3), "e5m2": (5, 2), "int8": 8}


@pytest.fixture(scope="module")
def ops():
    from b200q import ops as _ops

    return _ops


def rnd(shape, T, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape).astype(np.float32) / np.sqrt(rng.chisquare(4, shape) / 4).astype(np.float32)
    return qo.round_to((x * np.float32(scale)).astype(np.float32), T)


@pytest.mark.parametrize("fmt", list(FMT_BITS))
def test_mx_fake_known_answers(ops, fmt):
    g = load("mx_known_answers")
    x, want, block = g[fmt + "_in"], g[fmt + "_out"], int(g[fmt + "_block"])
    rng = np.random.default_rng(5)
    sign = (rng.integers(0, 2, x.shape) * 2 - 1).astype(np.float32)
    y = f32_from_tensor(ops.mx_fake(tensor_from_f32(x * sign, "f32"), block, FMT_BITS[fmt]))
    assert np.allclose(y, want * sign, rtol=1e-5, atol=1e-8 if fmt == "e2m1" else 1e-3)
    assert same_values(y, qo.mx_fake(x * sign, block, fmt))


@pytest.mark.parametrize("T", TS)
@pytest.mark.parametrize("fmt", list(FMT_BITS))
@pytest.mark.parametrize("block", [8, 16, 32])
def test_mx_fake_vs_oracle(ops, T, fmt, block):
    for i, (shape, scale) in enumerate([((64, 256), 1.0), ((7, 3, 96), 300.0), ((33, 64), 1e-4)]):
        x = rnd(shape, T, 31 * block + i, scale)
        x.reshape(-1)[:block] = 0  # one all-zero block
        y = f32_from_tensor(ops.mx_fake(tensor_from_f32(x, T), block, FMT_BITS[fmt]))
        assert same_values(y, qo.mx_fake(x, block, fmt, T)), (shape, scale)


def test_mx_fake_ragged_last_dim_and_large(ops):
    x = rnd((5, 50), "bf16", 3)
    y = f32_from_tensor(ops.mx_fake(tensor_from_f32(x, "bf16"), 32, (4, 3)))
    assert y.shape == x.shape and same_values(y, qo.mx_fake(x, 32, "e4m3", "bf16"))
    x = rnd((2048, 4096), "bf16", 4)
    y = f32_from_tensor(ops.mx_fake(tensor_from_f32(x, "bf16"), 32, (2, 1)))
    assert same_values(y, qo.mx_fake(x, 32, "e2m1", "bf16"))
    # idempotent: quantised values are fixed points of the same block scale
    y2 = f32_from_tensor(ops.mx_fake(tensor_from_f32(y, "bf16"), 32, (2, 1)))
    assert same_values(y2, y)


@pytest.mark.parametrize("T", TS)
def test_mxfp4_quantize_golden(ops, T):
    from b200q.qtensor import MXFP4QTensor

    g = load("mxfp4")
    for j in range(3):
        k = f"{T}_{j}"
        x, block = to_f32(g[k + "_x"], T), int(g[k + "_block"])
        q, s = MXFP4QTensor.quantize(tensor_from_f32(x, T), block)
        assert np.array_equal(q._quantized_data.cpu().numpy(), g[k + "_packed"]), k
        assert np.array_equal(s.cpu().numpy(), g[k + "_scales"]), k
        deq = q.dequantize(scale=s, block_sizes={-1: block})
        assert deq.dtype == tensor_from_f32(x, T).dtype
        assert same_bits(f32_from_tensor(deq), to_f32(g[k + "_deq"], T)), k


@pytest.mark.parametrize("T", TS)
def test_mxfp4_quantize_vs_oracle_large(ops, T):
    x = rnd((1024, 2048), T, 77, 0.3)
    packed, scales = ops.mxfp4_quantize(tensor_from_f32(x, T), 32)
    p, s = qo.mxfp4_quantize(x, 32)
    assert np.array_equal(packed.cpu().numpy(), p) and np.array_equal(scales.cpu().numpy(), s)


def test_mx_configs_through_quantizer_and_compress(ops):
    import b200q as mtq
    from b200q.nn import TensorQuantizer
    from b200q.qtensor import MXFP4QTensor

    x = tensor_from_f32(rnd((16, 128), "bf16", 9), "bf16")
    for cfg, fmt in ((mtq.MXFP8_DEFAULT_CFG, "e4m3"), (mtq.MXFP6_DEFAULT_CFG, "e3m2"),
                     (mtq.MXFP4_DEFAULT_CFG, "e2m1"), (mtq.MXINT8_DEFAULT_CFG, "int8")):
        q = TensorQuantizer(dict(cfg["quant_cfg"]["*weight_quantizer"]))
        y = q(x)
        assert same_values(f32_from_tensor(y), qo.mx_fake(f32_from_tensor(x), 32, fmt, "bf16")), fmt
    lin = torch.nn.Linear(128, 64, bias=False, device="cuda", dtype=torch.bfloat16)
    w = lin.weight.detach().clone()
    model = torch.nn.Sequential(lin)
    mtq.quantize(model, mtq.MXFP4_DEFAULT_CFG, lambda m: m(x))
    out_fake = model(x)
    mtq.compress(model)
    inner = model[0].weight.get_qtensor()
    assert isinstance(inner, MXFP4QTensor)
    p, s = qo.mxfp4_quantize(f32_from_tensor(w), 32)
    assert np.array_equal(inner._quantized_data.cpu().numpy(), p)
    assert np.array_equal(model[0].weight_quantizer._scale.cpu().numpy(), s)
    out_real = model(x)
    # the packed weight follows MXFP4QTensor's rule (ties toward zero), not the fake kernel's RNE:
    # compare the real-quant forward with a matmul on the oracle's dequantised weight
    wd = tensor_from_f32(qo.mxfp4_dequantize(p, s, 32, "bf16"), "bf16")
    assert torch.allclose(out_real.float(), (model[0].input_quantizer(x) @ wd.T).float(), rtol=1e-2, atol=1e-2)
    assert (out_fake.float() - out_real.float()).abs().mean() < 0.05 * out_real.float().abs().mean()
