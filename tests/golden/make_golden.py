"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself on CPU.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py --ref /path/to/TensorRT-Model-Optimizer

The reference is imported unmodified with three shims (it cannot be pip-installed offline):
its distribution version is supplied, the optional ``pulp`` / ``torchprofile`` imports are
stubbed, and ``fp4_compatible`` is forced False so that NVFP4QTensor.quantize does not probe for
a GPU.  Inputs are seeded; every file stores inputs and the reference outputs as raw bit
patterns (uint16 for half/bf16, uint8 for fp8) so that nothing is lost in storage.
"""
from __future__ import annotations

import argparse
import importlib.metadata as md
import sys
import types
import warnings
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def import_reference(ref_root: str):
    real_version = md.version

    def version(name):
        return "0.40.0" if name == "nvidia-modelopt" else real_version(name)

    md.version = version

    class _Stub(types.ModuleType):
        def __getattr__(self, k):
            if k.startswith("__"):
                raise AttributeError(k)
            return type(k, (), {})

    for m in ("pulp", "torchprofile", "torchprofile.profile"):
        sys.modules.setdefault(m, _Stub(m))
    sys.path.insert(0, ref_root)
    warnings.filterwarnings("ignore")
    import modelopt.torch.quantization as mtq  # noqa: F401
    import modelopt.torch.quantization.qtensor.nvfp4_tensor as nv

    nv.fp4_compatible = lambda: False
    return mtq


TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as a numpy integer array."""
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def gen(shape, T, seed, scale=1.0, heavy=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if heavy:  # Student-t(4) like weights with outliers
        chi = torch.randn((4, *shape), generator=g).pow(2).sum(0) / 4
        x = x / chi.sqrt()
    return (x * scale).to(TD[T])


def golden_fake_int(out):
    from modelopt.torch.quantization.tensor_quant import fake_tensor_quant
    from modelopt.torch.quantization.utils import reduce_amax

    cases = {}
    i = 0
    for T in ("f32", "f16", "bf16"):
        for bits_ in (3, 4, 5, 7, 8, 11):
            for unsigned in (False, True):
                for narrow in (True, False):
                    x = gen((6, 32), T, 100 + i, scale=0.7)
                    if unsigned:
                        x = x.abs()
                    for axis in (None, 0, 1):
                        if axis is None:
                            amax = reduce_amax(x) * 0.8
                        else:
                            red = [d for d in range(2) if d != axis]
                            amax = reduce_amax(x, axis=red) * 0.8
                        y = fake_tensor_quant(x, amax.float(), None, bits_, unsigned, narrow)
                        k = f"{T}_b{bits_}_u{int(unsigned)}_n{int(narrow)}_a{axis}"
                        cases[k + "_x"] = bits(x)
                        cases[k + "_amax"] = bits(amax.float())
                        cases[k + "_y"] = bits(y)
                    i += 1
    # tiny amax -> zeros (epsilon rule), per-channel amax with one dead channel
    x = gen((8, 32), "f32", 7)
    amax = torch.full((8, 1), 0.5)
    amax[3] = 1e-9
    cases["tiny_x"] = bits(x)
    cases["tiny_amax"] = bits(amax)
    cases["tiny_y"] = bits(fake_tensor_quant(x, amax, None, 8, False, True))
    np.savez_compressed(out / "fake_int.npz", **cases)


def golden_fake_e4m3(out):
    from modelopt.torch.quantization.tensor_quant import scaled_e4m3
    from modelopt.torch.quantization.utils import reduce_amax

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        x = gen((32, 128), T, 200 + i, scale=3.0)
        amax = reduce_amax(x)  # in range: the eager cast equals the saturating kernel here
        cases[f"{T}_x"] = bits(x)
        cases[f"{T}_amax"] = bits(amax.float())
        cases[f"{T}_y"] = bits(scaled_e4m3(x, amax, None, 4, 3))
        cases[f"{T}_y_noamax"] = bits(scaled_e4m3(x, None, None, 4, 3))
        for axis in (0, 1):
            am = reduce_amax(x, axis=[1 - axis])
            cases[f"{T}_amax_a{axis}"] = bits(am.float())
            cases[f"{T}_y_a{axis}"] = bits(scaled_e4m3(x, am, None, 4, 3))
    np.savez_compressed(out / "fake_e4m3.npz", **cases)


def golden_nvfp4(out):
    from modelopt.torch.quantization.qtensor import NVFP4QTensor

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        for j, (shape, sc, heavy) in enumerate([((16, 64), 0.02, True), ((8, 48), 1.0, False),
                                                ((4, 40), 5.0, False)]):
            x = gen(shape, T, 300 + 10 * i + j, scale=sc, heavy=heavy)
            if j == 1:
                x[0, :16] = 0  # an all-zero block
                x[1, 3] = -0.0
            q, s, s2 = NVFP4QTensor.quantize(x.clone(), 16)
            k = f"{T}_{j}"
            cases[k + "_x"] = bits(x)
            cases[k + "_packed"] = bits(q._quantized_data)
            cases[k + "_scales"] = bits(s)
            cases[k + "_s2"] = bits(s2.reshape(1))
            if shape[-1] % 16 == 0:  # the reference's dequantize cannot undo its own padding
                d = q.dequantize(scale=s, double_scale=s2, block_sizes={-1: 16})
                cases[k + "_deq"] = bits(d)
            # externally supplied (clipped) amax: block scales may overflow the E4M3 cast
            s2c = NVFP4QTensor.get_weights_scaling_factor_2(x) * 0.5
            q2, sb2, _ = NVFP4QTensor.quantize(x.clone(), 16, weights_scaling_factor_2=s2c)
            cases[k + "_clip_s2"] = bits(s2c.reshape(1))
            cases[k + "_clip_packed"] = bits(q2._quantized_data)
            cases[k + "_clip_scales"] = bits(sb2)
    # _cast_fp4 at and around every rounding boundary, both signs
    pts = []
    for b in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.0, 0.5, 1, 1.5, 2, 3, 4, 6, 7.5, 100.0):
        for d in (0.0, 1e-3, -1e-3, 6e-8, -6e-8):
            pts += [b + d, -(b + d)]
    v = torch.tensor(pts + [float("nan"), float("inf"), -float("inf"), -0.0, -1e-30, 1e-30],
                     dtype=torch.float32)
    cases["cast_v"] = bits(v)
    cases["cast_code"] = bits(NVFP4QTensor._cast_fp4(v.clone()))
    np.savez_compressed(out / "nvfp4.npz", **cases)


def golden_int4(out):
    from modelopt.torch.quantization.qtensor import INT4QTensor

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        for j, (shape, block) in enumerate([((8, 256), 128), ((6, 40), 16), ((2, 24), 32)]):
            x = gen(shape, T, 400 + 10 * i + j, scale=0.05)
            q, s = INT4QTensor.quantize(x, block)  # CPU branch of the reference
            k = f"{T}_{j}"
            cases[k + "_x"] = bits(x)
            cases[k + "_block"] = np.array(block)
            cases[k + "_packed"] = bits(q._quantized_data)
            cases[k + "_scales"] = bits(s)
            cases[k + "_deq"] = bits(q.dequantize(scale=s, block_sizes={-1: block}))
    np.savez_compressed(out / "int4.npz", **cases)


def golden_q8(out):
    from modelopt.torch.quantization.qtensor import FP8QTensor, INT8QTensor

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        x = gen((16, 96), T, 500 + i, scale=2.0)
        cases[f"{T}_x"] = bits(x)
        for name, cls in (("fp8", FP8QTensor), ("int8", INT8QTensor)):
            for tag, kw in (("t", {}), ("a0", {"axis": 0}), ("blk", {"block_sizes": {-1: 32}})):
                q, s = cls.quantize(x, **kw)
                cases[f"{T}_{name}_{tag}_q"] = bits(q._quantized_data)
                cases[f"{T}_{name}_{tag}_s"] = bits(s.reshape(-1))
    np.savez_compressed(out / "q8.npz", **cases)


def golden_amax(out):
    from modelopt.torch.quantization.calib import MaxCalibrator
    from modelopt.torch.quantization.utils import reduce_amax, reduce_block_amax

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        x = gen((4, 12, 64), T, 600 + i)
        cases[f"{T}_x"] = bits(x)
        cases[f"{T}_all"] = bits(reduce_amax(x).reshape(1))
        for axis in (0, 1, 2, -1):
            red = [d for d in range(3) if d != axis % 3]
            cases[f"{T}_ax{axis}"] = bits(reduce_amax(x, axis=red).reshape(-1))
        for blk in (16, 32):
            cases[f"{T}_blk{blk}"] = bits(reduce_block_amax(x, {-1: blk}).reshape(-1))
        cal = MaxCalibrator(8, 1, False)
        for b in range(3):
            cal.collect(gen((4, 12, 64), T, 650 + 3 * i + b, scale=1.0 + b))
        cases[f"{T}_cal_ax1"] = bits(cal.compute_amax().reshape(-1))
    np.savez_compressed(out / "amax.npz", **cases)


def golden_hist(out):
    from modelopt.torch.quantization.calib import HistogramCalibrator

    cases = {}
    cal = HistogramCalibrator(8, None, False, num_bins=2048)
    for b in range(3):
        x = gen((64, 512), "bf16", 700 + b, scale=1.0 + 0.6 * b)
        cases[f"x{b}"] = bits(x)
        cal.collect(x)
        cases[f"hist{b}"] = cal._calib_hist.cpu().numpy().astype(np.int64)
        cases[f"edges{b}"] = cal._calib_bin_edges.cpu().numpy().astype(np.float32)
    for p in (99.0, 99.9, 99.99, 100.0):
        cases[f"pct_{p}"] = np.array(cal.compute_amax("percentile", percentile=p).item(), dtype=np.float32)
    cases["entropy"] = np.array(cal.compute_amax("entropy").item(), dtype=np.float32)
    # the sequence of the reference's own test_torch_hist (tests/unit/torch/quantization/
    # test_calibrator.py:141-181): 19 bins, 15-element batches, the second kind forces growth
    torch.manual_seed(0)
    x_1 = torch.rand(15)
    x_1[0] = 0
    x_2 = torch.rand(15) + 1
    x_2[1] = 0
    small = HistogramCalibrator(8, None, False, num_bins=19, torch_hist=True)
    small.collect(x_1)
    cases["small_x1"], cases["small_x2"] = x_1.numpy().copy(), x_2.numpy().copy()
    cases["small_hist0"] = small._calib_hist.cpu().numpy().astype(np.int64)
    for r in range(3):
        small.collect(x_2)
        small.collect(x_1)
        cases[f"small_hist{r + 1}"] = small._calib_hist.cpu().numpy().astype(np.int64)
        cases[f"small_edges{r + 1}"] = small._calib_bin_edges.cpu().numpy().astype(np.float32)
        cases[f"small_pct{r + 1}"] = np.array(small.compute_amax("percentile", percentile=99.99).item(), np.float32)
    np.savez_compressed(out / "hist.npz", **cases)


def golden_export(out):
    from modelopt.torch.export.quant_utils import (get_scaling_factor_from_weight, pack_int4_in_uint8,
                                                   to_quantized_weight)
    from modelopt.torch.quantization.qtensor import NVFP4QTensor

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        w = gen((64, 256), T, 800 + i, scale=0.05)
        cases[f"{T}_w"] = bits(w)
        s4 = get_scaling_factor_from_weight(w, 128)
        cases[f"{T}_int4_scale"] = bits(s4)
        cases[f"{T}_int4_packed"] = bits(pack_int4_in_uint8(w, s4))
        s8 = get_scaling_factor_from_weight(w, 0)
        cases[f"{T}_int8_scale"] = bits(s8)
        cases[f"{T}_int8_q"] = bits(to_quantized_weight(w, s8, "int8_sq"))
        sf = w.abs().amax().float() / 448.0
        cases[f"{T}_fp8_scale"] = bits(sf.reshape(1))
        cases[f"{T}_fp8_q"] = bits(to_quantized_weight(w, sf, "fp8"))
        wsf2 = NVFP4QTensor.get_weights_scaling_factor_2(w)
        wsf, _ = NVFP4QTensor.get_weights_scaling_factor(w, 16, wsf2)
        cases[f"{T}_nvfp4_wsf"] = bits(wsf)
        cases[f"{T}_nvfp4_wsf2"] = bits(wsf2.reshape(1))
        cases[f"{T}_nvfp4_packed"] = bits(to_quantized_weight(w, wsf, "nvfp4", wsf2, 16))
    np.savez_compressed(out / "export.npz", **cases)


def golden_mxfp4(out):
    from modelopt.torch.quantization.qtensor import MXFP4QTensor

    cases = {}
    for i, T in enumerate(("f32", "f16", "bf16")):
        for j, (shape, block) in enumerate([((8, 128), 32), ((3, 5, 64), 32), ((4, 64), 16)]):
            x = gen(shape, T, 900 + 10 * i + j, scale=(0.02, 1.0, 40.0)[j], heavy=(j == 1))
            if j == 0:
                x[0, :32] = 0          # an all-zero block
                x[1, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]).to(x.dtype)  # ties
                x[1, 8:32] = 0
            q, s = MXFP4QTensor.quantize(x, block)
            k = f"{T}_{j}"
            cases[k + "_x"] = bits(x)
            cases[k + "_block"] = np.array(block)
            cases[k + "_packed"] = bits(q._quantized_data)
            cases[k + "_scales"] = bits(s)
            cases[k + "_deq"] = bits(q.dequantize(scale=s, block_sizes={-1: block}))
    np.savez_compressed(out / "mxfp4.npz", **cases)


def golden_mx_known_answers(out, ref_root):
    """The known-answer tables of the reference's MX tests, read from the test source as data
    (tests/gpu/torch/quantization/test_quantize_mxformats_cuda.py: test_mxfp4, test_mxfp6,
    test_mxfp8, test_mxint8); those tests need a GPU and the compiled extension, their tables
    do not."""
    import ast

    src = (Path(ref_root) / "tests/gpu/torch/quantization/test_quantize_mxformats_cuda.py").read_text()
    plan = {"test_mxfp4": (["e2m1"], 8), "test_mxfp6": (["e3m2", "e2m3"], 16),
            "test_mxfp8": (["e4m3", "e5m2"], 8), "test_mxint8": (["int8"], 8)}
    cases = {}
    for fn in ast.parse(src).body:
        if not isinstance(fn, ast.FunctionDef) or fn.name not in plan:
            continue
        fmts, block = plan[fn.name]
        test_in, outs = None, []
        for node in ast.walk(fn):
            if isinstance(node, ast.Assign) and isinstance(node.targets[0], ast.Name) \
                    and node.targets[0].id in ("test_in", "test_out"):
                table = np.array(ast.literal_eval(node.value.args[0]), dtype=np.float32)
                if node.targets[0].id == "test_in":
                    test_in = table
                else:
                    outs.append((node.lineno, table))
        outs = [t for _, t in sorted(outs, key=lambda p: p[0])]
        assert test_in is not None and len(outs) == len(fmts), fn.name
        for fmt, t in zip(fmts, outs):
            assert t.shape == test_in.shape
            cases[f"{fmt}_in"], cases[f"{fmt}_out"], cases[f"{fmt}_block"] = test_in, t, np.array(block)
    assert len(cases) == 18
    np.savez_compressed(out / "mx_known_answers.npz", **cases)


def golden_bias(out):
    """Affine (bias) quantisation through the reference's TensorQuantizer on CPU: static mean,
    static max_min and dynamic bias, INT8 and FP8, two calibration batches of a 4-D tensor."""
    from modelopt.torch.quantization.config import QuantizerAttributeConfig
    from modelopt.torch.quantization.nn import TensorQuantizer

    cases = {}
    xs = [gen((2, 3, 8, 16), "f32", 1200 + i, scale=1.0 + i) + 0.75 * (i + 1) for i in range(2)]
    for i, x in enumerate(xs):
        cases[f"x{i}"] = bits(x)
    cfgs = {"fp8_mean": dict(num_bits=(4, 3), axis=None, bias={-2: None, -4: None, "type": "static"}),
            "int8_maxmin": dict(num_bits=8, axis=None, bias={-1: None, "type": "static", "method": "max_min"}),
            "int8_dynamic": dict(num_bits=8, axis=None, bias={-2: None, "type": "dynamic"})}
    for tag, kw in cfgs.items():
        q = TensorQuantizer(QuantizerAttributeConfig(**kw))
        q.enable_calib(); q.disable_quant()
        for x in xs:
            q(x)
        q.load_calib_amax()
        if q.bias_type == "static":
            q.load_calib_bias()
            cases[f"{tag}_bias"] = bits(q._bias_value)
        q.enable_quant(); q.disable_calib()
        cases[f"{tag}_amax"] = bits(q._amax.reshape(-1))
        cases[f"{tag}_y"] = bits(q(xs[1]))
    np.savez_compressed(out / "bias.npz", **cases)


def golden_reference_test_tables(out, ref_root):
    """Known answers held by the reference's own GPU tests, taken from their source as data:

    * tests/gpu/torch/quantization/test_qtensor_cuda.py, test_qtensor_accuracy: (num_bits,
      block_sizes, axis, input, dequantised output) rows for INT4 / INT8 / FP8 real quantisation
      (the NF4 rows belong to a format outside this package; the MXFP4 row has no expected output);
    * the same file, test_cast_fp4_equivalence and test_nvfp4_quantize: inputs, with the codes /
      packed bytes / scales produced by the reference's NVFP4QTensor on CPU;
    * tests/gpu/torch/quantization/test_tensor_quant_cuda.py, Testfp4.test_cuda_ext_fp4: the
      E2M1 value and tie tables for NVFP4 fake quantisation (block 16, global amax = max|x|).
    """
    import ast

    from modelopt.torch.quantization.qtensor import NVFP4QTensor

    cases = {}
    src = (Path(ref_root) / "tests/gpu/torch/quantization/test_qtensor_cuda.py").read_text()
    tree = ast.parse(src)

    def params_of(fn_name, first_arg):
        for node in ast.walk(tree):
            if isinstance(node, ast.FunctionDef) and node.name == fn_name:
                for dec in node.decorator_list:
                    if isinstance(dec, ast.Call) and dec.args and \
                            ast.unparse(dec.args[0]).replace("'", '"').startswith(first_arg):
                        return eval(compile(ast.Expression(dec.args[1]), "<ref-test-data>", "eval"), {"torch": torch})
        raise KeyError(fn_name)

    rows = params_of("test_qtensor_accuracy", '("num_bits"')
    n = 0
    for num_bits, block_sizes, axis, x, y in rows:
        if y is None or (block_sizes and "scale_block_sizes" in block_sizes):
            continue
        k = f"acc{n}_"
        cases[k + "num_bits"] = np.array(num_bits)
        cases[k + "blocks"] = np.array(sorted((block_sizes or {}).items()), dtype=np.int64).reshape(-1, 2)
        cases[k + "axis"] = np.array(-99 if axis is None else axis)
        cases[k + "x"] = bits(x)
        cases[k + "y"] = bits(y)
        n += 1
    cases["acc_count"] = np.array(n)

    for i, x in enumerate(params_of("test_cast_fp4_equivalence", '"test_input"')[1:]):   # [0] is randn
        cases[f"cast{i}_x"] = x.numpy().copy()   # the reference casts in place
        cases[f"cast{i}_codes"] = NVFP4QTensor._cast_fp4(x).numpy()
    cases["cast_count"] = np.array(i + 1)

    for i, x in enumerate(params_of("test_nvfp4_quantize", '"test_input"')):
        if x.shape[-1] % 8:
            x = torch.nn.functional.pad(x, (0, 8 - x.shape[-1] % 8))        # the reference pads to the block
        for T in ("f32", "f16", "bf16"):
            xt = x.to(TD[T])
            q, s, s2 = NVFP4QTensor.quantize(xt, 8)
            k = f"nvq{i}_{T}_"
            cases[k + "x"] = bits(xt)
            cases[k + "packed"] = bits(q._quantized_data)
            cases[k + "scales"] = bits(s)
            cases[k + "scale2"] = bits(s2.reshape(1))
    cases["nvq_count"] = np.array(i + 1)

    src = (Path(ref_root) / "tests/gpu/torch/quantization/test_tensor_quant_cuda.py").read_text()
    fn = next(nd for nd in ast.walk(ast.parse(src)) if isinstance(nd, ast.FunctionDef) and nd.name == "test_cuda_ext_fp4")
    lits = []
    for node in ast.walk(fn):
        if isinstance(node, ast.Call) and ast.unparse(node.func) == "torch.tensor" and isinstance(node.args[0], ast.List):
            lits.append((node.lineno, np.array(ast.literal_eval(node.args[0]), dtype=np.float32)))
    lits = [t for _, t in sorted(lits, key=lambda p: p[0])]
    assert len(lits) == 8 and all(t.shape == (1, 8) for t in lits)
    # the test perturbs the third and fourth inputs by -0.1 / +0.1 (all but the last element)
    below, above = lits[4].copy(), lits[6].copy()
    below[:, :-1] -= np.float32(0.1)
    above[:, :-1] += np.float32(0.1)
    for i, (x, y) in enumerate([(lits[0], lits[1]), (lits[2], lits[3]), (below, lits[5]), (above, lits[7])]):
        cases[f"fp4fake{i}_x"], cases[f"fp4fake{i}_y"] = x, y
    np.savez_compressed(out / "reference_test_tables.npz", **cases)


def golden_fp8_gemm(out):
    """The reference's FP8 per-tensor linear (backends/fp8_per_tensor_gemm.py) on the CPU: its own
    ``_to_fp8`` and ``_fp8_gemm_impl`` run eagerly (torch.compile switched off), torch._scaled_mm
    being the CPU kernel of this torch build."""
    import torch._dynamo
    torch._dynamo.config.disable = True
    from modelopt.torch.quantization.backends import fp8_per_tensor_gemm as ref

    class Q:  # stands in for a TensorQuantizer: the function only reads .amax
        def __init__(self, amax):
            self.amax = amax

    class M:  # stands in for a RealQuantLinear with an uncompressed weight
        pass

    data = {}
    for i, (m, n, k, T, with_bias) in enumerate([(64, 128, 256, "bf16", True), (100, 136, 80, "bf16", False),
                                                 (32, 64, 512, "f16", True), (48, 96, 128, "f32", True)]):
        x = gen((m, k), T, 100 + i, 2.0)
        w = gen((n, k), T, 200 + i, 0.05, heavy=True)
        bias = gen((n,), T, 300 + i) if with_bias else None
        mod = M()
        mod.input_quantizer, mod.weight_quantizer = Q(x.abs().amax()), Q(w.abs().amax())
        mod.weight = w
        y = ref.fp8_per_tensor_gemm(mod, x, bias)
        data[f"case{i}_x"], data[f"case{i}_w"], data[f"case{i}_y"] = bits(x), bits(w), bits(y)
        data[f"case{i}_a8"] = bits(ref._to_fp8(x, mod._scale_a))
        data[f"case{i}_b8"] = bits(ref._to_fp8(w, mod._scale_b))
        data[f"case{i}_scale_a"], data[f"case{i}_scale_b"] = mod._scale_a.numpy(), mod._scale_b.numpy()
        if bias is not None:
            data[f"case{i}_bias"] = bits(bias)
        data[f"case{i}_meta"] = np.array([m, n, k, {"f32": 0, "f16": 1, "bf16": 2}[T], int(with_bias)])
    np.savez_compressed(out / "fp8_gemm.npz", **data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a TensorRT-Model-Optimizer checkout")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    import_reference(args.ref)
    torch.manual_seed(0)
    fns = {"fake_int": golden_fake_int, "fake_e4m3": golden_fake_e4m3, "nvfp4": golden_nvfp4,
           "int4": golden_int4, "q8": golden_q8, "amax": golden_amax, "hist": golden_hist, "export": golden_export, "mxfp4": golden_mxfp4, "bias": golden_bias,
           "fp8_gemm": golden_fp8_gemm}
    for name, fn in fns.items():
        if args.only and name not in args.only.split(","):
            continue
        fn(HERE)
        print("wrote", name)
    if not args.only or "reference_test_tables" in args.only.split(","):
        golden_reference_test_tables(HERE, args.ref)
        print("wrote reference_test_tables")
    if not args.only or "mx_known_answers" in args.only.split(","):
        golden_mx_known_answers(HERE, args.ref)
        print("wrote mx_known_answers")


if __name__ == "__main__":
    main()
