"""``TensorQuantizer`` / ``SequentialQuantizer`` behaviour, after the reference's own test files
(tests/_test_utils/torch/quantization/tensor_quantizer_common.py run by
tests/gpu/torch/quantization/test_tensor_quantizer_cuda.py): default fake quant, per tensor / per channel,
disable, state loading, properties and setters, calibration at construction, max calibration, histogram
read-outs, pre_quant_scale known answers, modelopt state, amax export shapes, save / restore, backward,
block_sizes given as axes, block quantisation with and without padding against the reshaped per-row
form, E4M3 and NVFP4 quantisers, sequential quantisers.  All tensors live on the GPU."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


def _rand(*shape, seed=0, uniform=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    fn = torch.rand if uniform else torch.randn
    return fn(*shape, generator=g, device="cuda")


def _tq(mtq, amax=None, if_quant=True, if_calib=False, **cfg):
    return mtq.nn.TensorQuantizer(mtq.QuantizerAttributeConfig(**cfg), if_quant=if_quant, if_calib=if_calib,
                                  amax=amax).cuda()


def quant(x, amax, num_bits=8):
    intmax = 2.0 ** (num_bits - 1) - 1.0
    scale = intmax / amax
    return torch.clamp((x * scale).round_(), -intmax, intmax) / scale


NVFP4 = dict(num_bits=(2, 1), block_sizes={-1: 16, "type": "dynamic", "scale_bits": (4, 3)})


# ---- the shared quantiser cases (tensor_quantizer_common.py:31-343) ---------------------------------------

def test_default_is_fake_tensor_quant(mtq):
    x = _rand(3, 7)
    want = mtq.tensor_quant.fake_tensor_quant(x, x.abs().max(), None)
    assert torch.allclose(mtq.nn.TensorQuantizer()(x), want)


def test_per_tensor_scale(mtq):
    x = _rand(31, seed=1)
    assert torch.allclose(_tq(mtq, num_bits=8, narrow_range=True)(x), quant(x, x.abs().max()))


def test_per_channel_scale(mtq):
    x = _rand(5, 5, 4, 8, seed=2)
    amax = torch.amax(x.abs(), dim=(1, 2, 3), keepdim=True)
    assert torch.allclose(_tq(mtq, num_bits=8, axis=0)(x), quant(x, amax), rtol=1e-2)


def test_disable(mtq):
    x = _rand(3, 7, seed=3)
    assert torch.equal(_tq(mtq, enable=False)(x), x)


def test_state_loading(mtq):
    amax = [3.14, 2.718]
    q = _tq(mtq, amax=amax, num_bits=(4, 3))
    q.load_state_dict(q.state_dict())
    assert torch.allclose(q.amax, torch.tensor(amax, device="cuda"))


def test_properties(mtq):
    q = _tq(mtq, amax=3.14)
    q.amax = 0.577
    assert q.amax == torch.tensor(0.577, device="cuda")
    assert q.step_size == 0.577 / 127.0
    q2 = _tq(mtq)
    amax = torch.tensor([3.142, 2.718], device="cuda")
    q2.amax = amax
    assert torch.allclose(q2.amax, amax)
    assert mtq.nn.TensorQuantizer().amax is None
    with pytest.raises(RuntimeError, match="shape"):
        q2.amax = torch.tensor([1.0, 2.0, 3.0])


def test_calibration_from_construction(mtq):
    q = _tq(mtq, if_calib=True, if_quant=False, axis=(0, 1))
    q(_rand(7, 6, 7, 7, seed=4, uniform=True))
    q.load_calib_amax()
    assert q.amax.numel() == 7 * 6


def test_max_calibration(mtq):
    from b200q import utils

    q = _tq(mtq, axis=0)
    q.enable_calib()
    with pytest.raises(RuntimeError, match="Calibrator returned None"):
        q.load_calib_amax()
    x1, x2 = _rand(7, 6, 7, 7, seed=5, uniform=True), _rand(7, 6, 7, 7, seed=6, uniform=True)
    q(x1)
    q(x2)
    q.disable_calib()
    want = torch.max(utils.reduce_amax(x1, axis=(1, 2, 3), keepdims=True),
                     utils.reduce_amax(x2, axis=(1, 2, 3), keepdims=True))
    assert torch.equal(q._calibrator.compute_amax(), want)
    q.load_calib_amax()
    assert torch.equal(q.amax, want)


def test_entropy_and_percentile_calibration(mtq):
    q = _tq(mtq, if_calib=True, if_quant=False, calibrator="histogram")
    x1, x2 = _rand(3, 6, 7, 7, seed=7, uniform=True), _rand(3, 6, 7, 7, seed=8, uniform=True)
    q(x1)
    q(x2)
    q.load_calib_amax("entropy")
    assert torch.equal(q._calibrator.compute_amax("entropy"), q.amax)
    q._calibrator.reset()
    q(x1)
    q(x2)
    q.load_calib_amax("percentile", percentile=99.99)
    assert torch.equal(q._calibrator.compute_amax("percentile", percentile=99.99), q.amax)
    assert 0.9 < q.amax.item() <= 1.0


def test_setters(mtq):
    q = mtq.nn.TensorQuantizer()
    q.num_bits = 7
    q.unsigned = True
    assert q.num_bits == 7 and q.unsigned


def test_pre_quant_scale_known_answers(mtq):
    q = _tq(mtq, amax=127.0, axis=1, num_bits=8)
    q2 = _tq(mtq, amax=127.0, axis=1, num_bits=8)
    x = torch.tensor([[0, 0.4, 1.1, 2.0]], device="cuda")
    assert torch.allclose(q(x), torch.tensor([[0.0, 0, 1, 2]], device="cuda"))
    q.pre_quant_scale = 2.0
    assert torch.allclose(q(x), torch.tensor([[0.0, 1, 2, 4]], device="cuda"))
    q2.pre_quant_scale = torch.tensor([[1.0, 2.0, 3.0, 4.0]], device="cuda")
    assert torch.allclose(q2(x), torch.tensor([[0.0, 1, 3, 8]], device="cuda"))


def test_set_from_attribute_config(mtq):
    q = mtq.nn.TensorQuantizer()
    q.set_from_attribute_config({"num_bits": 4})
    assert q.num_bits == 4
    q.set_from_attribute_config({"axis": -1})
    assert q.axis == -1
    q.set_from_attribute_config({"enable": False})
    assert q._disabled


def test_modelopt_state(mtq):
    ref = _tq(mtq, amax=10.0, num_bits=4)
    test = mtq.nn.TensorQuantizer()
    state = ref.get_modelopt_state()
    for k in ("_num_bits", "_axis", "_unsigned", "_narrow_range", "_fake_quant", "_disabled", "_block_sizes",
              "_if_quant", "_if_calib"):
        assert k in state and state[k] == getattr(ref, k)
    assert "_amax" not in state and "_amax" in state["_pytorch_state_metadata"]["buffers"]
    test.set_from_modelopt_state(state)
    test.load_state_dict(ref.state_dict())
    test.cuda()
    x = _rand(10, 10, seed=9)
    assert torch.equal(ref(x), test(x))


def test_amax_export_shapes(mtq):
    a = _rand(4, 6, 8, seed=10)
    for block, blocks_per_row in ((4, 2), (8, 1)):
        q = _tq(mtq, num_bits=4, block_sizes={-1: block})
        assert not hasattr(q, "_amax_shape_for_export")
        q(a)
        q.enable_calib()
        q(a)
        q.load_calib_amax()
        amax = q.export_amax()
        assert q._amax_shape_for_export == (4, 6, -1)
        assert amax.shape == (4, 6, blocks_per_row)
        assert torch.equal(amax, a.reshape(4, 6, blocks_per_row, block).abs().amax(dim=-1))
    q = _tq(mtq, num_bits=4, axis=0)
    q.enable_calib()
    q(a)
    q.load_calib_amax()
    assert not hasattr(q, "_amax_shape_for_export") and q.export_amax().shape == (4,)
    q = _tq(mtq, num_bits=4)
    q.enable_calib()
    q(a)
    q.load_calib_amax()
    assert q.export_amax().shape == (1,)


def test_save_restore(mtq):
    ref = _tq(mtq, num_bits=4, axis=0)
    ref.enable_calib()
    ref(_rand(4, 6, 8, seed=11))
    ref(_rand(4, 6, 8, seed=12))
    ref.load_calib_amax()
    ref.disable_calib()
    test = mtq.nn.TensorQuantizer()
    test.set_from_modelopt_state(ref.get_modelopt_state())
    test.load_state_dict(ref.state_dict())
    test.cuda()
    x = _rand(4, 6, 8, seed=13)
    assert torch.equal(ref(x), test(x))


def test_backward_runs(mtq):
    x = _rand(3, 7, seed=14).requires_grad_(True)
    mtq.nn.TensorQuantizer()(x).sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))


def test_block_sizes_given_as_axes(mtq):
    w, x = _rand(3, 3, seed=15), _rand(1, 2, 3, seed=16)
    assert torch.equal(_tq(mtq, num_bits=8, block_sizes={1: None})(w), _tq(mtq, num_bits=8, axis=0)(w))
    assert torch.equal(_tq(mtq, num_bits=8, block_sizes={0: None, 1: None})(x), _tq(mtq, num_bits=8, axis=-1)(x))


# ---- block quantisation (:346-448) ------------------------------------------------------------------------

def _blockwise(mtq, a, block_sizes, calibrate=True):
    q = _tq(mtq, num_bits=8, block_sizes=block_sizes)
    if calibrate:
        q.enable_calib()
    out = q(a)
    if calibrate:
        q.load_calib_amax()
    return q, out


def test_blocks_along_the_last_dimension(mtq):
    a = _rand(8, 4, seed=17)
    amax = a.view(-1, 2).abs().amax(dim=-1, keepdim=True)
    want = mtq.tensor_quant.fake_tensor_quant(a.view(-1, 2), amax, None, 8, False, False).view_as(a)
    for bs in ({-1: 2}, {1: 2}):
        q, out = _blockwise(mtq, a, bs)
        assert torch.equal(q.amax, amax) and torch.equal(out, want)


def test_blocks_over_two_dimensions(mtq):
    a = _rand(2, 6, 4, seed=18)
    amax = a.reshape(2, 2, 3, 2, 2).abs().amax(dim=(2, 4), keepdim=True)
    want = mtq.tensor_quant.fake_tensor_quant(a.reshape(2, 2, 3, 2, 2), amax, None, 8, False, False).view_as(a)
    for bs in ({-1: 2, 1: 3}, {1: 3, 2: 2}):
        assert torch.allclose(_blockwise(mtq, a, bs, calibrate=False)[1], want)


def test_blocks_with_padding(mtq):
    a = _rand(3, 4, 5, seed=19)
    padded = F.pad(a, (0, 1))
    amax = padded.view(-1, 2).abs().amax(dim=-1, keepdim=True)
    want = mtq.tensor_quant.fake_tensor_quant(padded.view(-1, 2), amax, None, 8, False, False).view_as(padded)[:, :, :5]
    for bs in ({-1: 2}, {2: 2}):
        q, out = _blockwise(mtq, a, bs)
        assert torch.equal(q.amax, amax) and torch.equal(out, want)


def test_blocks_over_two_dimensions_with_padding(mtq):
    a = _rand(2, 10, 5, seed=20)
    padded = F.pad(a, (0, 1, 0, 2))
    amax = padded.view(2, 4, 3, 3, 2).abs().amax(dim=(2, 4), keepdim=True)
    want = mtq.tensor_quant.fake_tensor_quant(padded.view(2, 4, 3, 3, 2), amax, None, 8, False, False
                                              ).view_as(padded)[:, :10, :5]
    q, out = _blockwise(mtq, a, {-1: 2, 1: 3})
    assert torch.equal(q.amax.reshape(-1), amax.reshape(-1)) and torch.allclose(out, want)
    assert torch.allclose(_blockwise(mtq, a, {1: 3, 2: 2}, calibrate=False)[1], want)


# ---- E4M3 and NVFP4 quantisers (test_tensor_quantizer_cuda.py:42-118) -------------------------------------

@pytest.mark.parametrize(("E", "M", "axis"), [(5, 2, None), (4, 3, None), (4, 3, 1), (7, 3, None)])
def test_e4m3_quantiser(mtq, E, M, axis):  # noqa: N803
    if (E, M) != (4, 3):
        with pytest.raises(ValueError):
            mtq.QuantizerAttributeConfig(num_bits=(E, M), axis=axis)
        return
    q = _tq(mtq, num_bits=(E, M), axis=axis)
    x = _rand(3, 6, 7, 7, seed=21, uniform=True)
    assert torch.equal(q(x), mtq.tensor_quant.scaled_e4m3(x, q._get_amax(x), None, E, M))


def test_fp4_quantiser(mtq):
    q = _tq(mtq, **NVFP4)
    x = _rand(2, 1, 16, seed=22, uniform=True)
    want = mtq.tensor_quant.dynamic_block_quant(x, 16, x.abs().amax(), None, (2, 1), (4, 3))
    assert torch.equal(q(x), want)
    assert q._get_amax(x) == x.abs().amax()


def test_fp4_backward_masks_beyond_amax(mtq):
    q = _tq(mtq, **NVFP4)
    x = _rand(2, 1, 16, seed=23, uniform=True)
    q.amax = torch.median(x.abs())
    x.requires_grad_(True)
    q(x).sum().backward()
    assert torch.equal(x.grad, (x.detach().abs() <= q.amax).float())


def test_fp4_non_contiguous_input(mtq):
    contiguous = torch.ones(2, 16, device="cuda")
    large = torch.ones(2, 32, device="cuda")
    large[:, :16] = _rand(2, 16, seed=24)
    view = large[:, 16:]
    assert torch.equal(contiguous, view) and not view.is_contiguous()
    q = _tq(mtq, axis=None, enable=True, **NVFP4)
    assert torch.equal(q(contiguous), q(view))


# ---- sequential quantisers (:451-520) ---------------------------------------------------------------------

def test_sequential_quantizer_applies_its_members_in_order(mtq):
    TQ, SQ = mtq.nn.TensorQuantizer, mtq.nn.SequentialQuantizer
    cfgs = [{"num_bits": 4}, {"block_sizes": {-1: 4}}, {"enable": False}]
    nq = SQ(TQ(), TQ(), TQ())
    singles = [TQ() for _ in cfgs]
    for member, single, cfg in zip(nq, singles, cfgs):
        member.set_from_attribute_config(cfg)
        single.set_from_attribute_config(cfg)
    x = _rand(2, 16, seed=25)
    want = x
    for single in singles:
        want = single(want)
    assert torch.equal(nq(x), want)


def test_sequential_quantizer_is_swapped_out_and_back(mtq):
    SQ = mtq.nn.SequentialQuantizer
    model = torch.nn.Module()
    model.model = torch.nn.Sequential(mtq.nn.QuantLinear(4, 4), torch.nn.ReLU())
    seq = SQ(mtq.nn.TensorQuantizer(), mtq.nn.TensorQuantizer())
    model.model[0].weight_quantizer = seq
    with SQ.convert_to_single_quantizer(model):
        assert not any(isinstance(m, SQ) for m in model.modules())
    assert model.model[0].weight_quantizer is seq
    assert not hasattr(model.model[0], "_original_weight_quantizer")


def test_sequential_quantizer_attributes(mtq):
    sq = mtq.nn.SequentialQuantizer(mtq.nn.TensorQuantizer(), mtq.nn.TensorQuantizer()).cuda()
    sq.disable()
    assert not sq[0].is_enabled and not sq[1].is_enabled
    sq.enable()
    assert sq[0].is_enabled and sq[1].is_enabled
    mtq.model_calib.max_calibrate(sq, lambda m: m(_rand(1, 4, seed=26)))
    assert sq[0].amax is not None and sq[1].amax is not None
    sq.reset_amax()
    assert sq[0].amax is None and sq[1].amax is None
    assert sq.fake_quant is True
    sq[0]._fake_quant = False
    assert sq.fake_quant is False and sq[1]._fake_quant is True


# ---- affine (bias) quantisation and printing (tests/unit/torch/quantization/test_affine_quant.py:52-98,
# ---- test_print.py) ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("num_bits", [(2, 1), (4, 3)])
@pytest.mark.parametrize("bias_type", ["static", "dynamic"])
@pytest.mark.parametrize("method", ["mean", "max_min"])
@pytest.mark.parametrize("axis", [(-1,), (-1, -3), (-1, -2, -3)])
def test_bias_calibration_shapes(mtq, num_bits, bias_type, method, axis):
    from b200q.model_calib import enable_stats_collection, finish_stats_collection

    x = _rand(2, 3, 4, 16, seed=40)
    cfg = {"num_bits": num_bits, "bias": {**dict.fromkeys(axis), "type": bias_type, "method": method}}
    if num_bits == (2, 1):
        cfg["block_sizes"] = {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}
    q = _tq(mtq, **cfg)
    enable_stats_collection(q)
    y = q(x)
    finish_stats_collection(q)
    assert y.shape == x.shape
    positive = {a % x.dim() for a in axis}
    want = tuple(1 if d in positive else n for d, n in enumerate(x.shape))
    if bias_type == "static":
        assert tuple(q._bias_calibrator._calib_bias.shape) == want
        assert torch.allclose(q._bias_calibrator._calib_bias, q.bias_value)
    out = q(x)
    assert out.shape == x.shape and torch.isfinite(out).all()


def test_printing(mtq, capsys):
    print(mtq.nn.TensorQuantizer())
    model = torch.nn.Sequential(torch.nn.Linear(33, 65), mtq.nn.QuantLinear(33, 65))
    print(model)
    print(mtq.calib.MaxCalibrator(7, 1, False))
    hist = mtq.calib.HistogramCalibrator(8, None, True)
    hist.collect(_rand(10, seed=41, uniform=True))
    print(hist)
    text = capsys.readouterr().out
    assert "TensorQuantizer" in text and "QuantLinear" in text and "MaxCalibrator" in text and "HistogramCalibrator" in text
