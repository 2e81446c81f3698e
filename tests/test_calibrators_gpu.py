"""The calibrator cases of the reference's own test file (tests/unit/torch/quantization/test_calibrator.py:
MaxCalibrator simple / per-axis / tracked / shape change, HistogramCalibrator growth and skip_zeros, the
entropy, mse and percentile read-outs on one and two tensors, unsigned data, argument range,
calibrate_weights per tensor and per channel), run on CUDA tensors through the kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def calib():
    import b200q

    return b200q.calib


def _rand(*shape, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.rand(*shape, generator=g, device="cuda")


# ---- MaxCalibrator (reference :28-90) ---------------------------------------------------------------

def test_max_simple_run(calib):
    cal = calib.MaxCalibrator(8, None, False)
    x1, x2 = _rand(16, seed=1), _rand(16, seed=2)
    cal.collect(x1)
    cal.collect(x2)
    assert cal.compute_amax().item() == torch.max(x1.max(), x2.max()).item()
    calib.MaxCalibrator(8, None, True)


@pytest.mark.parametrize("axis", [0, -4])
def test_max_fine_grain(calib, axis):
    from b200q import utils

    cal = calib.MaxCalibrator(8, axis, False)
    x1, x2 = _rand(3, 4, 2, 2, seed=3), _rand(3, 4, 2, 2, seed=4)
    cal.collect(x1)
    cal.collect(x2)
    got = cal.compute_amax()
    assert got.shape[0] == 3
    assert torch.equal(got, utils.reduce_amax(torch.max(x1, x2), axis=(1, 2, 3)))
    cal.reset()
    assert cal.compute_amax() is None


def test_max_track_amax(calib):
    cal = calib.MaxCalibrator(8, None, False, track_amax=True)
    x1, x2 = _rand(16, seed=5), _rand(16, seed=6)
    cal.collect(x1)
    cal.collect(x2)
    assert cal.compute_amax().item() == torch.max(x1.max(), x2.max()).item()
    np.testing.assert_array_equal(cal.amaxs[0], x1.max().cpu().numpy())
    np.testing.assert_array_equal(cal.amaxs[1], x2.max().cpu().numpy())


def test_max_shape_change_raises(calib):
    cal = calib.MaxCalibrator(8, 0, False)
    cal.collect(_rand(3, 4, 2, 2))
    with pytest.raises(RuntimeError, match="shape changed"):
        cal.collect(_rand(4, 4, 2, 2))


# ---- HistogramCalibrator (reference :93-138) --------------------------------------------------------

def test_histogram_growth(calib):
    """A second batch beyond the first one's range extends the histogram at the same bin width ("append");
    the outlier 256 does not drag the mse amax away from 255."""
    x1 = torch.tensor([0, 255, 255, 255, 255, 255], device="cuda")
    x2 = torch.tensor([0, 255, 255, 255, 255, 256], device="cuda")
    cal = calib.HistogramCalibrator(8, None, False, num_bins=2048, grow_method="append")
    cal.collect(x1)
    cal.collect(x2)
    assert abs(cal.compute_amax("mse", start_bin=128).item() - 255.0) < 0.5
    assert cal._num_bins > 2048              # the live length is read back with the first read-out
    assert abs(cal.compute_amax("entropy", start_bin=128).item() - 255.0) < 1.5


def test_histogram_skip_zeros(calib):
    x1 = torch.tensor([0, 0, 0, 0, 0, 1, 2, 3, 4, 5], device="cuda")
    x2 = torch.tensor([0, 0, 0, 0, 0, 6, 7, 8, 9, 10], device="cuda")
    cal = calib.HistogramCalibrator(8, None, False, num_bins=2048, skip_zeros=True)
    cal.collect(x1)
    cal.collect(x2)
    amax = cal.compute_amax("percentile", percentile=50, start_bin=128)
    assert abs(amax.item() - 5.0) < 10 / 2048 + 5 / 2048


# ---- entropy (reference :184-245) -------------------------------------------------------------------

@pytest.mark.parametrize("unsigned", [False, True])
def test_entropy_discards_an_outlier(calib, unsigned):
    cal = calib.HistogramCalibrator(8, None, unsigned, num_bins=2048)
    x = _rand(11, 7, 3, 3, seed=7)
    x[1, 1, 1, 1] = 10.0
    cal.collect(x)
    assert cal.compute_amax("entropy", start_bin=128).item() < 1.1


def test_entropy_two_tensors(calib):
    cal = calib.HistogramCalibrator(8, None, False, num_bins=2048)
    x = _rand(11, 7, 3, 3, seed=8)
    x[1, 1, 1, 1] = 10.0
    cal.collect(x)
    cal.collect(_rand(11, 7, 3, 3, seed=9))
    assert cal.compute_amax("entropy", start_bin=128).item() < 1.1
    repr(cal)


# ---- mse from the histogram (reference :247-300) ----------------------------------------------------

def test_hist_mse_one_tensor(calib):
    cal = calib.HistogramCalibrator(8, None, False, num_bins=32)
    x = torch.full((4, 4, 4), 255.0, device="cuda")
    x[1, 1, 1] = 256.0
    cal.collect(x)
    amax = cal.compute_amax("mse", start_bin=16).item()
    assert abs(amax - 255.0) < abs(amax - 256.0)


def test_hist_mse_unsigned(calib):
    cal = calib.HistogramCalibrator(8, None, True, num_bins=32)
    x = torch.full((11, 7, 3, 3), 512.0, device="cuda")
    x[1, 1, 1, 1] = 513.0
    cal.collect(x)
    amax = cal.compute_amax("mse", start_bin=8).item()
    assert abs(amax - 512.0) < abs(amax - 513.0)


def test_hist_mse_two_tensors(calib):
    cal = calib.HistogramCalibrator(8, None, False)
    x = torch.full((11, 7, 3, 3), 255.0, device="cuda")
    x[1, 1, 1, 1] = 256.0
    cal.collect(x)
    cal.collect(torch.full((11, 7, 3, 3), 255.0, device="cuda"))
    amax = cal.compute_amax("mse").item()
    assert abs(amax - 255.0) < abs(amax - 256.0)
    repr(cal)


# ---- percentile (reference :302-361) ----------------------------------------------------------------

def test_percentile_one_tensor(calib):
    cal = calib.HistogramCalibrator(8, None, False)
    cal.collect(torch.arange(100, device="cuda"))
    assert abs(cal.compute_amax("percentile", percentile=90).item() - 89.0) < 100 / 1024


def test_percentile_unsigned(calib):
    cal = calib.HistogramCalibrator(8, None, True)
    cal.collect(torch.arange(100, device="cuda"))
    assert abs(cal.compute_amax("percentile", percentile=80).item() - 79.0) < 100 / 2048


def test_percentile_two_tensors(calib):
    cal = calib.HistogramCalibrator(8, None, False)
    cal.collect(torch.arange(100, device="cuda"))
    cal.collect(torch.arange(0, 50, 0.5, device="cuda"))
    assert abs(cal.compute_amax("percentile", percentile=99).item() - 97.0) < 100 / 1024


def test_percentile_range_is_checked(calib):
    cal = calib.HistogramCalibrator(8, None, False)
    cal.collect(torch.arange(100, device="cuda"))
    with pytest.raises(ValueError, match="range"):
        cal.compute_amax("percentile", percentile=-10)
    with pytest.raises(ValueError, match="range"):
        cal.compute_amax("percentile", percentile=200)


# ---- calibrate_weights (reference :364-435) ---------------------------------------------------------

def _two_linears():
    import b200q as mtq

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 48), torch.nn.ReLU(), torch.nn.Linear(48, 32)).cuda()
    mtq.replace_quant_module(model)
    return model


def test_calibrate_weights_max_equals_the_quantisers_own_calibration(calib):
    ref, test = _two_linears(), _two_linears()
    test.load_state_dict(ref.state_dict())
    for m in ref.modules():
        if hasattr(m, "weight_quantizer"):
            m.weight_quantizer.enable_calib()
            m.weight_quantizer.disable_quant()
            m.weight_quantizer(m.weight)
            m.weight_quantizer.load_calib_amax()
    calib.calibrate_weights(test, method="max")
    for a, b in zip(ref.modules(), test.modules()):
        if hasattr(a, "weight_quantizer"):
            assert torch.equal(a.weight_quantizer.amax, b.weight_quantizer.amax)
            assert a.weight_quantizer.amax.shape == b.weight_quantizer.amax.shape


@pytest.mark.parametrize("method", ["mse", "percentile"])
def test_calibrate_weights_per_tensor_and_per_channel(calib, method):
    model = _two_linears()
    calib.calibrate_weights(model, method=method, perchannel=False)
    ref = calib.HistogramCalibrator(8, None, False)
    ref.collect(model[0].weight)
    assert model[0].weight_quantizer.amax.item() == ref.compute_amax(method).item()
    model = _two_linears()
    calib.calibrate_weights(model, method=method, perchannel=True)
    ref = calib.HistogramCalibrator(8, None, False)
    ref.collect(model[2].weight[1])
    assert model[2].weight_quantizer.amax.reshape(-1)[1].item() == ref.compute_amax(method).item()
