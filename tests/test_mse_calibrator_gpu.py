"""MseCalibrator behaviour, after the reference's own test file
(tests/unit/torch/quantization/test_mse_calibrator.py: outliers shrink the chosen amax, unsigned data,
accumulation over several collects, a custom error function, reset, per-channel search with independent
channels), on CUDA tensors.  Every case runs twice: through the candidate loop over the quantiser (what
the reference does) and with the one-pass kernel enabled (``fused=``) — the kernel takes the case when
its layout rules allow (at most 16 candidates, 32 sixteen-byte packs behind a channel axis) and must
then choose the same amax."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _quantizer(amax, axis=None, unsigned=False):
    import b200q as mtq

    cfg = mtq.QuantizerAttributeConfig(num_bits=8, axis=axis, unsigned=unsigned)
    return mtq.nn.TensorQuantizer(cfg, amax=amax).cuda()


def _quant_func(tq):
    def fn(x, amax):
        saved, if_quant, if_calib = tq._amax.clone(), tq._if_quant, tq._if_calib
        tq._amax, tq._if_quant, tq._if_calib = amax, True, False
        try:
            return tq(x)
        finally:
            tq._amax, tq._if_quant, tq._if_calib = saved, if_quant, if_calib
    return fn


def _mse_at(x, a, unsigned=False):
    qmin, qmax = (0, 255) if unsigned else (-128, 127)
    s = torch.clamp(a / max(abs(qmin), abs(qmax)), min=torch.finfo(torch.float32).eps)
    return ((x - torch.clamp(torch.round(x / s), qmin, qmax) * s) ** 2).mean()


def _calibrator(amax, tq, fused, **kw):
    from b200q.calib import MseCalibrator

    spec = {"num_bits": 8, "unsigned": tq._unsigned, "narrow_range": tq._narrow_range} if fused else None
    return MseCalibrator(amax=amax, quant_func=_quant_func(tq), fused=spec, **kw)


@pytest.fixture(params=[False, True], ids=["loop", "kernel"])
def fused(request):
    return request.param


def test_an_outlier_is_clipped(fused):
    x = torch.ones(1024, device="cuda")
    x[0] = 10.0
    amax = x.abs().max()
    tq = _quantizer(amax)
    cal = _calibrator(amax, tq, fused, num_steps=16, start_multiplier=0.1, stop_multiplier=1.5)
    cal.collect(x)
    best = cal.compute_amax()
    assert (cal._loss_buf is not None) == fused
    assert torch.isfinite(best) and 0 < best <= x.abs().max() * 1.5 + 1e-6
    assert _mse_at(x, best) <= _mse_at(x, torch.tensor(1.0, device="cuda")) + 1e-6


def test_a_negative_outlier_is_clipped(fused):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.rand(4096, generator=g, device="cuda") * 2.0 - 1.0
    x[0] = -12.0
    amax = x.abs().max()
    tq = _quantizer(amax)
    cal = _calibrator(amax, tq, fused, num_steps=16, start_multiplier=0.1, stop_multiplier=1.2)
    cal.collect(x)
    best = cal.compute_amax()
    assert torch.isfinite(best) and 0 < best <= x.abs().max() * 1.2 + 1e-6
    assert _mse_at(x, best) <= _mse_at(x, torch.tensor(1.0, device="cuda")) + 1e-6


def test_unsigned_data(fused):
    x = torch.full((11, 7, 3, 3), 512.0, device="cuda")
    x[1, 1, 1, 1] = 513.0
    amax = x.abs().max()
    tq = _quantizer(amax, unsigned=True)
    cal = _calibrator(amax, tq, fused, num_steps=16, start_multiplier=0.5, stop_multiplier=1.2)
    cal.collect(x)
    best = cal.compute_amax()
    assert torch.isfinite(best) and 0 < best <= x.abs().max() * 1.2 + 1e-6
    assert _mse_at(x, best, unsigned=True) < 1.0


def test_collects_accumulate(fused):
    x1 = torch.full((2048,), 2.0, device="cuda")
    x1[0] = 16.0
    amax = x1.abs().max()
    tq = _quantizer(amax)
    cal = _calibrator(amax, tq, fused, num_steps=16, start_multiplier=0.1, stop_multiplier=1.5)
    cal.collect(x1)
    after_one = [float(l) for l in cal._losses_sum]
    cal.collect(torch.full((2048,), 2.0, device="cuda"))
    after_two = [float(l) for l in cal._losses_sum]
    assert all(b >= a for a, b in zip(after_one, after_two)) and any(b > a for a, b in zip(after_one, after_two))
    best = cal.compute_amax()
    assert torch.isfinite(best) and 0 < best <= amax * 1.5 + 1e-6


def test_a_custom_error_function_takes_the_loop():
    from b200q.calib import MseCalibrator

    x = torch.full((512,), 5.0, device="cuda")
    x[0] = 10.0
    amax = x.abs().max()
    tq = _quantizer(amax)
    calls = []

    def l1(a, b):
        calls.append(1)
        return torch.abs(a - b)

    cal = MseCalibrator(amax=amax, num_steps=10, start_multiplier=0.5, stop_multiplier=1.5, quant_func=_quant_func(tq),
                        error_func=l1, fused={"num_bits": 8, "unsigned": False, "narrow_range": tq._narrow_range})
    cal.collect(x)
    assert len(calls) == 10 and cal._loss_buf is None
    best = cal.compute_amax()
    assert torch.isfinite(best) and 0 < best <= amax * 1.5 + 1e-6


def test_reset_clears_the_state(fused):
    x = torch.full((512,), 2.0, device="cuda")
    amax = x.abs().max()
    tq = _quantizer(amax)
    cal = _calibrator(amax, tq, fused, num_steps=10)
    cal.collect(x)
    assert cal.compute_amax() is not None
    cal.reset()
    assert cal.compute_amax() is None
    cal.collect(x)                       # and it can be used again
    assert cal.compute_amax() is not None


def test_per_channel_shapes_and_accumulation(fused):
    """2 x 3 weights (too narrow for the kernel: it defers to the loop), three batches."""
    amax = torch.tensor([[3.0], [6.0]], device="cuda")
    tq = _quantizer(amax, axis=0)
    cal = _calibrator(amax, tq, fused, axis=0, num_steps=15, start_multiplier=0.5, stop_multiplier=2.0)
    for rows in ([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], [[0.5, 1.5, 2.5], [3.5, 4.5, 5.5]], [[1.2, 2.2, 3.2], [4.2, 5.2, 6.2]]):
        cal.collect(torch.tensor(rows, device="cuda"))
    assert cal._loss_buf is None
    best = cal.compute_amax()
    assert best.shape == amax.shape and torch.isfinite(best).all() and (best > 0).all()


def test_channels_are_optimised_independently(fused):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.zeros(2, 1024, device="cuda")
    x[0] = torch.randn(1024, generator=g, device="cuda") * 0.5 + 1.0
    x[1] = torch.randn(1024, generator=g, device="cuda") * 5.0 + 100.0
    amax = x.abs().amax(dim=1, keepdim=True)
    tq = _quantizer(amax, axis=0)
    cal = _calibrator(amax, tq, fused, axis=0, num_steps=16, start_multiplier=0.5, stop_multiplier=1.5)
    cal.collect(x)
    assert (cal._loss_buf is not None) == fused          # 1024 elements per channel: the kernel's layout
    best = cal.compute_amax()
    assert best.shape == amax.shape and torch.isfinite(best).all() and (best > 0).all()
    assert best[1, 0] > best[0, 0] * 10


def test_loop_and_kernel_choose_the_same_amax():
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(64, 2048, generator=g, device="cuda") * torch.exp(torch.randn(64, 1, generator=g, device="cuda"))
    x[:, 0] *= 6
    chosen = []
    for fused in (False, True):
        amax = x.abs().amax(dim=1, keepdim=True)
        tq = _quantizer(amax, axis=0)
        cal = _calibrator(amax, tq, fused, axis=0, num_steps=10)
        cal.collect(x)
        cal.collect(x * 0.5)
        chosen.append(cal.compute_amax().clone())
    assert (chosen[0] == chosen[1]).float().mean() >= 0.97      # a near-tie between two candidates may flip
