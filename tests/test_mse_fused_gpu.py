"""All MSE-search candidates in one pass (``b200q_mse_candidates``) against the candidate loop it
replaces (reference: modelopt/torch/quantization/calib/mse.py:76-100 — per candidate a fake-quant pass,
``F.mse_loss(reduction="none")`` and a sum).

Tolerance on the losses, against a float64 sum of the loop's per-element errors:
|loss - want| <= 1e-5 * want + 2e-7 * sum(x^2).  The integer path forms x - r / scale from the exact
quotient (two FMAs) where the loop rounds the quotient to fp32 first: per element the error d moves by
at most half an ulp of the quotient q, so d^2 moves by at most |d| * ulp(q) <= 6e-8 * (d^2 + q^2) — the
second term of the bound (it only matters where x sits almost on the grid, as 16-bit inputs do).
Partial sums are fp32 per thread (the first term).  The selected amax — what calibration returns,
parity tolerance 1e-3 — is asserted equal."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _loop_losses(x, cands, axis, num_bits, unsigned, narrow):
    from b200q import ops

    xf = x.float()
    out = []
    for c in cands:
        if isinstance(num_bits, int):
            shape = [1] * x.dim()
            if axis is not None:
                shape[axis] = -1
            xq = ops.fake_int(xf, c.reshape(shape) if axis is not None else c.reshape(()), num_bits, unsigned, narrow)
        else:
            xq = ops.fake_e4m3(xf, c.reshape(()))
        d = (xf - xq).double() ** 2
        out.append(d.sum() if axis is None else d.sum(dim=[i for i in range(x.dim()) if i != axis % x.dim()]))
    return torch.stack([o.reshape(-1) for o in out])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,axis", [
    ((4096, 1024), None), ((1000, 333), None), ((7,), None), ((2, 300, 4096), None),
    ((512, 1024), 0), ((96, 256), 0), ((3, 64, 512), 1), ((1, 8192), 0),
])
@pytest.mark.parametrize("fmt", [(8, False, True), (4, False, False), (8, True, False), ((4, 3), False, False)])
def test_candidates_kernel_equals_the_loop(dtype, shape, axis, fmt):
    from b200q import ops

    num_bits, unsigned, narrow = fmt
    if not isinstance(num_bits, int) and axis is not None:
        pytest.skip("E4M3 fake quantisation is per tensor")
    g = torch.Generator(device="cuda").manual_seed(hash((shape, axis)) % 1000)
    x = (torch.randn(shape, generator=g, device="cuda") * 3).to(dtype)
    if unsigned:
        x = x.abs()
    assert ops.mse_candidates_supported(x, axis)
    base = x.abs().amax().float().reshape(1) if axis is None else \
        x.abs().float().amax(dim=[i for i in range(x.dim()) if i != axis]).reshape(-1)
    mult = torch.linspace(0.25, 4.0, 10, device="cuda")
    cands = base[None, :] * mult[:, None]
    loss = torch.zeros(cands.shape, dtype=torch.float64, device="cuda")
    ops.mse_candidates(x, cands, loss, axis, num_bits, unsigned, narrow)
    want = _loop_losses(x, cands, axis, num_bits, unsigned, narrow)
    energy = (x.double() ** 2).sum() if axis is None else \
        (x.double() ** 2).sum(dim=[i for i in range(x.dim()) if i != axis]).reshape(1, -1)
    assert ((loss - want).abs() <= 1e-5 * want + 2e-7 * energy).all(), (loss - want).abs().max()
    ops.mse_candidates(x, cands, loss, axis, num_bits, unsigned, narrow)      # accumulates
    assert ((loss - 2 * want).abs() <= 2e-5 * want + 4e-7 * energy).all()


def test_candidates_kernel_dead_and_tiny_amax():
    """amax 0 and amax below 2^-24 follow the stand-alone kernel's rules (integer: scale treated as
    dead, values pass through as zero codes; E4M3: the same)."""
    from b200q import ops

    x = torch.randn(64, 256, device="cuda").bfloat16()
    cands = torch.tensor([[0.0], [1e-9], [1.0], [float(x.abs().max())]], device="cuda")
    for bits in (8, (4, 3)):
        loss = torch.zeros(4, 1, dtype=torch.float64, device="cuda")
        ops.mse_candidates(x, cands, loss, None, bits, False, True)
        want = _loop_losses(x, cands, None, bits, False, True)
        assert torch.isfinite(loss).all()
        assert torch.allclose(loss, want, rtol=1e-5), (bits, loss, want)


def test_unsupported_layouts_are_refused_and_take_the_loop():
    from b200q import _cabi, ops
    from b200q.calib import MseCalibrator

    x = torch.randn(64, 100, device="cuda").bfloat16()          # 100 elements behind the channel axis
    assert not ops.mse_candidates_supported(x, 0)
    loss = torch.zeros(10, 64, dtype=torch.float64, device="cuda")
    with pytest.raises(_cabi.B200QError):
        ops.mse_candidates(x, torch.ones(10, 64, device="cuda"), loss, 0, 8, False, True)
    amax = x.abs().amax(dim=1, keepdim=True)
    fused = {"num_bits": 8, "unsigned": False, "narrow_range": True}
    cal = MseCalibrator(amax, axis=0, quant_func=lambda t, a: ops.fake_int(t, a, 8, False, True), fused=fused)
    cal.collect(x)
    assert cal._loss_buf is None                                   # the candidate loop ran
    assert cal.compute_amax().shape == amax.shape


@pytest.mark.parametrize("cfg_name", ["INT8_DEFAULT_CFG", "FP8_DEFAULT_CFG"])
def test_mse_calibrate_same_amax_with_and_without_the_kernel(cfg_name):
    """mtq.quantize(algorithm="mse") selects the same amax whether every candidate is evaluated in one
    launch or one by one through the quantiser, and the kernel is what runs by default."""
    import b200q as mtq
    from b200q import model_calib
    from b200q.calib import MseCalibrator

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up_proj = torch.nn.Linear(512, 1024, bias=False)
            self.down_proj = torch.nn.Linear(1024, 512, bias=False)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.up_proj(x)))

    torch.manual_seed(0)
    base = MLP().cuda().bfloat16()
    batches = [torch.randn(4, 64, 512, device="cuda").bfloat16() * 2 for _ in range(3)]
    got = []
    for fused in (True, False):
        m = copy.deepcopy(base)
        cfg = copy.deepcopy(getattr(mtq, cfg_name))
        cfg["algorithm"] = "mse"
        used = []
        orig = MseCalibrator.collect

        def spy(self, x, _orig=orig, _fused=fused, _used=used):
            if not _fused:
                self._fused = None
            _orig(self, x)
            _used.append(self._loss_buf is not None)

        MseCalibrator.collect = spy
        try:
            mtq.quantize(m, cfg, lambda mod: [mod(b) for b in batches])
        finally:
            MseCalibrator.collect = orig
        assert used and all(u == fused for u in used), (fused, used)
        got.append({n: q._amax.detach().float().clone() for n, q in m.named_modules()
                    if hasattr(q, "_amax") and q._amax is not None})
    assert got[0].keys() == got[1].keys() and len(got[0]) == 4
    for n in got[0]:
        same = (got[0][n] == got[1][n]).float().mean().item()
        assert same >= 0.98, (n, same)          # a near-tie between two candidates may flip
