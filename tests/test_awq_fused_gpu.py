"""The fused all-candidates awq_lite search kernel (CTA pairs, weight-side producer in shared memory)
against the two-kernel evaluation it replaces.

Products: against a float32 torch matmul of the same bf16 operands (the fake-quantised weight taken
from the stand-alone scale + quantise kernel, which is oracle-checked elsewhere), tolerance 1e-5
relative to the largest product: only the fp32 accumulation order differs.  Losses: against the same
formula in torch on the kernel's own products (1e-6) and against the unfused tensor-core kernel
(1e-3, the tolerance of the AWQ losses: bf16 roundings of the product flip with the summation order).
"""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n_alpha, m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).bfloat16()
    x = (torch.randn(m, k, generator=g, device="cuda") * torch.exp(torch.randn(k, generator=g, device="cuda"))).bfloat16()
    s = torch.exp(0.5 * torch.randn(n_alpha, k, generator=g, device="cuda"))
    w_s, x_s = s.bfloat16(), (1 / s).bfloat16()
    a_all = x.unsqueeze(0) * x_s.unsqueeze(1)
    ref = (x.float() @ w.float().T).bfloat16()
    return w, a_all, w_s, ref


@pytest.mark.parametrize("n_alpha,m,n,k", [
    (1, 128, 256, 128),        # one item, one W unit, rows of the odd CTA all beyond m
    (3, 256, 256, 256),        # one 256-row MMA per item
    (2, 512, 512, 1024),       # two 256-row MMAs per item, ring wrap-around (16 K slices)
    (3, 300, 288, 384),        # ragged rows and a ragged column slab
    (5, 1024, 1024, 512),      # two row slabs; 40 items
    (2, 48, 64, 128),          # fewer rows than one tile
])
def test_fused_search_products_and_losses(n_alpha, m, n, k):
    from b200q import ops

    w, a_all, w_s, ref = _case(n_alpha, m, n, k, seed=m + n + k)
    loss = torch.zeros(n_alpha, dtype=torch.float64, device="cuda")
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    c = torch.full((n_alpha, m, n), float("nan"), device="cuda")
    assert ops.awq_search_fused_supported(a_all[0], w, 128)
    ops.awq_search_fused(a_all, w, w_s, ref, loss, status, c_out=c)
    torch.cuda.synchronize()
    assert status.item() == 0, f"a bounded wait ran out: status {status.item():#x}"
    for a in range(n_alpha):
        wfq = ops.awq_scale_fake_int(w, w_s[a], 128, 4, False, False)
        want = a_all[a].float() @ wfq.float().T
        assert torch.allclose(c[a], want, rtol=1e-5, atol=1e-5 * float(want.abs().max())), a
        d = (c[a].bfloat16() - ref).float()
        want_loss = (d * d).sum().item()
        assert abs(loss[a].item() - want_loss) <= 1e-6 * want_loss, (a, loss[a].item(), want_loss)
    # accumulates into the same words, and a second launch finds every barrier and TMEM column free
    ops.awq_search_fused(a_all, w, w_s, ref, loss, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    d = (c.bfloat16() - ref).float()
    assert torch.allclose(loss, 2 * (d * d).sum(dim=(1, 2)).double(), rtol=1e-6)


def test_fused_search_blocks_outside_the_fast_path():
    """Blocks the in-kernel transform cannot handle with its verified-reciprocal multiply take the
    element-wise exact path: all-zero blocks (dead abs-max), blocks so small that 7 / amax leaves the
    safe division range, and both next to ordinary blocks in one warp."""
    from b200q import ops

    n_alpha, m, n, k = 2, 128, 256, 512
    w, a_all, w_s, ref = _case(n_alpha, m, n, k, seed=77)
    w = w.clone()
    w[3, 128:256] = 0                       # a dead block
    w[4:20, 0:128] = 0                      # dead blocks in every lane pair of a warp's first half
    w[40, 256:384] *= 1e-30                 # 7 / amax beyond 2^40
    w[41, 256:384] = (w[41, 256:384].float() * 1e-36).bfloat16()
    w[200:, :] = 0                          # the odd CTA's rows: everything dead
    loss = torch.zeros(n_alpha, dtype=torch.float64, device="cuda")
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    c = torch.full((n_alpha, m, n), float("nan"), device="cuda")
    ops.awq_search_fused(a_all, w, w_s, ref, loss, status, c_out=c)
    torch.cuda.synchronize()
    assert status.item() == 0
    for a in range(n_alpha):
        wfq = ops.awq_scale_fake_int(w, w_s[a], 128, 4, False, False)
        want = a_all[a].float() @ wfq.float().T
        assert torch.allclose(c[a], want, rtol=1e-5, atol=1e-5 * float(want.abs().max())), a
    assert float(c[:, :, 200:].abs().max()) == 0.0


def test_fused_search_many_items_per_pair_against_the_unfused_kernel():
    """More items than CTA pairs (every pair loops), long K: losses of all candidates against the
    two-kernel path, and bit-identical losses from run to run are not required (atomics) but 1e-12 is."""
    from b200q import ops

    n_alpha, m, n, k = 7, 512, 4096, 2048
    w, a_all, w_s, ref = _case(n_alpha, m, n, k, seed=9)
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    runs = []
    for _ in range(2):
        loss = torch.zeros(n_alpha, dtype=torch.float64, device="cuda")
        ops.awq_search_fused(a_all, w, w_s, ref, loss, status)
        runs.append(loss)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.allclose(runs[0], runs[1], rtol=1e-12)
    for a in range(n_alpha):
        wfq = ops.awq_scale_fake_int(w, w_s[a], 128, 4, False, False)
        acc = torch.zeros((), dtype=torch.float64, device="cuda")
        ops.awq_gemm_sqerr(a_all[a], wfq, ref, acc, status, splits=1)
        assert abs(runs[0][a].item() - acc.item()) <= 1e-3 * acc.item(), a
    assert status.item() == 0


def test_fused_search_refuses_what_it_does_not_cover():
    from b200q import _cabi, ops

    w, a_all, w_s, ref = _case(1, 128, 256, 128, seed=1)
    loss = torch.zeros(1, dtype=torch.float64, device="cuda")
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    with pytest.raises(_cabi.B200QError):
        ops.awq_search_fused(a_all, w, w_s, ref, loss, status, block=64)
    assert not ops.awq_search_fused_supported(a_all[0], w, 64)
    assert not ops.awq_search_fused_supported(a_all[0].float(), w, 128)
    assert not ops.awq_search_fused_supported(a_all[0][:, :64], w[:, :64], 128)


def test_awq_lite_same_selection_with_the_fused_search():
    """mtq.quantize(INT4_AWQ_CFG) picks the same alpha and scales, and reports losses within 1e-3,
    whether the candidates are evaluated by the fused kernel or by the two-kernel pipeline."""
    import b200q as mtq
    from b200q import model_calib

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up_proj = torch.nn.Linear(256, 512, bias=False)
            self.down_proj = torch.nn.Linear(512, 256, bias=False)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.up_proj(x)))

    torch.manual_seed(0)
    base = MLP().cuda().bfloat16()
    g = torch.Generator(device="cuda").manual_seed(1)
    mag = torch.exp(torch.randn(256, generator=g, device="cuda"))
    batches = [(torch.randn(256, 256, generator=g, device="cuda") * mag).bfloat16() for _ in range(2)]
    results = []
    for use in (True, False):
        model_calib.FUSED_AWQ_SEARCH = use
        try:
            m = copy.deepcopy(base)
            cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
            cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.1, "debug": True}
            mtq.quantize(m, cfg, lambda mod: [mod(b) for b in batches])
            results.append({n: (getattr(m, n).awq_lite.loss, getattr(m, n).awq_lite.best_alpha,
                                getattr(m, n).awq_lite.best_scale, getattr(m, n).weight.detach().clone())
                            for n in ("up_proj", "down_proj")})
        finally:
            model_calib.FUSED_AWQ_SEARCH = True
    for n in ("up_proj", "down_proj"):
        la, aa, sa, wa = results[0][n]
        lb, ab, sb, wb = results[1][n]
        for key in la:
            assert abs(la[key] - lb[key]) <= 1e-3 * lb[key], (n, key, la[key], lb[key])
        assert aa == ab and torch.equal(sa, sb) and torch.equal(wa, wb)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_awq_scale_acts_equals_the_broadcast_multiply(dtype):
    from b200q import ops

    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(300, 1024, generator=g, device="cuda") * 3).to(dtype)
    s = torch.exp(torch.randn(5, 1024, generator=g, device="cuda")).to(dtype)
    got = ops.awq_scale_acts(x, s)
    assert torch.equal(got, x.unsqueeze(0) * s.unsqueeze(1))


@pytest.mark.parametrize("n_alpha,m,n,k", [
    (1, 512, 1024, 512),       # one GEMM with the loss epilogue
    (3, 1024, 512, 256),       # two row slabs per candidate
    (2, 1300, 288, 384),       # ragged rows (three slabs, the last mostly empty) and a ragged column slab
    (4, 100, 96, 128),         # small everything
])
def test_pair_kernel_on_finished_weights(n_alpha, m, n, k):
    """b200q_awq_search_prequant: the CTA-pair kernel handed every candidate's weight already scaled and
    fake-quantised.  Products against a float32 torch matmul of the same bf16 operands (1e-5 of the
    largest product: summation order only), losses against the formula on the kernel's own products (1e-6)
    and against the stand-alone tensor-core kernel (1e-3)."""
    from b200q import ops

    w, a_all, w_s, ref = _case(n_alpha, m, n, k, seed=7 * m + n)
    wq_all = torch.stack([ops.awq_scale_fake_int(w, w_s[a], 128, 4, False, False) for a in range(n_alpha)])
    assert ops.awq_search_prequant_supported(a_all[0], w)
    loss = torch.zeros(n_alpha, dtype=torch.float64, device="cuda")
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    c = torch.full((n_alpha, m, n), float("nan"), device="cuda")
    ops.awq_search_prequant(a_all, wq_all, ref, loss, status, c_out=c)
    torch.cuda.synchronize()
    assert status.item() == 0
    for a in range(n_alpha):
        want = a_all[a].float() @ wq_all[a].float().T
        assert torch.allclose(c[a], want, rtol=1e-5, atol=1e-5 * float(want.abs().max())), a
        d = (c[a].bfloat16() - ref).float()
        want_loss = (d * d).sum().item()
        assert abs(loss[a].item() - want_loss) <= 1e-6 * want_loss
        if m % 128 == 0 and n % 128 == 0 and k % 64 == 0:
            acc = torch.zeros((), dtype=torch.float64, device="cuda")
            ops.awq_gemm_sqerr(a_all[a], wq_all[a], ref, acc, status, splits=1)
            assert abs(loss[a].item() - acc.item()) <= 1e-3 * acc.item()
    # the fused form on the raw weight gives the same losses
    loss2 = torch.zeros(n_alpha, dtype=torch.float64, device="cuda")
    ops.awq_search_fused(a_all, w, w_s, ref, loss2, status)
    assert status.item() == 0
    assert torch.allclose(loss, loss2, rtol=1e-6)


def test_awq_lite_with_a_large_batch_takes_the_finished_weight_path(monkeypatch):
    """A calibration batch of 2304 tokens (more than FUSED_AWQ_SEARCH_MAX_ROWS): the search writes each
    candidate's weight once and runs the pair kernel on the finished weights; same alpha, scales and
    folded weights as the two-kernel pipeline."""
    import b200q as mtq
    from b200q import model_calib, ops

    torch.manual_seed(0)
    base = torch.nn.Sequential(torch.nn.Linear(256, 512, bias=False)).cuda().bfloat16()
    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn(2304, 256, generator=g, device="cuda") * torch.exp(torch.randn(256, generator=g, device="cuda"))).bfloat16()
    calls = []
    real = ops.awq_search_prequant
    monkeypatch.setattr(ops, "awq_search_prequant", lambda *a, **k: (calls.append(a[0].shape), real(*a, **k))[1])
    results = []
    for use in (True, False):
        model_calib.FUSED_AWQ_SEARCH = use
        try:
            m = copy.deepcopy(base)
            cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
            cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.1, "debug": True}
            mtq.quantize(m, cfg, lambda mod: mod(x))
            results.append((m[0].awq_lite.loss, m[0].awq_lite.best_alpha, m[0].awq_lite.best_scale, m[0].weight.detach().clone()))
        finally:
            model_calib.FUSED_AWQ_SEARCH = True
    assert calls and calls[0][1:] == (2304, 256)
    assert not model_calib._SEARCH_SCRATCH
    (la, aa, sa, wa), (lb, ab, sb, wb) = results
    for key in la:
        assert abs(la[key] - lb[key]) <= 1e-3 * lb[key], (key, la[key], lb[key])
    assert aa == ab and torch.equal(sa, sb) and torch.equal(wa, wb)
