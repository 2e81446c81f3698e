"""The tcgen05 evaluation GEMM of awq_lite against a float32 torch matmul of the same bf16 data
(tolerance 1e-5 relative on the product: only the fp32 accumulation order differs) and the fused
squared-error reduction against the same formula in torch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 256), (256, 384, 512), (512, 1024, 4096)])
def test_awq_gemm_product_and_loss(m, n, k):
    from b200q import ops

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g, device="cuda").bfloat16()
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.05).bfloat16()
    ref = (a.float() @ b.float().T + 0.01 * torch.randn(m, n, generator=g, device="cuda")).bfloat16()
    acc = torch.zeros((), dtype=torch.float64, device="cuda")
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    c = torch.full((m, n), float("nan"), device="cuda")
    assert ops.awq_gemm_supported(a, b)
    ops.awq_gemm_sqerr(a, b, ref, acc, status, c_out=c)
    torch.cuda.synchronize()
    assert status.item() == 0, f"a bounded wait ran out: status {status.item()}"
    want = a.float() @ b.float().T
    assert torch.allclose(c, want, rtol=1e-5, atol=1e-5 * float(want.abs().max()))
    d = (c.bfloat16() - ref).float()
    loss = (d * d).sum().item()
    assert abs(acc.item() - loss) <= 1e-6 * loss
    # accumulates into the same word
    ops.awq_gemm_sqerr(a, b, ref, acc, status)
    torch.cuda.synchronize()
    assert abs(acc.item() - 2 * loss) <= 1e-6 * loss and status.item() == 0


def test_awq_gemm_unsupported_shapes_are_refused():
    from b200q import _cabi, ops

    a = torch.zeros(100, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    assert not ops.awq_gemm_supported(a, b)
    with pytest.raises(_cabi.B200QError):
        ops.awq_gemm_sqerr(a, b, torch.zeros(100, 128, device="cuda", dtype=torch.bfloat16),
                           torch.zeros((), dtype=torch.float64, device="cuda"),
                           torch.zeros((), dtype=torch.int32, device="cuda"))


def test_awq_lite_search_same_result_with_and_without_tensor_core_kernel():
    """The search picks the same alpha and scales whether candidates are evaluated by the fused
    tcgen05 kernel or by F.linear + the squared-error kernel (losses agree to 1e-3)."""
    import copy

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
        model_calib.USE_TENSOR_CORE_EVAL = use
        try:
            m = copy.deepcopy(base)
            cfg = copy.deepcopy(mtq.INT4_AWQ_CFG)
            cfg["algorithm"] = {"method": "awq_lite", "alpha_step": 0.1, "debug": True}
            mtq.quantize(m, cfg, lambda mod: [mod(b) for b in batches])
            results.append({n: (getattr(m, n).awq_lite.loss, getattr(m, n).awq_lite.best_alpha,
                                getattr(m, n).awq_lite.best_scale) for n in ("up_proj", "down_proj")})
        finally:
            model_calib.USE_TENSOR_CORE_EVAL = True
    for n in ("up_proj", "down_proj"):
        la, aa, sa = results[0][n]
        lb, ab, sb = results[1][n]
        for k in la:
            assert abs(la[k] - lb[k]) <= 1e-3 * lb[k], (n, k, la[k], lb[k])
        assert aa == ab and torch.equal(sa, sb)


@pytest.mark.parametrize("m,n,k,splits", [(128, 128, 256, 2), (256, 384, 1024, 4), (512, 512, 4096 + 64, 3),
                                          (512, 4096, 14336, None)])
def test_awq_gemm_split_k_matches_unsplit(m, n, k, splits):
    """Split-K: partial tiles summed in split order by the last CTA of a tile.  Same product to fp32
    summation order, loss within the 1e-3 of the AWQ losses (bf16 roundings of the product flip with
    the summation order), bit-identical from run to run, counters left at zero."""
    from b200q import ops

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g, device="cuda").bfloat16()
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.05).bfloat16()
    ref = (a.float() @ b.float().T + 0.01 * torch.randn(m, n, generator=g, device="cuda")).bfloat16()
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    if splits is None:
        splits = ops.awq_gemm_splits(m, n, k, a.device)
        assert splits >= 2                               # the down-projection shape is split by default
    outs = []
    for s in (1, splits, splits):
        acc = torch.zeros((), dtype=torch.float64, device="cuda")
        c = torch.full((m, n), float("nan"), device="cuda")
        ops.awq_gemm_sqerr(a, b, ref, acc, status, c_out=c, splits=s)
        torch.cuda.synchronize()
        assert status.item() == 0
        outs.append((c, acc.item()))
    (c1, l1), (c2, l2), (c3, l3) = outs
    assert torch.allclose(c2, c1, rtol=1e-5, atol=1e-5 * float(c1.abs().max()))
    assert abs(l2 - l1) <= 1e-3 * l1
    assert torch.equal(c2, c3) and l2 == l3 or abs(l2 - l3) <= 1e-12 * l2   # the sum order inside a tile is fixed
    for key, (_, counters) in ops._SPLITK_SCRATCH.items():
        assert int(counters.abs().sum()) == 0
