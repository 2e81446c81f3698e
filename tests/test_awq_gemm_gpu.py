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
