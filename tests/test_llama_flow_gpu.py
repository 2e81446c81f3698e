"""End-to-end flow on a small Llama-shaped model (HF module names): quantize -> calibrate ->
compress -> forward -> checkpoint export, for the NVFP4, FP8 and INT4-AWQ configurations."""
import copy

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


class RMSNorm(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))

    def forward(self, x):
        return self.weight * x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, d, heads, kv_heads):
        super().__init__()
        self.h, self.kv, self.hd = heads, kv_heads, d // heads
        self.q_proj = nn.Linear(d, d, bias=False)
        self.k_proj = nn.Linear(d, self.kv * self.hd, bias=False)
        self.v_proj = nn.Linear(d, self.kv * self.hd, bias=False)
        self.o_proj = nn.Linear(d, d, bias=False)

    def forward(self, x):
        b, t, d = x.shape
        q = self.q_proj(x).view(b, t, self.h, self.hd).transpose(1, 2)
        k = self.k_proj(x).view(b, t, self.kv, self.hd).transpose(1, 2).repeat_interleave(self.h // self.kv, 1)
        v = self.v_proj(x).view(b, t, self.kv, self.hd).transpose(1, 2).repeat_interleave(self.h // self.kv, 1)
        y = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(y.transpose(1, 2).reshape(b, t, d))


class MLP(nn.Module):
    def __init__(self, d, inter):
        super().__init__()
        self.gate_proj = nn.Linear(d, inter, bias=False)
        self.up_proj = nn.Linear(d, inter, bias=False)
        self.down_proj = nn.Linear(inter, d, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class Layer(nn.Module):
    def __init__(self, d, heads, kv_heads, inter):
        super().__init__()
        self.input_layernorm, self.post_attention_layernorm = RMSNorm(d), RMSNorm(d)
        self.self_attn, self.mlp = Attention(d, heads, kv_heads), MLP(d, inter)

    def forward(self, x):
        x = x + self.self_attn(self.input_layernorm(x))
        return x + self.mlp(self.post_attention_layernorm(x))


class TinyLlama(nn.Module):
    def __init__(self, vocab=512, d=256, heads=4, kv_heads=2, inter=512, layers=2):
        super().__init__()
        self.embed_tokens = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(Layer(d, heads, kv_heads, inter) for _ in range(layers))
        self.norm = RMSNorm(d)
        self.lm_head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids):
        x = self.embed_tokens(ids)
        for layer in self.layers:
            x = layer(x)
        return self.lm_head(self.norm(x))


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG", "INT4_AWQ_CFG"])
def test_llama_shaped_model_end_to_end(name):
    import b200q as mtq
    from b200q import export
    from b200q.nn import QuantLinear

    torch.manual_seed(0)
    model = TinyLlama().to(torch.bfloat16).cuda().eval()
    g = torch.Generator(device="cuda").manual_seed(1)
    batches = [torch.randint(0, 512, (4, 128), device="cuda", generator=g) for _ in range(2)]
    with torch.no_grad():
        ref = model(batches[0]).float()

    def loop(m):
        with torch.no_grad():
            for b in batches:
                m(b)

    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), loop)
    linears = {n: m for n, m in model.named_modules() if isinstance(m, QuantLinear)}
    assert len(linears) == 2 * 7 + 1
    assert not linears["lm_head"].weight_quantizer.is_enabled            # "*lm_head*" is excluded by the configs
    enabled = [n for n, m in linears.items() if m.weight_quantizer.is_enabled]
    assert len(enabled) == 14
    with torch.no_grad():
        fake = model(batches[0]).float()
    rel = (fake - ref).abs().mean() / ref.abs().mean()
    assert torch.isfinite(fake).all() and rel < (0.5 if name == "INT4_AWQ_CFG" else 0.35), float(rel)
    mtq.compress(model)
    with torch.no_grad():
        real = model(batches[0]).float()
    assert torch.isfinite(real).all()
    assert (real - fake).abs().mean() < 0.1 * fake.abs().mean() + 1e-3
    w = model.layers[0].mlp.up_proj.weight
    if name != "FP8_DEFAULT_CFG":
        assert w.dtype == torch.uint8 and w.shape == (512, 128)            # two 4-bit values per byte
    else:
        assert w.dtype == torch.float8_e4m3fn


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG"])
def test_llama_shaped_checkpoint_export(name):
    import b200q as mtq
    from b200q import export

    torch.manual_seed(0)
    model = TinyLlama().to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (2, 64), device="cuda")
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    sd = export.export_hf_state_dict(model, torch.bfloat16)
    assert "lm_head.weight" in sd and sd["lm_head.weight"].dtype == torch.bfloat16
    assert not any("quantizer" in k for k in sd)
    for layer in range(2):
        for lin in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                    "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
            p = f"layers.{layer}.{lin}."
            assert sd[p + "weight_scale"].numel() > 0 and sd[p + "input_scale"].numel() == 1
            if name == "NVFP4_DEFAULT_CFG":
                assert sd[p + "weight"].dtype == torch.uint8 and sd[p + "weight_scale"].dtype == torch.float8_e4m3fn
                assert sd[p + "weight_scale_2"].dtype == torch.float32
            else:
                assert sd[p + "weight"].dtype == torch.float8_e4m3fn


@pytest.mark.parametrize("name,do_compress", [("NVFP4_DEFAULT_CFG", True), ("INT4_AWQ_CFG", True),
                                              ("W4A8_AWQ_BETA_CFG", False), ("FP8_DEFAULT_CFG", False),
                                              ("INT8_SMOOTHQUANT_CFG", False)])
def test_save_and_restore_quantized_model(name, do_compress, tmp_path):
    """Checkpoint / resume: state_dict + modelopt_state of a quantised (and compressed) model,
    written to disk, restore a freshly constructed model to the same outputs."""
    import b200q as mtq
    from b200q.qtensor import QTensorWrapper

    torch.manual_seed(0)
    model = TinyLlama().to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (2, 64), device="cuda")
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    if do_compress:
        mtq.compress(model)
    with torch.no_grad():
        want = model(ids)
    torch.save({"model": model.state_dict(), "modelopt": mtq.modelopt_state(model)}, tmp_path / "ckpt.pt")

    ckpt = torch.load(tmp_path / "ckpt.pt", weights_only=False)
    torch.manual_seed(123)                                   # different initial weights
    fresh = TinyLlama().to(torch.bfloat16).cuda().eval()
    mtq.restore_from_modelopt_state(fresh, ckpt["modelopt"])
    missing, unexpected = fresh.load_state_dict(ckpt["model"], strict=True)
    assert not missing and not unexpected
    if do_compress:
        assert isinstance(fresh.layers[0].mlp.up_proj.weight, QTensorWrapper)
    with torch.no_grad():
        got = fresh(ids)
    assert torch.equal(got, want)
    assert [m for m, _ in mtq.modelopt_state(fresh)["modelopt_state_dict"]] == \
           [m for m, _ in ckpt["modelopt"]["modelopt_state_dict"]]


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG"])
def test_llama_shaped_model_runs_on_real_quant_gemms(name):
    """quantize -> compress -> enable_real_quant_gemm: every projection runs the tensor-core GEMM on
    the packed weight, and the logits stay close to the dequantise-then-bf16 path."""
    import b200q as mtq
    from b200q import backends, ops
    from b200q.nn import RealQuantLinear

    torch.manual_seed(0)
    model = TinyLlama().to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (4, 128), device="cuda")
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    mtq.compress(model)
    with torch.no_grad():
        want = model(ids).float()
    backends.enable_real_quant_gemm(model)
    with torch.no_grad():
        got = model(ids).float()
    ops.check_qgemm_status("cuda")
    layers = [m for m in model.modules() if isinstance(m, RealQuantLinear)]
    used = [m for m in layers if getattr(m, "_real_quant_gemm_impl", None) is not None]
    assert len(layers) == 14 and len(used) == 14          # 2 x (q, k, v, o, gate, up, down); lm_head is not quantised
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert cos > 0.999, cos
    assert (got - want).abs().max() <= 0.05 * want.abs().max()


def _nvfp4_weight_only_tree(n_layers, device, dtype=torch.bfloat16):
    """A Llama-shaped tree of linears (scaled-down dims, real names) with NVFP4 weight quantisers."""
    import b200q as mtq

    dims = {"q_proj": (256, 256), "k_proj": (64, 256), "v_proj": (64, 256), "o_proj": (256, 256),
            "gate_proj": (896, 256), "up_proj": (896, 256), "down_proj": (256, 896)}
    g = torch.Generator().manual_seed(0)
    layers = torch.nn.ModuleList()
    for _ in range(n_layers):
        layer = torch.nn.ModuleDict()
        for name, (n, k) in dims.items():
            lin = torch.nn.Linear(k, n, bias=False)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(n, k, generator=g) * 0.02)
            layer[name] = lin
        layers.append(layer)
    model = torch.nn.ModuleDict({"layers": layers}).to(device=device, dtype=dtype)
    mtq.replace_quant_module(model)
    mtq.set_quantizer_by_cfg(model, {"*weight_quantizer": {"num_bits": (2, 1), "block_sizes": {-1: 16, "type": "dynamic", "scale_bits": (4, 3)}, "axis": None, "enable": True},
                                     "*input_quantizer": {"enable": False}, "default": {"enable": False}})
    return model


@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_compress_packs_nvfp4_weights_with_the_grouped_kernels(where, monkeypatch):
    """mtq.compress on a Llama-shaped tree: all NVFP4 weights of a device go through ONE grouped abs-max
    launch and ONE grouped quantise launch (a host-resident model is streamed through the GPU instead),
    and every packed weight, block scale and global scale equals what the per-weight path
    (``NVFP4QTensor.quantize``, oracle-checked elsewhere) produces; a calibrated, clipped weight amax is
    honoured."""
    import b200q as mtq
    from b200q import ops
    from b200q.qtensor import NVFP4QTensor

    model = _nvfp4_weight_only_tree(2, where)
    originals = {n: m.weight.detach().clone().cuda() for n, m in model.named_modules() if hasattr(m, "weight_quantizer")}
    assert len(originals) == 14
    clipped = "layers.1.down_proj"
    wq = dict(model.named_modules())[clipped].weight_quantizer
    wq.amax = (originals[clipped].float().abs().max() * 0.7).to(where)
    launches = []
    real = ops.NvFp4Group.run
    monkeypatch.setattr(ops.NvFp4Group, "run", lambda self, *a, **k: (launches.append(self.n), real(self, *a, **k))[1])
    mtq.compress(model)
    torch.cuda.synchronize()
    if where == "cuda":
        assert launches == [14], "one grouped pass for all fourteen weights"
    else:
        assert sum(launches) == 14 and len(launches) <= 8
    for name, w in originals.items():
        m = dict(model.named_modules())[name]
        assert m.weight.dtype == torch.uint8 and m.weight.device.type == where
        s2 = None
        if name == clipped:
            s2 = NVFP4QTensor.get_weights_scaling_factor_2_from_quantizer(type("Q", (), {"_amax": wq._amax.cuda()}))
        q, sc, d = NVFP4QTensor.quantize(w, 16, weights_scaling_factor_2=s2)
        assert torch.equal(m.weight.data.cuda(), q._quantized_data), name
        assert torch.equal(m.weight_quantizer._scale.view(torch.uint8).cuda(), sc.view(torch.uint8)), name
        assert m.weight_quantizer._double_scale.item() == d.item(), name
    if where == "cuda":
        x = torch.randn(8, 256, device="cuda", dtype=torch.bfloat16)
        y = model["layers"][0]["q_proj"](x)
        assert torch.isfinite(y).all()
