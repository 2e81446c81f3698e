"""The quantize -> compress flow on a Hugging Face ``LlamaForCausalLM`` (random weights, a small
configuration built in memory: nothing is downloaded): the module tree the reference's LLM PTQ examples
hand to ``mtq.quantize``.  Every ``nn.Linear`` of the decoder becomes a quantised linear layer, ``lm_head``
stays unquantised (the configurations' ``*lm_head*`` rule), calibration sees the model's own forward, and
the compressed model still produces logits close to the fake-quantised one."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

transformers = pytest.importorskip("transformers")


def _tiny_llama(seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(seed)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                      tie_word_embeddings=False)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG", "INT4_AWQ_CFG", "INT8_SMOOTHQUANT_CFG"])
def test_quantize_and_compress_a_hugging_face_llama(name):
    import b200q as mtq
    from b200q.nn import QuantLinear, RealQuantLinear
    from b200q.qtensor import QTensorWrapper

    model = _tiny_llama()
    g = torch.Generator(device="cuda").manual_seed(1)
    batches = [torch.randint(0, 512, (2, 64), generator=g, device="cuda") for _ in range(3)]
    with torch.no_grad():
        plain = model(batches[0]).logits.float()

    def loop(m):
        with torch.no_grad():
            for ids in batches:
                m(ids)

    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), loop)
    linears = {n: m for n, m in model.named_modules() if isinstance(m, torch.nn.Linear)}
    assert len(linears) == 2 * 7 + 1
    for n, m in linears.items():
        assert isinstance(m, QuantLinear), n
        assert m.weight_quantizer.is_enabled == ("lm_head" not in n), n
        if "lm_head" not in n:
            assert m.weight_quantizer.amax is not None or m.weight_quantizer.is_mx_format, n
    with torch.no_grad():
        fake = model(batches[0]).logits.float()
    assert torch.isfinite(fake).all()
    cos = torch.nn.functional.cosine_similarity(fake.flatten(), plain.flatten(), dim=0)
    assert cos > (0.92 if "4" in name else 0.99), float(cos)       # 4-bit weights (and activations): coarse

    mtq.compress(model)
    packed = [n for n, m in linears.items() if isinstance(m.weight, QTensorWrapper)]
    assert len(packed) == 2 * 7 and all(isinstance(linears[n], RealQuantLinear) for n in packed)
    with torch.no_grad():
        real = model(batches[0]).logits.float()
    assert torch.isfinite(real).all()
    cos = torch.nn.functional.cosine_similarity(real.flatten(), fake.flatten(), dim=0)
    assert cos > 0.99, float(cos)
    state = mtq.modelopt_state(model)
    fresh = _tiny_llama(seed=5)
    mtq.restore_from_modelopt_state(fresh, state)
    fresh.load_state_dict(model.state_dict())
    with torch.no_grad():
        assert torch.equal(fresh(batches[0]).logits, model(batches[0]).logits)


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG", "INT4_AWQ_CFG"])
def test_export_a_hugging_face_llama_with_its_shared_input_layers_made_fusable(name):
    """``export_hf_state_dict`` on the Hugging Face module tree (reference unified_export_hf.py:90-232, 233-392):
    q / k / v and gate / up read one tensor each and leave with common scales; with AWQ their averaged pre-quant
    scale moves into the RMSNorm in front of them (o_proj and down_proj keep theirs), and the model still
    computes what it computed before the layers were re-smoothed."""
    import b200q as mtq
    from b200q import export

    model = _tiny_llama()
    g = torch.Generator(device="cuda").manual_seed(1)
    batches = [torch.randint(0, 512, (2, 64), generator=g, device="cuda") for _ in range(3)]

    def loop(m):
        with torch.no_grad():
            for ids in batches:
                m(ids)

    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), loop)
    with torch.no_grad():
        before = model(batches[0]).logits.float()
    norm_before = model.model.layers[0].input_layernorm.weight.clone()
    fused = export.requantize_resmooth_fused_llm_layers(copy.deepcopy(model))
    if name == "FP8_DEFAULT_CFG":
        assert fused == {}
    else:
        assert fused == {f"model.layers.{i}.{first}": [f"model.layers.{i}.{first.split('.')[0]}.{p}" for p in group]
                         for i in range(2) for first, group in (("self_attn.q_proj", ("q_proj", "k_proj", "v_proj")),
                                                                ("mlp.gate_proj", ("gate_proj", "up_proj")))}
    if name == "INT4_AWQ_CFG":
        probe = copy.deepcopy(model)
        export.requantize_resmooth_fused_llm_layers(probe)
        with torch.no_grad():
            after = probe(batches[0]).logits.float()
        cos = torch.nn.functional.cosine_similarity(after.flatten(), before.flatten(), dim=0)
        assert cos > 0.98, float(cos)             # the groups leave their own best scale for the average: 4-bit rounding moves
    sd = export.export_hf_state_dict(model, torch.bfloat16)
    attn, mlp = "model.layers.0.self_attn.", "model.layers.0.mlp."
    if name == "NVFP4_DEFAULT_CFG":
        for key in ("input_scale", "weight_scale_2"):
            assert torch.equal(sd[attn + "q_proj." + key], sd[attn + "k_proj." + key])
            assert torch.equal(sd[attn + "q_proj." + key], sd[attn + "v_proj." + key])
            assert torch.equal(sd[mlp + "gate_proj." + key], sd[mlp + "up_proj." + key])
        assert sd[attn + "q_proj.weight"].dtype == torch.uint8
    if name == "INT4_AWQ_CFG":
        for layer in ("q_proj", "k_proj", "v_proj"):
            assert attn + layer + ".pre_quant_scale" not in sd
        assert attn + "o_proj.pre_quant_scale" in sd and mlp + "down_proj.pre_quant_scale" in sd
        assert not torch.equal(sd["model.layers.0.input_layernorm.weight"], norm_before)
    assert not any("_amax" in k or "quantizer" in k for k in sd)


@pytest.mark.parametrize("name", ["NVFP4_DEFAULT_CFG", "FP8_DEFAULT_CFG"])
def test_export_hf_checkpoint_writes_tensors_record_and_config(name, tmp_path):
    """Reference modelopt/torch/export/unified_export_hf.py:556-615: the directory holds the packed tensors
    (read back bit for bit), ``hf_quant_config.json`` and a ``config.json`` that carries the record."""
    import json

    from safetensors import safe_open

    import b200q as mtq
    from b200q import export

    model = _tiny_llama()
    ids = torch.randint(0, 512, (2, 64), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    state, record = export.export_hf_checkpoint(model, torch.bfloat16, tmp_path)
    algorithm = "NVFP4" if "NVFP4" in name else "FP8"
    assert record["quantization"]["quant_algo"] == algorithm
    assert record["quantization"]["exclude_modules"] == ["lm_head"]
    assert json.loads((tmp_path / "hf_quant_config.json").read_text()) == record
    config = json.loads((tmp_path / "config.json").read_text())
    assert config["quantization_config"]["quant_algo"] == algorithm
    assert config["quantization_config"]["ignore"] == ["lm_head"]
    files = sorted(p.name for p in tmp_path.glob("*.safetensors"))
    assert files
    seen = {}
    for f in files:
        with safe_open(str(tmp_path / f), framework="pt") as reader:
            for key in reader.keys():
                seen[key] = reader.get_tensor(key)
    assert set(seen) == set(state)
    key = "model.layers.0.self_attn.q_proj.weight"
    assert seen[key].dtype == (torch.uint8 if algorithm == "NVFP4" else torch.float8_e4m3fn)
    for k, v in state.items():
        assert torch.equal(seen[k].view(torch.uint8) if v.element_size() == 1 else seen[k],
                           v.cpu().view(torch.uint8) if v.element_size() == 1 else v.cpu()), k


@pytest.mark.parametrize("name", ["INT4_AWQ_CFG", "NVFP4_AWQ_LITE_CFG"])
@pytest.mark.parametrize("heads", [(4, 4), (4, 2), (4, 1)])      # MHA, GQA, MQA
def test_pattern_fuse_prequant(name, heads):
    """Reference tests/gpu/torch/export/test_quant_utils.py:41-101: the pre-quant scales of o_proj and down_proj
    move into v_proj and up_proj (averaged over the query heads of a key / value head first); the layers that
    gave them up are marked, and the logits stay within the reference test's tolerance."""
    from transformers import LlamaConfig, LlamaForCausalLM

    import b200q as mtq
    from b200q import export

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=heads[0],
                      num_key_value_heads=heads[1], max_position_embeddings=128, vocab_size=256)
    model = LlamaForCausalLM(cfg).cuda().eval()
    ids = torch.randint(0, 256, (1, 16), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    with torch.no_grad():
        before = model(ids).logits
    export.fuse_prequant_to_linear(model, fuse_grouped_heads=True)
    for target in ("model.layers.0.self_attn.o_proj", "model.layers.0.mlp.down_proj",
                   "model.layers.1.self_attn.o_proj", "model.layers.1.mlp.down_proj"):
        layer = model.get_submodule(target)
        assert not hasattr(layer.input_quantizer, "_pre_quant_scale"), target
        assert getattr(layer, "fused_with_prequant", False), target
    with torch.no_grad():
        after = model(ids).logits
    assert torch.allclose(before, after, rtol=1e-1, atol=5e-1)


@pytest.mark.parametrize(("name", "fused"), [
    ("FP8_DEFAULT_CFG", True), ("NVFP4_DEFAULT_CFG", True), ("NVFP4_AWQ_LITE_CFG", True), ("INT4_AWQ_CFG", True),
    ("W4A8_AWQ_BETA_CFG", True), ("INT8_WEIGHT_ONLY_CFG", False)])
def test_exported_safetensors_share_scales_across_fused_projections(name, fused, tmp_path):
    """Reference tests/gpu/torch/export/test_unified_hf_export_and_check_safetensors.py:24-131 without the
    example script around it: a small Llama is quantised with each format, exported, and the safetensors are
    read back: gate / up and q / k / v agree on ``input_scale``, ``weight_scale_2`` and ``prequant_scale``."""
    from safetensors import safe_open

    import b200q as mtq
    from b200q import export

    model = _tiny_llama()
    ids = torch.randint(0, 512, (2, 64), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(ids))
    export.export_hf_checkpoint(model, torch.bfloat16, tmp_path)
    files = sorted(tmp_path.glob("*.safetensors"))
    assert files
    tensors = {}
    for f in files:
        with safe_open(str(f), framework="pt") as reader:
            for key in reader.keys():
                tensors[key] = reader.get_tensor(key)
    assert tensors
    checked = 0
    for key, value in tensors.items():
        if not (fused and key.endswith(("input_scale", "weight_scale_2", "prequant_scale"))):
            continue
        for first, second in (("gate_proj", "up_proj"), ("q_proj", "k_proj"), ("q_proj", "v_proj")):
            if first in key:
                assert torch.allclose(value.float(), tensors[key.replace(first, second)].float()), key
                checked += 1
    if fused and name != "INT4_AWQ_CFG":      # INT4 AWQ has weight-only layers: no such scales to compare
        assert checked > 0
    packed = tensors["model.layers.0.mlp.up_proj.weight"]
    assert packed.element_size() == 1
