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
