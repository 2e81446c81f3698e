"""QuantLinear against the reference's own cases (tests/unit/torch/quantization/test_quant_linear.py):
with no calibrated amax a quantiser uses the tensor's own abs-max, so the layer must equal F.linear on
operands fake-quantised by hand — per tensor, per output row, with multi-dimensional inputs, at other
bit widths — exactly (rtol = atol = 0); disabled quantisers give the plain layer; class-level default
descriptors are honoured."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def m():
    import b200q
    from b200q import tensor_quant, utils
    from b200q.nn import quant_linear

    class NS:
        pass

    ns = NS()
    ns.mtq, ns.tq, ns.utils, ns.ql = b200q, tensor_quant, utils, quant_linear
    ns.cfg = b200q.QuantizerAttributeConfig
    return ns


def _x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator(device="cuda").manual_seed(seed), device="cuda")


def test_weight_fake_per_tensor(m):
    layer = m.ql.QuantLinear(2, 2, bias=False, quant_desc_weight=m.cfg(axis=None)).cuda()
    layer.input_quantizer.disable()
    x = _x(2, 2)
    w = layer.weight.detach().clone()
    want = F.linear(x, m.tq.fake_tensor_quant(w, w.abs().max()))
    assert torch.equal(layer(x), want)


def test_weight_fake_per_channel(m):
    layer = m.ql.QuantLinear(3, 5, bias=False, quant_desc_weight=m.cfg(num_bits=8, axis=0)).cuda()
    layer.input_quantizer.disable()
    x = _x(32, 3)
    w = layer.weight.detach().clone()
    amax = m.utils.reduce_amax(w, axis=1, keepdims=True)
    assert torch.equal(layer(x), F.linear(x, m.tq.fake_tensor_quant(w, amax)))


def test_input_fake_per_tensor(m):
    layer = m.ql.QuantLinear(3, 5, bias=False).cuda()
    layer.weight_quantizer.disable()
    x = _x(32, 3, seed=1)
    want = F.linear(m.tq.fake_tensor_quant(x, x.abs().max()), layer.weight.detach())
    assert torch.equal(layer(x), want)


@pytest.mark.parametrize("shape", [(32, 3), (4, 17, 9, 3)])
def test_everything_quantised_per_tensor(m, shape):
    layer = m.ql.QuantLinear(3, 5, bias=True, quant_desc_weight=m.cfg()).cuda()
    x = _x(*shape, seed=2)
    w = layer.weight.detach().clone()
    want = F.linear(m.tq.fake_tensor_quant(x, x.abs().max()), m.tq.fake_tensor_quant(w, w.abs().max()), layer.bias)
    assert torch.equal(layer(x), want)


def test_everything_quantised_per_channel(m):
    layer = m.ql.QuantLinear(3, 5, bias=False, quant_desc_weight=m.cfg(num_bits=8, axis=0)).cuda()
    x = _x(2, 3, seed=3)
    w = layer.weight.detach().clone()
    want = F.linear(m.tq.fake_tensor_quant(x, x.abs().max()),
                    m.tq.fake_tensor_quant(w, w.abs().max(dim=1, keepdim=True)[0]))
    assert torch.equal(layer(x), want)


def test_other_precisions(m):
    d_in, d_w = m.cfg(num_bits=4), m.cfg(num_bits=3)
    layer = m.ql.QuantLinear(3, 5, bias=False, quant_desc_input=d_in, quant_desc_weight=d_w).cuda()
    x = _x(2, 3, seed=4)
    qi, qw = m.mtq.nn.TensorQuantizer(d_in).cuda(), m.mtq.nn.TensorQuantizer(d_w).cuda()
    assert torch.equal(layer(x), F.linear(qi(x), qw(layer.weight.detach().clone())))


def test_disabled_quantisers_give_the_plain_layer(m):
    layer = m.ql.QuantLinear(3, 5, bias=True, quant_desc_input=m.cfg(num_bits=16),
                             quant_desc_weight=m.cfg(num_bits=16, axis=0)).cuda()
    plain = torch.nn.Linear(3, 5, bias=True).cuda()
    plain.load_state_dict(layer.state_dict())
    layer.input_quantizer.disable()
    layer.weight_quantizer.disable()
    x = _x(2, 3, seed=5)
    assert torch.equal(layer(x), plain(x))


def test_class_level_default_descriptors(m):
    layer = m.ql.QuantLinear(4, 16)
    assert layer.input_quantizer.axis is None and layer.weight_quantizer.axis == 0
    saved = (m.ql.QuantLinear.default_quant_desc_input, m.ql.QuantLinear.default_quant_desc_weight)
    try:
        m.ql.QuantLinear.default_quant_desc_input = m.cfg(num_bits=11)
        m.ql.QuantLinear.default_quant_desc_weight = m.cfg(num_bits=13, axis=1)
        layer = m.ql.QuantLinear(4, 16)
        assert layer.input_quantizer.num_bits == 11 and layer.weight_quantizer.axis == 1
    finally:
        m.ql.QuantLinear.default_quant_desc_input, m.ql.QuantLinear.default_quant_desc_weight = saved
