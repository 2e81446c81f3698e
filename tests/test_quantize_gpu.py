"""``mtq.quantize`` on the reference's small linear model with the configurations of the reference's own
test file (tests/unit/torch/quantization/test_quantize_cpu.py): double quantisation through sequential
quantisers with awq_lite, INT8 with the mse search, an invalid configuration, a forward loop without
arguments, a custom calibrator class surviving save / restore, per-class configuration, static weights
with dynamic per-token activations, and block_sizes given as axes.  The model and data live on the GPU;
convolution rows are absent (only linear layers are on this library's path)."""
import copy

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mtq():
    import b200q

    return b200q


class SimpleLinear(nn.Module):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))

    def forward(self, x):
        return self.net(x)

    @staticmethod
    def get_input():
        return torch.randn(2, 16, device="cuda")


WINT4INT8_CFG = {
    "quant_cfg": {"*weight_quantizer": [{"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                                        {"num_bits": 8, "axis": 0, "enable": True}],
                  "*input_quantizer": {"num_bits": 8, "axis": None, "enable": True}},
    "algorithm": "awq_lite",
}
INT8_MSE_CFG = {"quant_cfg": {"*weight_quantizer": {"num_bits": 8, "axis": 0},
                              "*input_quantizer": {"num_bits": 8, "axis": None}}, "algorithm": "mse"}
STATIC_WEIGHT_DYNAMIC_ACTIVATION_CFG = {
    "quant_cfg": {"*weight_quantizer": {"num_bits": 8, "axis": 0},
                  "*input_quantizer": {"num_bits": 8, "axis": (0, 1), "type": "dynamic"},
                  "default": {"enable": False}},
    "algorithm": "max",
}


def _model(seed=0):
    torch.manual_seed(seed)
    return SimpleLinear().cuda()


@pytest.mark.parametrize("cfg", [WINT4INT8_CFG, INT8_MSE_CFG], ids=["wint4int8_awq_lite", "int8_mse"])
def test_quantize_runs(mtq, cfg):
    model = _model()
    data = [model.get_input() for _ in range(2)]
    with torch.no_grad():
        plain = model(data[0])
    mtq.quantize(model, copy.deepcopy(cfg), lambda m: [m(b) for b in data])
    layers = [m for m in model.net if isinstance(m, nn.Linear)]
    assert all(mtq.nn.quant_linear.is_quantized_linear(m) for m in layers)
    if cfg is WINT4INT8_CFG:
        assert all(isinstance(m.weight_quantizer, mtq.nn.SequentialQuantizer) for m in layers)
        assert all(q.amax is not None for m in layers for q in m.weight_quantizer)
    with torch.no_grad():
        out = model(data[0])
    assert torch.isfinite(out).all() and (out - plain).abs().mean() <= 0.5 * plain.abs().mean() + 0.05


def test_an_invalid_configuration_is_refused(mtq):
    cfg = {"quant_cfg": {"*": {"num_bits": 4, "axis": 0, "block_sizes": {-1: 128}}}, "algorithm": "max"}
    with pytest.raises(ValueError, match="axis must be None when block_sizes is not None."):
        mtq.quantize(_model(), cfg)


def test_a_forward_loop_without_arguments(mtq):
    model = _model()
    data = [model.get_input() for _ in range(2)]

    def forward_loop():
        for batch in data:
            model(batch)

    mtq.quantize(model, copy.deepcopy(mtq.INT8_DEFAULT_CFG), forward_loop=forward_loop)
    assert all(m.input_quantizer.amax is not None for m in model.net if isinstance(m, nn.Linear))


def test_a_custom_calibrator_survives_save_and_restore(mtq):
    class DoublingMaxCalibrator(mtq.calib.MaxCalibrator):
        def compute_amax(self, *args, **kwargs):
            return 2 * super().compute_amax(*args, **kwargs)

    cfg = {"quant_cfg": {"*": {"num_bits": 4, "axis": None, "enable": True,
                               "calibrator": (DoublingMaxCalibrator, (4, None, False))}}, "algorithm": "max"}
    ref = _model()
    x = ref.get_input()
    mtq.quantize(ref, cfg, lambda m: m(x))
    assert torch.equal(ref.net[0].input_quantizer.amax, 2 * x.abs().amax())
    fresh = _model(seed=1)
    mtq.restore_from_modelopt_state(fresh, mtq.modelopt_state(ref))
    fresh.load_state_dict(ref.state_dict())
    with torch.no_grad():
        assert torch.allclose(ref(x), fresh(x))
    for name, m in fresh.named_modules():
        if name.endswith("quantizer"):
            assert type(m._calibrator) is DoublingMaxCalibrator


def test_per_class_configuration(mtq):
    cfg = {"quant_cfg": {"nn.Linear": {"*": {"num_bits": 4, "axis": -1, "enable": True}},
                         "nn.BatchNorm2d": {"*": {"enable": False}},
                         "*output_quantizer": {"num_bits": 8, "enable": True}}, "algorithm": "max"}
    model = _model()
    x = model.get_input()
    mtq.quantize(model, cfg, lambda m: m(x))
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear):
            for q in (m.weight_quantizer, m.input_quantizer):
                assert q.num_bits == 4 and q.axis == -1 and q.is_enabled
        if name.endswith("output_quantizer"):
            assert m.is_enabled and m.num_bits == 8


def test_static_weights_with_dynamic_activations(mtq):
    model = _model()
    x = model.get_input()
    mtq.quantize(model, copy.deepcopy(STATIC_WEIGHT_DYNAMIC_ACTIVATION_CFG), lambda m: m(m.get_input()))
    for name, m in model.named_modules():
        if name.endswith("weight_quantizer"):
            assert m.amax is not None
        if name.endswith("input_quantizer"):
            assert m.amax is None
    assert torch.isfinite(model(x)).all()
    model = _model()
    mtq.quantize(model, copy.deepcopy(STATIC_WEIGHT_DYNAMIC_ACTIVATION_CFG))           # no forward loop at all
    assert all(m.amax is not None for n, m in model.named_modules() if n.endswith("weight_quantizer"))


def test_block_sizes_given_as_axes_equal_the_axis_form(mtq):
    ref_cfg = {"quant_cfg": {"*weight_quantizer": {"num_bits": 8, "axis": 0},
                             "*input_quantizer": {"num_bits": 8, "axis": None, "type": "dynamic"},
                             "default": {"enable": False}}, "algorithm": "max"}
    cfg = {"quant_cfg": {"*weight_quantizer": {"num_bits": 8, "block_sizes": {1: None}},
                         "*input_quantizer": {"num_bits": 8, "block_sizes": {0: None, 1: None}, "type": "dynamic"},
                         "default": {"enable": False}}, "algorithm": "max"}
    model_ref = _model()
    model = copy.deepcopy(model_ref)
    x = model_ref.get_input()
    mtq.quantize(model_ref, ref_cfg, lambda m: m(x))
    mtq.quantize(model, cfg, lambda m: m(x))
    with torch.no_grad():
        assert torch.allclose(model_ref(x), model(x))
    for a, b in zip(model_ref.net, model.net):
        if hasattr(a, "weight_quantizer"):
            assert torch.equal(a.weight_quantizer.amax.reshape(-1), b.weight_quantizer.amax.reshape(-1))


def test_rotated_query_and_key_quantisers_of_a_registered_attention_module(mtq):
    """Reference tests/gpu/torch/quantization/test_hadamard.py:46-82, with the attention class registered by
    hand (``mtq.register``) instead of generated by the reference's Hugging Face plugin: rotating both the
    query and the key by the same orthonormal Hadamard matrix leaves q·kᵀ, hence the output, unchanged;
    rotating the key alone does not."""
    import torch.nn.functional as F

    class Attention(nn.Module):
        def forward(self, q, k, v):
            return F.scaled_dot_product_attention(q, k, v)

    class QuantAttention(Attention):
        def _setup(self):
            self.q_bmm_quantizer = mtq.nn.TensorQuantizer()
            self.k_bmm_quantizer = mtq.nn.TensorQuantizer()
            self.v_bmm_quantizer = mtq.nn.TensorQuantizer()

        def forward(self, q, k, v):
            return super().forward(self.q_bmm_quantizer(q), self.k_bmm_quantizer(k), self.v_bmm_quantizer(v))

    mtq.register(original_cls=Attention, quantized_cls=QuantAttention)
    try:
        model = nn.Sequential(Attention()).cuda()
        mtq.replace_quant_module(model)
        assert isinstance(model[0], QuantAttention)
        mtq.set_quantizer_by_cfg(model, {"*": {"enable": False}})
        g = torch.Generator(device="cuda").manual_seed(0)
        q, k, v = (torch.randn(2, 4, 16, 64, generator=g, device="cuda") for _ in range(3))
        want = model[0](q, k, v)
        assert torch.equal(want, F.scaled_dot_product_attention(q, k, v))
        with mtq.set_quantizer_by_cfg_context(model, {"*[qk]_bmm_quantizer": {"rotate": True, "enable": False}}):
            assert model[0].q_bmm_quantizer._rotate and model[0].k_bmm_quantizer._rotate
            both = model[0](q, k, v)
        assert not model[0].q_bmm_quantizer._rotate
        assert torch.allclose(both, want, atol=0.05)
        with mtq.set_quantizer_by_cfg_context(model, {"*k_bmm_quantizer": {"rotate": True, "enable": False}}):
            key_only = model[0](q, k, v)
        assert not torch.allclose(key_only, want, atol=0.05)
    finally:
        mtq.unregister(Attention)


@pytest.mark.parametrize(("name", "rtol", "atol"), [("FP8_DEFAULT_CFG", 1e-3, 1e-2), ("NVFP4_DEFAULT_CFG", 1e-3, 5e-1)])
def test_torch_export_of_a_quantized_model(mtq, name, rtol, atol):
    """Reference tests/gpu/torch/quantization/test_torch_export.py: ``torch.export`` traces the quantised
    model through the registered ops (their meta implementations) and the exported program reproduces the
    eager output."""
    from b200q.utils import export_torch_mode

    class SimpleNetwork(nn.Module):
        def __init__(self):
            super().__init__()
            self.linear1 = nn.Linear(16, 32)
            self.linear2 = nn.Linear(32, 16)

        def forward(self, x):
            return self.linear2(torch.relu(self.linear1(x)))

    torch.manual_seed(42)
    x = torch.randn(2, 16, device="cuda")
    model = SimpleNetwork().eval().cuda()
    with torch.inference_mode():
        mtq.quantize(model, copy.deepcopy(getattr(mtq, name)), lambda m: m(x))
        want = model(x)
        with export_torch_mode():
            program = torch.export.export(model, (x,), strict=False)
            got = program.module()(x)
    assert torch.allclose(want, got, rtol=rtol, atol=atol)
    ops_seen = {str(n.target) for n in program.graph.nodes if n.op == "call_function"}
    assert any("quantize_op" in t for t in ops_seen), ops_seen


def test_quantizer_context_restores_everything_but_what_calibration_added(mtq):
    """Reference tests/unit/torch/quantization/test_tensor_quant_cpu.py:104-134: inside
    ``set_quantizer_by_cfg_context`` only the output quantisers are on and get calibrated; afterwards the
    model computes what it computed before and every other buffer is untouched."""
    cfg = {"quant_cfg": {"*weight_quantizer": [{"num_bits": 4, "block_sizes": {-1: 128, "type": "static"}, "enable": True},
                                               {"num_bits": 8, "axis": 0, "enable": True}],
                         "*input_quantizer": {"num_bits": 8, "enable": True},
                         "default": {"enable": False}},
           "algorithm": "awq_full"}
    model = _model().eval()
    x = model.get_input()
    mtq.quantize(model, cfg, lambda m: m(x))
    state = {k: v.clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        want = model(x)
    mtq.set_quantizer_by_cfg(model, {"*output_quantizer": {"enable": True}})
    with mtq.set_quantizer_by_cfg_context(model, {"*": {"enable": False}, "*output_quantizer": {"enable": True}}):
        for name, m in model.named_modules():
            if isinstance(m, mtq.nn.TensorQuantizer):
                assert m.is_enabled == name.endswith("output_quantizer"), name
        mtq.calibrate(model, "max", lambda m: m(x * 10))
    mtq.set_quantizer_by_cfg(model, {"*output_quantizer": {"enable": False}})
    with torch.no_grad():
        assert torch.allclose(model(x), want)
    for k, v in model.state_dict().items():
        if "output_quantizer" not in k:
            assert torch.equal(v, state[k]), k


def _data_parallel_rank(rank, world, port):
    import os

    import torch.distributed as dist

    import b200q

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank % torch.cuda.device_count())
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = _model()                                     # the same weights on every rank
        g = torch.Generator(device="cuda").manual_seed(10 + rank)
        batches = [torch.randn(2, 16, device="cuda", generator=g) * (1 + rank) for _ in range(2)]

        def forward_loop(m):
            for b in batches:
                m(b)

        alone = copy.deepcopy(model)
        b200q.replace_quant_module(alone)
        b200q.set_quantizer_by_cfg(alone, b200q.INT8_DEFAULT_CFG["quant_cfg"])
        b200q.model_calib.max_calibrate(alone, forward_loop, distributed_sync=False)
        b200q.quantize(model, b200q.INT8_DEFAULT_CFG, forward_loop)
        checked = 0
        for (name, q), (_, q_alone) in zip(model.named_modules(), alone.named_modules()):
            if isinstance(q, b200q.nn.TensorQuantizer) and "output_quantizer" not in name:
                # the reference's check: the amax already is the MAX over the ranks
                over_ranks = q.amax.clone()
                dist.all_reduce(over_ranks, op=dist.ReduceOp.MAX)
                assert torch.equal(over_ranks, q.amax), name
                # and it is the MAX of what each rank finds on its own batches
                mine = q_alone.amax.clone()
                dist.all_reduce(mine, op=dist.ReduceOp.MAX)
                assert torch.equal(mine, q.amax), name
                checked += 1
        assert checked == 6
    finally:
        dist.destroy_process_group()


def test_data_parallel_max_calibration_over_two_ranks(mtq):
    """Reference tests/unit/torch/quantization/test_dist.py:28-47 with the tensors on the GPU: two ranks
    (gloo; one GPU each when there are two, else both on the one GPU) calibrate INT8 on different batches
    and end with the same amax, the maximum over both."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_data_parallel_rank, args=(2, port), nprocs=2, join=True)
