"""Factory behaviour (reference ``tests/test_factory.py`` and ``tests/test_legacy.py``)."""
import pytest
import torch
from torch import nn

import tensor_parallel_b200 as tp


@pytest.mark.parametrize("sharded", [False, True, None])
def test_factory_plain_module(sharded):
    model = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=sharded)
    assert isinstance(wrapped, tp.TensorParallel)
    assert (wrapped.sharding_manager is not None) == bool(sharded)  # None is falsy through the factory


def test_class_default_is_sharded():
    model = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    assert tp.TensorParallel(model, ["cpu", "cpu"]).sharding_manager is not None


def test_legacy_sharded_shim():
    model = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=False)
    same = tp.Sharded(wrapped)
    assert same is wrapped and wrapped.sharding_manager is not None
    with pytest.raises(RuntimeError, match="already applied"):
        wrapped.apply_sharding()


def test_output_device_selection():
    model = nn.Sequential(nn.Linear(8, 16), nn.Linear(16, 4))
    with pytest.raises(ValueError):
        tp.TensorParallel(model, ["cpu", "cpu"], output_device="cpu", output_device_index=1)
    wrapped = tp.TensorParallel(model, ["cpu", "cpu"], output_device_index=1)
    x = torch.randn(3, 8)
    torch.testing.assert_close(wrapped(x), model(x), atol=1e-6, rtol=1e-5)


def test_single_container_required():
    with pytest.raises(ValueError, match="container"):
        tp.TensorParallel(nn.Linear(4, 4), ["cpu", "cpu"])


def test_hf_model_gets_pretrained_wrapper():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.GPT2Config(vocab_size=100, n_positions=32, n_embd=32, n_layer=1, n_head=4, attn_implementation="eager")
    model = transformers.GPT2LMHeadModel(cfg)
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"])
    assert isinstance(wrapped, transformers.PreTrainedModel)
    assert isinstance(wrapped, tp.TensorParallelPreTrainedModel)
    assert isinstance(wrapped.wrapped_model, tp.TensorParallel)


def test_register_predefined_config():
    """A user-supplied rule table for a new ``model_type`` is picked up by the factory; double registration is refused."""
    import tensor_parallel_b200 as tp
    from torch import nn

    class Cfg:
        model_type = "my_two_layer_net"

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.config = Cfg()
            self.up = nn.Linear(8, 16)
            self.down = nn.Linear(16, 8)

        def forward(self, x):
            return self.down(torch.relu(self.up(x)))

    seen = []

    def getter(model_config, devices):
        seen.append(len(devices))
        return tp.Config(
            state_rules={r"up\.(weight|bias)$": tp.Split(world_size=len(devices), dim=0), r"down\.weight$": tp.Split(world_size=len(devices), dim=1),
                         r"down\.bias$": tp.Scale(world_size=len(devices))},
            input_rules={}, output_rules={r"^down$": {0: "sum"}}, attr_rules={})

    tp.register_predefined_config("my_two_layer_net", getter)
    try:
        with pytest.raises(ValueError):
            tp.register_predefined_config("my_two_layer_net", getter)
        torch.manual_seed(0)
        net = Net()
        x = torch.randn(3, 8)
        want = net(x)
        wrapped = tp.tensor_parallel(net, ["cpu", "cpu"])
        torch.testing.assert_close(wrapped(x), want, atol=1e-5, rtol=1e-5)
        assert seen == [2]
    finally:
        tp.PREDEFINED_CONFIGS.pop("my_two_layer_net", None)
