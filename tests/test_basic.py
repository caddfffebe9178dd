"""Generic-module tests with the automatic config on repeated CPU devices (world sizes 1-4,
3 included on purpose: uneven splits and padding).  Modelled on the reference's
``tests/test_basic.py``; the oracle is always the unsplit module on the same inputs."""
import pytest
import torch
from torch import nn

import tensor_parallel_b200 as tp
from tensor_parallel_b200 import Config, Split, TensorParallel


@pytest.mark.parametrize("devices", [None, ("cpu",), ("cpu", "cpu"), ("cpu", "cpu", "cpu")])
def test_basic_attributes(devices):
    model = nn.Sequential(nn.Linear(12, 24), nn.ReLU(), nn.Linear(24, 6))
    wrapped = TensorParallel(model, devices)
    for shard in wrapped.module_shards:
        for sub in shard.modules():
            if isinstance(sub, nn.Linear):
                assert sub.weight.shape == (sub.out_features, sub.in_features)


@pytest.mark.parametrize("emb_cls", [nn.Embedding, nn.EmbeddingBag])
@pytest.mark.parametrize("devices", [None, ("cpu",), ("cpu", "cpu"), ("cpu", "cpu", "cpu")])
@pytest.mark.parametrize("sharded", [False, True])
def test_embeds_and_linear(emb_cls, devices, sharded):
    torch.manual_seed(0)
    model = nn.Sequential(emb_cls(num_embeddings=1337, embedding_dim=64), nn.LayerNorm(64), nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 10))
    ids = torch.randint(0, 1337, (17, 9))
    ref = model(ids)
    ref.norm().backward()
    ref_grad = model[0].weight.grad.clone()
    ref_ln_grad = model[1].weight.grad.clone()
    model.zero_grad()

    wrapped = TensorParallel(model, devices, sharded=sharded)
    out = wrapped(ids)
    out.norm().backward()
    torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-5)
    if devices is not None and len(devices) > 1:
        grads = [shard[0].tp_wrapped_module.weight.grad for shard in wrapped.module_shards]
        torch.testing.assert_close(torch.cat(grads, dim=1), ref_grad, atol=1e-6, rtol=1e-5)
        if sharded:
            # ZeRO-3: the flat shards receive the full (summed, unscaled) gradient of replicated params
            mgr = wrapped.sharding_manager
            stacked = torch.stack([f.grad for f in mgr.flat_shards])
            full = dict(zip(mgr.sharded_param_names, mgr._combine(stacked)))
            torch.testing.assert_close(full["1.weight"], ref_ln_grad, atol=1e-6, rtol=1e-5)


CONV_CASES = [
    (nn.Conv1d, (3, 8, 20)), (nn.Conv2d, (3, 8, 12, 12)), (nn.Conv3d, (2, 8, 9, 9, 9)),
    (nn.ConvTranspose1d, (3, 8, 20)), (nn.ConvTranspose2d, (3, 8, 12, 12)), (nn.ConvTranspose3d, (2, 8, 5, 5, 5)),
]


@pytest.mark.parametrize("conv_cls,shape", CONV_CASES)
@pytest.mark.parametrize("extra", [dict(), dict(stride=2), dict(dilation=2), dict(groups=2), dict(padding=1)])
@pytest.mark.parametrize("world", [2, 3, 4])
def test_convs(conv_cls, shape, extra, world):
    torch.manual_seed(0)
    bn = {3: nn.BatchNorm1d, 4: nn.BatchNorm2d, 5: nn.BatchNorm3d}[len(shape)]
    model = nn.Sequential(conv_cls(8, 16, kernel_size=3, **extra), bn(16), nn.ReLU(), conv_cls(16, 8, kernel_size=3, **extra), bn(8))
    x = torch.randn(*shape, requires_grad=True)
    ref = model(x)
    ref.norm().backward()
    ref_grad, x.grad = x.grad.clone(), None
    wrapped = TensorParallel(model, ["cpu"] * world)
    out = wrapped(x)
    out.norm().backward()
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-3)
    torch.testing.assert_close(x.grad, ref_grad, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_sharded_num_params(world):
    model = nn.Sequential(nn.Linear(64, 128), nn.LayerNorm(128), nn.Linear(128, 30), nn.LayerNorm(30))
    n_original = sum(p.numel() for p in model.parameters())
    plain = TensorParallel(model, ["cpu"] * world, sharded=False)
    sharded = TensorParallel(model, ["cpu"] * world, sharded=True)
    n_plain = sum(p.numel() for p in plain.parameters())
    n_sharded = sum(p.numel() for p in sharded.parameters())
    if world == 1:
        assert n_plain == n_sharded == n_original
        return
    replicated = 2 * 128 + 2 * 30  # the LayerNorm parameters
    assert n_plain == n_original + (world - 1) * replicated
    padding = n_sharded - n_original
    assert 0 <= padding < world * 4, padding  # each of the 4 replicated tensors can force < world pad elements
    lengths = {f.numel() for f in sharded.sharding_manager.flat_shards}
    assert len(lengths) == 1


def test_flat_shard_layout_is_deterministic():
    model = nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8), nn.Linear(8, 8), nn.LayerNorm(8))
    names = [TensorParallel(model, ["cpu"] * 3, sharded=True).sharding_manager.sharded_param_names for _ in range(3)]
    assert names[0] == names[1] == names[2] == tuple(sorted(names[0]))
    layout = TensorParallel(model, ["cpu"] * 3, sharded=True).sharding_manager.layout()
    assert layout["sizes_with_pad"][0][:2] == [3, 3] and layout["sizes_with_pad"][2][:2] == [2, 2]


def test_zero3_regather_is_version_gated():
    model = nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8))
    wrapped = TensorParallel(model, ["cpu", "cpu"], sharded=True)
    mgr = wrapped.sharding_manager
    calls = []
    original = mgr._gather
    mgr._gather = lambda all_cuda: (calls.append(1), original(all_cuda))[1]
    x = torch.randn(2, 8)
    wrapped(x)
    wrapped(x)  # gradient accumulation step: no optimizer step in between -> no new gather
    assert len(calls) == 1
    opt = torch.optim.SGD(wrapped.parameters(), lr=0.1)
    wrapped(x).sum().backward()
    opt.step()
    wrapped(x)
    assert len(calls) == 2


def test_config_backward_compatibility():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8))
    world = 2

    def legacy_split(dim):
        return lambda tensor, rank: torch.tensor_split(tensor, world, dim=dim)[rank]

    def legacy_merge(dim):
        return lambda tensors: torch.cat([t.cpu() for t in tensors], dim=dim)

    def build(kind):
        if kind == "modern":
            s0, s1 = Split(world, 0), Split(world, 1)
        elif kind == "callable":
            s0, s1 = legacy_split(0), legacy_split(1)
        else:
            s0, s1 = (legacy_split(0), legacy_merge(0)), (legacy_split(1), legacy_merge(1))
        return Config(
            state_rules={r"^0\.(weight|bias)$": s0, r"^2\.weight$": s1, r"^2\.bias$": tp.Scale(world)},
            input_rules={}, output_rules={r"^2$": {0: "sum"}}, attr_rules={},
        )

    states = {}
    x = torch.randn(5, 16)
    for kind in ("modern", "callable", "tuple"):
        wrapped = TensorParallel(model, ["cpu"] * world, tensor_parallel_config=build(kind))
        torch.testing.assert_close(wrapped(x), model(x), atol=1e-6, rtol=1e-5)
        states[kind] = wrapped.state_dict()
    for kind in ("callable", "tuple"):
        assert states[kind].keys() == states["modern"].keys()
        for key in states["modern"]:
            torch.testing.assert_close(states[kind][key], states["modern"][key])
    wrapped = TensorParallel(model, ["cpu"] * world, tensor_parallel_config=build("tuple"))
    with tp.save_tensor_parallel(wrapped):
        merged = wrapped.state_dict()
    for key, value in model.state_dict().items():
        torch.testing.assert_close(merged[key], value)


def test_conflicting_rules_raise():
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
    cfg = Config({}, {}, {r"^0$": {0: "sum"}, r"0": {0: "gather -1"}}, {})
    with pytest.raises(ValueError, match="conflicting"):
        TensorParallel(model, ["cpu", "cpu"], tensor_parallel_config=cfg)


def test_moving_wrapped_model_is_detected():
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
    wrapped = TensorParallel(model, ["cpu", "cpu"])
    wrapped._sanity_check_params[1] = nn.Parameter(torch.empty(0, device="meta"), requires_grad=False)
    with pytest.raises(ValueError, match="no longer on their devices"):
        wrapped(torch.randn(2, 4))


@pytest.mark.parametrize("sharded", [False, True])
def test_deepcopy_of_a_wrapped_model(sharded):
    """A wrapped model can be deep-copied (the copy gets its own rank threads and failure domain) and trained without
    touching the original."""
    import copy

    from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    model = LlamaForCausalLM(LlamaConfig(vocab_size=90, hidden_size=32, intermediate_size=86, num_hidden_layers=2, num_attention_heads=4))
    ids = torch.randint(0, 90, (2, 9))
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=sharded)
    with torch.no_grad():
        want = wrapped(input_ids=ids).logits
    clone = copy.deepcopy(wrapped)
    with torch.no_grad():
        torch.testing.assert_close(clone(input_ids=ids).logits, want)
    clone(input_ids=ids, labels=ids).loss.backward()
    assert all(p.grad is None for p in wrapped.parameters())
    assert any(p.grad is not None for p in clone.parameters())
