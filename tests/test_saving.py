"""Checkpoint layouts: un-sharded save equals the original state dict; sharded layout round
trips; plain state dicts convert to the sharded layout and load into a meta-initialised model.
Modelled on the reference's ``tests/test_saving.py``."""
import pytest
import torch
from torch import nn

import tensor_parallel_b200 as tp
from tensor_parallel_b200.models.gpt2 import GPT2Config, GPT2LMHeadModel
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM
from tensor_parallel_b200.models.t5 import T5Config, T5ForConditionalGeneration


def _models():
    torch.manual_seed(0)
    return {
        "gpt2": GPT2LMHeadModel(GPT2Config(vocab_size=90, n_positions=32, n_embd=32, n_layer=2, n_head=4)),
        "llama": LlamaForCausalLM(LlamaConfig(vocab_size=90, hidden_size=32, intermediate_size=86, num_hidden_layers=2, num_attention_heads=4)),
        "t5": T5ForConditionalGeneration(T5Config(vocab_size=90, d_model=32, d_kv=8, d_ff=48, num_layers=2, num_heads=4)),
    }


def _assert_same_state(got, want):
    assert set(got.keys()) == set(want.keys())
    for key, value in want.items():
        assert got[key].shape == value.shape, key
        torch.testing.assert_close(got[key].cpu(), value.cpu(), msg=key)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_no_parallelism_zero_3(world):
    model = nn.Sequential(nn.Linear(16, 32), nn.LayerNorm(32), nn.Linear(32, 7))
    wrapped = tp.TensorParallel(model, ["cpu"] * world, tensor_parallel_config=tp.Config({}, {}, {}, {}), sharded=True)
    with tp.save_tensor_parallel(wrapped):
        state = wrapped.state_dict()
    if world == 1:
        state = {k.replace("module_shards.0.", ""): v for k, v in state.items()}
    _assert_same_state(state, model.state_dict())


@pytest.mark.parametrize("name", ["gpt2", "llama", "t5"])
@pytest.mark.parametrize("sharded", [False, True])
@pytest.mark.parametrize("world", [2, 3])
def test_unsharded_save_equals_original(name, sharded, world):
    model = _models()[name]
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=sharded)
    with tp.save_tensor_parallel(wrapped):
        state = wrapped.state_dict()
    _assert_same_state(state, model.state_dict())
    assert wrapped.preserve_shards_when_saving  # restored on exit


def test_exact_key_matching_for_numbered_modules():
    """``0.weight`` must not swallow ``10.weight`` when shards are merged."""
    model = nn.Sequential(*[nn.Linear(6, 6) for _ in range(11)])
    wrapped = tp.TensorParallel(model, ["cpu", "cpu"], sharded=False)
    with tp.save_tensor_parallel(wrapped):
        _assert_same_state(wrapped.state_dict(), model.state_dict())


@pytest.mark.parametrize("name", ["gpt2", "llama"])
def test_save_keep_shards(name):
    model = _models()[name]
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    state = wrapped.state_dict()
    assert any(k.startswith("module_shards.1.") for k in state)
    assert "_sanity_check_params.0" in state and "sharding_manager.flat_shards.1" in state
    fresh = tp.tensor_parallel(_models()[name], ["cpu", "cpu"], sharded=True)
    with torch.no_grad():
        for p in fresh.parameters():
            p.add_(1.0)
    fresh.load_state_dict(state)
    ids = torch.randint(0, 90, (2, 6))
    torch.testing.assert_close(fresh(input_ids=ids).logits, wrapped(input_ids=ids).logits)


@pytest.mark.parametrize("world", [2, 3])
def test_convert_state_dict_and_meta_loading(world):
    model = _models()["llama"]
    with torch.device("meta"):
        skeleton = LlamaForCausalLM(model.config)
    wrapped = tp.tensor_parallel(skeleton, ["cpu"] * world, sharded=False)
    assert all(p.device.type == "meta" for n, p in wrapped.named_parameters() if "_sanity_check" not in n)
    with pytest.raises(RuntimeError, match="meta"):
        wrapped.apply_sharding()
    # convert in two partial chunks (memory-efficient loading)
    full = model.state_dict()
    keys = list(full)
    for chunk in (keys[: len(keys) // 2], keys[len(keys) // 2 :]):
        converted = tp.convert_state_dict({k: full[k] for k in chunk}, wrapped.tensor_parallel_config, world_size=world)
        tp.load_sharded_state_dict_(wrapped, converted, strict=False)
    assert not any(p.device.type == "meta" for p in wrapped.parameters())
    wrapped.apply_sharding()
    ids = torch.randint(0, 90, (2, 6))
    torch.testing.assert_close(wrapped(input_ids=ids).logits, model(input_ids=ids).logits, atol=3e-5, rtol=1e-5)
    device_map = tp.infer_sharded_device_map(wrapped)
    assert set(device_map.values()) == {torch.device("cpu")}
    assert all(("module_shards." in k) or ("_sanity_check_params." in k) or ("flat_shards." in k) for k in device_map)


def test_meta_loading_keeps_tied_weights_tied():
    model = _models()["gpt2"]
    with torch.device("meta"):
        skeleton = GPT2LMHeadModel(model.config)
    wrapped = tp.tensor_parallel(skeleton, ["cpu", "cpu"], sharded=False)
    converted = tp.convert_state_dict(model.state_dict(), wrapped.tensor_parallel_config, world_size=2)
    tp.load_sharded_state_dict_(wrapped, converted, strict=False)
    for shard in wrapped.module_shards:
        assert shard.lm_head.tp_wrapped_module.weight is shard.transformer.wte.tp_wrapped_module.weight
    ids = torch.randint(0, 90, (2, 6))
    torch.testing.assert_close(wrapped(input_ids=ids).logits, model(input_ids=ids).logits, atol=3e-5, rtol=1e-5)


def test_converted_keys_match_live_keys():
    model = _models()["gpt2"]
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=False)
    live = set(wrapped.state_dict().keys())
    source = {k: v for k, v in model.state_dict().items()}
    converted = set(tp.convert_state_dict(source, wrapped.tensor_parallel_config, world_size=2).keys())
    assert converted == live
    prefixed = tp.convert_state_dict(source, wrapped.tensor_parallel_config, world_size=2, for_pretrained=True)
    assert all(k.startswith("wrapped_model.") for k in prefixed)


def test_device_map_rank_parsing():
    from tensor_parallel_b200.parallel.checkpoint import infer_sharded_data_device_id

    assert infer_sharded_data_device_id("wrapped_model.module_shards.3.transformer.h.0.attn.weight") == 3
    assert infer_sharded_data_device_id("_sanity_check_params.12") == 12
    assert infer_sharded_data_device_id("sharding_manager.flat_shards.1") == 1
    with pytest.raises(KeyError):
        infer_sharded_data_device_id("transformer.h.0.weight")


def test_rewrap_with_a_different_world_size_after_training_steps():
    """The recovery path when the set of devices changes: the un-sharded checkpoint is independent of the world size, so a
    model trained on 2 ranks (ZeRO-3 shards included) continues on 3 ranks with identical outputs."""
    torch.manual_seed(3)
    model = _models()["llama"]
    ids = torch.randint(0, 90, (2, 12))
    two = tp.tensor_parallel(model, ["cpu"] * 2, sharded=True)
    opt = torch.optim.SGD(two.parameters(), lr=0.05)
    for _ in range(2):
        two(input_ids=ids, labels=ids).loss.backward()
        opt.step()
        opt.zero_grad()
    with torch.no_grad():
        want = two(input_ids=ids).logits
    with tp.save_tensor_parallel(two):
        state = {k: v.clone() for k, v in two.state_dict().items()}
    fresh = LlamaForCausalLM(LlamaConfig(vocab_size=90, hidden_size=32, intermediate_size=86, num_hidden_layers=2, num_attention_heads=4))
    fresh.load_state_dict(state)
    three = tp.tensor_parallel(fresh, ["cpu"] * 3, sharded=True)
    with torch.no_grad():
        got = three(input_ids=ids).logits
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["llama", "gpt2"])
@pytest.mark.parametrize("world", [2, 3])
def test_convert_state_dict_emits_flat_shards(name, world):
    """A plain state dict converts to exactly the state dict of a model wrapped with ``sharded=True`` (flat shards included,
    tied aliases of sharded parameters dropped) and loads straight into one."""
    model = _models()[name]
    reference = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    want = reference.state_dict()
    names = tp.replicated_parameter_names(model, reference.tensor_parallel_config)
    assert tuple(names) == tuple(reference.sharding_manager.sharded_param_names)
    converted = tp.convert_state_dict(model.state_dict(), reference.tensor_parallel_config, world_size=world, sharded_param_names=names)
    tensor_keys = {k for k in want if not k.endswith("_extra_state")}
    assert set(converted) == tensor_keys
    for key in tensor_keys:
        torch.testing.assert_close(converted[key], want[key], msg=key)
    # loads into a differently initialised sharded model and reproduces the outputs
    torch.manual_seed(99)
    other = tp.tensor_parallel(type(model)(model.config), ["cpu"] * world, sharded=True)
    other.load_state_dict(converted, strict=False)
    ids = torch.randint(0, 90, (2, 6))
    with torch.no_grad():
        torch.testing.assert_close(other(input_ids=ids).logits, model(input_ids=ids).logits, atol=3e-5, rtol=1e-5)


def test_flat_shard_layout_is_saved_and_checked():
    """The sharded layout's state dict carries the ZeRO-3 layout (names, shapes, piece sizes); a model whose flat shards
    are cut differently refuses it, and a checkpoint without the metadata (reference-written) still loads."""
    import torch
    from torch import nn

    import tensor_parallel_b200 as tp

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(16, 32), nn.LayerNorm(32), nn.Linear(32, 8), nn.LayerNorm(8))

    model = tp.TensorParallel(make(), ["cpu", "cpu"], sharded=True)
    state = model.state_dict()
    layout = state["sharding_manager._extra_state"]
    assert layout["names"] == list(model.sharding_manager.sharded_param_names) and len(layout["sizes_with_pad"]) == 2
    same = tp.TensorParallel(make(), ["cpu", "cpu"], sharded=True)
    same.load_state_dict(state)
    names = list(model.sharding_manager.sharded_param_names)
    other = tp.TensorParallel(make(), ["cpu", "cpu"], sharded=True, sharded_param_names=names[::-1])
    import pytest

    with pytest.raises(RuntimeError, match="different layout"):
        other.load_state_dict(state)
    legacy = {k: v for k, v in state.items() if not k.endswith("_extra_state")}
    same.load_state_dict(legacy)
