"""LoRA-augmented linears under tensor parallelism (reference ``tests/test_transformers.py`` with ``use_lora=True``;
rules from ``src/tensor_parallel/config.py:128-154``).  ``peft`` is not needed: the adapter below has the layout of
``peft.tuners.lora.Linear`` (a linear layer that owns ``lora_A`` / ``lora_B`` module dicts)."""
import pytest
import torch
from torch import nn

import tensor_parallel_b200 as tp
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM


class LoraLinear(nn.Linear):
    def __init__(self, base: nn.Linear, r: int = 4, alpha: float = 8.0):
        super().__init__(base.in_features, base.out_features, bias=base.bias is not None)
        self.weight, self.bias = base.weight, base.bias
        self.lora_A = nn.ModuleDict({"default": nn.Linear(base.in_features, r, bias=False)})
        self.lora_B = nn.ModuleDict({"default": nn.Linear(r, base.out_features, bias=False)})
        nn.init.normal_(self.lora_B["default"].weight, std=0.05)  # (peft starts from zero; non-zero makes the test meaningful)
        self.scaling = alpha / r

    def forward(self, x):
        return super().forward(x) + self.lora_B["default"](self.lora_A["default"](x)) * self.scaling


def _lora_llama():
    torch.manual_seed(0)
    model = LlamaForCausalLM(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                                         num_key_value_heads=2))
    for layer in model.model.layers:
        layer.self_attn.q_proj = LoraLinear(layer.self_attn.q_proj)   # column-parallel base: lora_B is split like it
        layer.self_attn.v_proj = LoraLinear(layer.self_attn.v_proj)
        layer.self_attn.o_proj = LoraLinear(layer.self_attn.o_proj)   # row-parallel base: lora_A sees the gathered input
        layer.mlp.down_proj = LoraLinear(layer.mlp.down_proj)
    return model


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("sharded", [False, True])
def test_lora_forward_and_gradients(world, sharded):
    model = _lora_llama()
    ids = torch.randint(0, 64, (2, 9))
    ref = model(input_ids=ids, labels=ids)
    ref.loss.backward()
    grads = {n: p.grad.clone() for n, p in model.named_parameters() if "lora_" in n}
    model.zero_grad()
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=sharded)
    out = wrapped(input_ids=ids, labels=ids)
    torch.testing.assert_close(out.logits, ref.logits, atol=2e-5, rtol=1e-4)
    out.loss.backward()
    with tp.save_tensor_parallel(wrapped):
        names = set(wrapped.state_dict().keys())
    assert any("lora_A" in n for n in names) and any("lora_B" in n for n in names)
    def param(shard, name):
        return {n.replace("tp_wrapped_module.", ""): q for n, q in shard.named_parameters()}[name]

    # a replicated adapter matrix (lora_A of a column-parallel base) only sees its rank's slice of lora_B downstream:
    # the per-rank gradients are partial and add up to the full one (sharded=True sums them into the ZeRO-3 flat shards)
    name = "model.layers.0.self_attn.q_proj.lora_A.default.weight"
    if not sharded:
        total = sum(param(shard, name).grad for shard in wrapped.module_shards)
        torch.testing.assert_close(total, grads[name], atol=2e-5, rtol=1e-3)
    # a split adapter matrix (lora_B of a column-parallel base) carries its slice of the gradient
    name_b = "model.layers.0.self_attn.q_proj.lora_B.default.weight"
    pieces = [param(shard, name_b).grad for shard in wrapped.module_shards]
    assert pieces[0].shape[0] < grads[name_b].shape[0]
    torch.testing.assert_close(torch.cat(pieces, dim=0), grads[name_b], atol=2e-5, rtol=1e-3)


@pytest.mark.parametrize("world", [2, 3])
def test_reduce_replicated_gradients_keeps_replicas_exact(world):
    """Without ZeRO-3 a replicated parameter only receives its rank's share of the gradient; summing the shares gives every
    replica the gradient of the unsplit model (norm weights and the replicated LoRA matrices alike)."""
    model = _lora_llama()
    ids = torch.randint(0, 64, (2, 9))
    model(input_ids=ids, labels=ids).loss.backward()
    want = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=False)
    wrapped(input_ids=ids, labels=ids).loss.backward()
    reduced = wrapped.reduce_replicated_gradients()
    assert reduced > 0
    checked = 0
    for shard in wrapped.module_shards:
        for name, p in shard.named_parameters():
            if name in wrapped.modified_parameters_names:
                continue
            torch.testing.assert_close(p.grad, want[name.replace("tp_wrapped_module.", "")], atol=3e-5, rtol=1e-3, msg=name)
            checked += 1
    assert checked >= 2 * world
    assert tp.tensor_parallel(_lora_llama(), ["cpu"] * world, sharded=True).reduce_replicated_gradients() == 0
