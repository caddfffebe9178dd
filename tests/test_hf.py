"""Hugging Face integration on the installed ``transformers``: the tiny GPT-2 configuration
(2 layers, d_model 128, 4 heads, FFN 512, vocab 1000, fp32, two CPU ranks, ZeRO-3 on,
batch 4 x 32, labels = inputs): logits, loss, gradients, state-dict round trip, generation."""
import pytest
import torch

import tensor_parallel_b200 as tp

transformers = pytest.importorskip("transformers")


def _tiny_gpt2():
    torch.manual_seed(0)
    cfg = transformers.GPT2Config(vocab_size=1000, n_positions=64, n_embd=128, n_layer=2, n_head=4, n_inner=512,
                                  initializer_range=0.02, attn_implementation="eager",
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    return transformers.GPT2LMHeadModel(cfg)


@pytest.mark.parametrize("world", [2, 3])
def test_tiny_gpt2_training_parity_and_round_trip(world):
    model = _tiny_gpt2()
    ids = torch.randint(0, 1000, (4, 32), generator=torch.Generator().manual_seed(1))
    ref = model(input_ids=ids, labels=ids)
    ref.loss.backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()

    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    assert isinstance(wrapped, tp.TensorParallelPreTrainedModel)
    out = wrapped(input_ids=ids, labels=ids)
    torch.testing.assert_close(out.logits, ref.logits, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.loss, ref.loss, atol=1e-6, rtol=1e-6)
    out.loss.backward()

    tpm = wrapped.wrapped_model
    shard0 = tpm.module_shards[0]
    c_fc = shard0.transformer.h[0].mlp.tp_wrapped_module.c_fc.weight.grad
    expected = torch.tensor_split(ref_grads["transformer.h.0.mlp.c_fc.weight"], world, dim=1)[0]
    torch.testing.assert_close(c_fc, expected, atol=1e-6, rtol=1e-4)
    mgr = tpm.sharding_manager
    assert len(mgr.sharded_param_names) == 10  # every LayerNorm weight and bias
    stacked = torch.stack([f.grad for f in mgr.flat_shards])
    for name, grad in zip(mgr.sharded_param_names, mgr._combine(stacked)):
        torch.testing.assert_close(grad, ref_grads[name.replace("tp_wrapped_module.", "")], atol=1e-6, rtol=1e-4)

    sharded_keys = list(wrapped.state_dict().keys())
    assert all(k.startswith("wrapped_model.") for k in sharded_keys)
    assert "wrapped_model.module_shards.0.transformer.h.0.mlp.tp_wrapped_module.c_fc.weight" in sharded_keys
    with tp.save_tensor_parallel(wrapped):
        merged = wrapped.state_dict()
    want = model.state_dict()
    assert set(merged) == set(want)
    for k, v in want.items():
        torch.testing.assert_close(merged[k], v, msg=k)
    fresh = _tiny_gpt2()
    with torch.no_grad():
        for p in fresh.parameters():
            p.zero_()
    fresh.load_state_dict(merged)
    torch.testing.assert_close(fresh(input_ids=ids).logits, ref.logits)


@pytest.mark.parametrize("kwargs", [dict(do_sample=False), dict(num_beams=3, do_sample=False)])
def test_hf_generate(kwargs):
    model = _tiny_gpt2().eval()
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    prompt = torch.randint(0, 1000, (2, 5), generator=torch.Generator().manual_seed(2))
    mask = torch.ones_like(prompt)
    want = model.generate(prompt, attention_mask=mask, max_new_tokens=5, pad_token_id=0, **kwargs)
    got = wrapped.generate(prompt, attention_mask=mask, max_new_tokens=5, pad_token_id=0, **kwargs)
    assert torch.equal(got, want)


def test_fallback_to_autoconfig_for_drifted_models():
    """Llama in current transformers no longer matches the era table (call signature changed);
    the wrapper must notice and fall back instead of mis-slicing."""
    cfg = transformers.LlamaConfig(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                   num_attention_heads=4, num_key_value_heads=4, attn_implementation="eager")
    model = transformers.LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 100, (2, 6))
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"])
    torch.testing.assert_close(wrapped(input_ids=ids).logits, model(input_ids=ids).logits, atol=1e-5, rtol=1e-5)
