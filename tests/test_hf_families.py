"""Current Hugging Face model classes (random tiny configs, no download) under the predefined rule tables: the logits of the
tensor-parallel wrapper equal those of the unsplit model, with and without ZeRO-3, and a chained cached call works.
The reference's tables patch attributes of 2023-era modules and break on newer ``transformers``; here attribute rules
skip names a module does not have, and both the remote-code and the in-library Falcon attribute names are covered."""
import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import AutoConfig, AutoModelForCausalLM  # noqa: E402

import tensor_parallel_b200 as tp  # noqa: E402

V = 96
CASES = {
    "llama": dict(model_type="llama", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "gpt2": dict(model_type="gpt2", vocab_size=V, n_embd=32, n_layer=2, n_head=4, n_positions=64),
    "bloom": dict(model_type="bloom", vocab_size=V, hidden_size=32, n_layer=2, n_head=4),
    "gpt_neox": dict(model_type="gpt_neox", vocab_size=V, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64),
    "opt": dict(model_type="opt", vocab_size=V, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, ffn_dim=64, max_position_embeddings=64, word_embed_proj_dim=32),
    "gptj": dict(model_type="gptj", vocab_size=V, n_embd=32, n_layer=2, n_head=4, rotary_dim=4, n_positions=64),
    "falcon": dict(model_type="falcon", vocab_size=V, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_kv_heads=2, new_decoder_architecture=True),
    "mistral": dict(model_type="mistral", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "qwen2": dict(model_type="qwen2", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "qwen3": dict(model_type="qwen3", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8),
    "gemma": dict(model_type="gemma", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8),
    "gemma2": dict(model_type="gemma2", vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                   query_pre_attn_scalar=8, sliding_window=16),
    "codegen": dict(model_type="codegen", vocab_size=V, n_embd=64, n_layer=2, n_head=8, rotary_dim=4, n_positions=64),
}


def _model(name):
    torch.manual_seed(0)
    cfg = AutoConfig.for_model(**CASES[name])
    return AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").eval()


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("sharded", [False, True])
def test_hf_decoder_families(name, sharded):
    model = _model(name)
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = model(input_ids=ids).logits
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=sharded)
    assert isinstance(wrapped, tp.TensorParallelPreTrainedModel)
    sums = [a for per in wrapped.tensor_parallel_config.output_rules.values() for a in per.values()
            if a == "sum" or type(a).__name__.endswith("AllReduce")]
    assert sums, "the automatic config was used instead of the family's rule table"
    with torch.no_grad():
        got = wrapped(input_ids=ids).logits
    torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("name", ["llama", "gpt2", "falcon", "mistral", "qwen2", "qwen3", "gemma", "gemma2"])
def test_hf_chained_cache_calls(name):
    model = _model(name)
    a, b = torch.randint(0, V, (2, 5)), torch.randint(0, V, (2, 1))
    with torch.no_grad():
        r1 = model(input_ids=a, use_cache=True)
        r2 = model(input_ids=b, past_key_values=r1.past_key_values, use_cache=True)
    wrapped = tp.tensor_parallel(_model(name), ["cpu", "cpu"])
    with torch.no_grad():
        o1 = wrapped(input_ids=a, use_cache=True)
        o2 = wrapped(input_ids=b, past_key_values=o1.past_key_values, use_cache=True)
    torch.testing.assert_close(o1.logits, r1.logits, atol=3e-5, rtol=1e-4)
    torch.testing.assert_close(o2.logits, r2.logits, atol=3e-5, rtol=1e-4)


def test_hf_t5_forward_and_generate():
    """``transformers`` 5.x T5: the attention modules return their position bias where older versions returned the
    key / value pair, and keep the cache in a stateful object; forward, greedy and beam generation match the unsplit model."""
    from transformers import T5ForConditionalGeneration

    torch.manual_seed(0)
    cfg = AutoConfig.for_model(model_type="t5", vocab_size=V, d_model=32, d_kv=8, d_ff=48, num_layers=2, num_heads=4, decoder_start_token_id=0)
    model = T5ForConditionalGeneration(cfg).eval()
    ids, dec = torch.randint(0, V, (2, 7)), torch.randint(0, V, (2, 4))
    with torch.no_grad():
        want = model(input_ids=ids, decoder_input_ids=dec).logits
    greedy = model.generate(ids, max_new_tokens=5, do_sample=False)
    beams = model.generate(ids, max_new_tokens=5, do_sample=False, num_beams=3)
    for sharded in (False, True):
        wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=sharded)
        with torch.no_grad():
            got = wrapped(input_ids=ids, decoder_input_ids=dec).logits
        torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)
    assert torch.equal(wrapped.generate(ids, max_new_tokens=5, do_sample=False), greedy)
    assert torch.equal(wrapped.generate(ids, max_new_tokens=5, do_sample=False, num_beams=3), beams)


def test_hf_bert_three_ranks_zero3():
    from transformers import BertModel

    torch.manual_seed(0)
    cfg = AutoConfig.for_model(model_type="bert", vocab_size=V, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                               max_position_embeddings=64)
    model = BertModel(cfg).eval()
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = model(input_ids=ids).last_hidden_state
    wrapped = tp.tensor_parallel(model, ["cpu"] * 3, sharded=True)
    with torch.no_grad():
        got = wrapped(input_ids=ids).last_hidden_state
    torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("name", ["llama", "bloom"])
@pytest.mark.parametrize("kwargs", [{}, {"num_beams": 3}])
def test_hf_generate_matches_unsplit(name, kwargs):
    model = _model(name)
    ids = torch.randint(0, V, (2, 6))
    want = model.generate(ids, max_new_tokens=5, do_sample=False, pad_token_id=0, **kwargs)
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"])
    assert torch.equal(wrapped.generate(ids, max_new_tokens=5, do_sample=False, pad_token_id=0, **kwargs), want)


def test_hf_save_pretrained_round_trip(tmp_path):
    """``save_pretrained`` inside ``save_tensor_parallel`` writes a checkpoint that the plain class loads (the reference's
    README flow), here from a ZeRO-3 sharded wrapper."""
    model = _model("llama")
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = model(input_ids=ids).logits
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    with tp.save_tensor_parallel(wrapped):
        wrapped.save_pretrained(str(tmp_path))
    reloaded = AutoModelForCausalLM.from_pretrained(str(tmp_path), attn_implementation="eager").eval()
    with torch.no_grad():
        got = reloaded(input_ids=ids).logits
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("layout", ["multi_query", "multi_query_sequential", "per_head", "grouped"])
@pytest.mark.parametrize("world", [2, 3])
def test_hf_falcon_layouts(layout, world):
    """The four fused-QKV layouts of Falcon: multi-query (falcon-7b: all query heads, then one shared key and value head,
    with the attention / MLP branches in parallel or in sequence), one (q, k, v) triple per head (falcon-rw) and key / value
    groups (falcon-40b).  Chained cached calls and the un-sharded save must match the unsplit model."""
    kw = {"multi_query": dict(multi_query=True, new_decoder_architecture=False, parallel_attn=True),
          "multi_query_sequential": dict(multi_query=True, new_decoder_architecture=False, parallel_attn=False),
          "per_head": dict(multi_query=False, new_decoder_architecture=False, parallel_attn=True),
          "grouped": dict(num_kv_heads=3, new_decoder_architecture=True)}[layout]
    cfg = AutoConfig.for_model(model_type="falcon", vocab_size=V, hidden_size=48, num_hidden_layers=2, num_attention_heads=6, bias=False, alibi=False, **kw)
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").eval()
    a, b = torch.randint(0, V, (2, 7)), torch.randint(0, V, (2, 1))
    with torch.no_grad():
        r1 = model(input_ids=a, use_cache=True)
        r2 = model(input_ids=b, past_key_values=r1.past_key_values, use_cache=True)
    torch.manual_seed(0)
    wrapped = tp.tensor_parallel(AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").eval(), ["cpu"] * world)
    with torch.no_grad():
        o1 = wrapped(input_ids=a, use_cache=True)
        o2 = wrapped(input_ids=b, past_key_values=o1.past_key_values, use_cache=True)
    torch.testing.assert_close(o1.logits, r1.logits, atol=3e-5, rtol=1e-4)
    torch.testing.assert_close(o2.logits, r2.logits, atol=3e-5, rtol=1e-4)
    with tp.save_tensor_parallel(wrapped):
        merged = wrapped.state_dict()
    for key, value in model.state_dict().items():
        assert torch.equal(merged[key], value), key


def test_hf_falcon_too_few_groups_is_refused():
    cfg = AutoConfig.for_model(model_type="falcon", vocab_size=V, hidden_size=48, num_hidden_layers=1, num_attention_heads=6, num_kv_heads=2,
                               new_decoder_architecture=True, bias=False, alibi=False)
    model = AutoModelForCausalLM.from_config(cfg, attn_implementation="eager")
    with pytest.raises(ValueError, match="key/value groups"):
        tp.tensor_parallel(model, ["cpu"] * 3)


@pytest.mark.parametrize("model_type", ["llama", "qwen2"])
@pytest.mark.parametrize("world", [2, 3])
def test_hf_tied_head_keeps_the_tie(model_type, world):
    """``tie_word_embeddings=True`` (small Llama-3.2 / Qwen2 checkpoints): the head shares the hidden-split embedding slice,
    reads its slice of the hidden state and the partial logits are summed; the un-sharded save equals the original."""
    torch.manual_seed(0)
    cfg = AutoConfig.for_model(model_type=model_type, vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=True)
    model = AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").eval()
    assert model.lm_head.weight is model.model.embed_tokens.weight
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = model(input_ids=ids).logits
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    with torch.no_grad():
        got = wrapped(input_ids=ids).logits
    torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)
    with tp.save_tensor_parallel(wrapped):
        merged = wrapped.state_dict()
    assert set(merged) == set(model.state_dict())
    for key, value in model.state_dict().items():
        assert torch.equal(merged[key], value), key


UNEVEN = {
    "llama_2kv_3ranks": (3, dict(model_type="llama", vocab_size=V, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2)),
    "llama_mqa": (2, dict(model_type="llama", vocab_size=V, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=1)),
    "gpt2_4heads_3ranks": (3, CASES["gpt2"]),
    "bloom_4heads_3ranks": (3, CASES["bloom"]),
    "gpt_neox_4heads_3ranks": (3, CASES["gpt_neox"]),
    "opt_4heads_3ranks": (3, CASES["opt"]),
    "gptj_4heads_3ranks": (3, CASES["gptj"]),
}


@pytest.mark.parametrize("case", list(UNEVEN))
def test_hf_uneven_head_splits(case):
    """Head counts that do not divide by the number of ranks (some ranks own one head more; a rank may own none)."""
    world, kw = UNEVEN[case]
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(AutoConfig.for_model(**kw), attn_implementation="eager").eval()
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = model(input_ids=ids).logits
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    with torch.no_grad():
        got = wrapped(input_ids=ids).logits
    torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)


def test_hf_t5_training_step_with_zero3():
    """Seq2seq training step on the Hugging Face T5 class (gated-GeLU, untied head - the FLAN-T5 shape): loss, gradients of
    the tensor-parallel slices and of the ZeRO-3 flat shards equal those of the unsplit model."""
    from transformers import T5ForConditionalGeneration

    torch.manual_seed(0)
    cfg = AutoConfig.for_model(model_type="t5", vocab_size=V, d_model=32, d_kv=8, d_ff=48, num_layers=2, num_heads=4, decoder_start_token_id=0,
                               feed_forward_proj="gated-gelu", tie_word_embeddings=False, dropout_rate=0.0)
    model = T5ForConditionalGeneration(cfg)
    ids, labels = torch.randint(0, V, (2, 7)), torch.randint(0, V, (2, 4))
    ref = model(input_ids=ids, labels=labels)
    ref.loss.backward()
    grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    out = wrapped(input_ids=ids, labels=labels)
    torch.testing.assert_close(out.loss, ref.loss, atol=1e-5, rtol=1e-5)
    out.loss.backward()
    inner = wrapped.wrapped_model
    manager = inner.sharding_manager
    stacked = torch.stack([f.grad for f in manager.flat_shards])
    for name, grad in zip(manager.sharded_param_names, manager._combine(stacked)):
        torch.testing.assert_close(grad, grads[name.replace("tp_wrapped_module.", "")], atol=3e-5, rtol=1e-3, msg=name)
    for rank, shard in enumerate(inner.module_shards):
        for shard_name, p in shard.named_parameters():
            original = shard_name.replace("tp_wrapped_module.", "")
            for pattern, action in inner.tensor_parallel_config.state_rules.items():
                if pattern.search(original):
                    expected = grads[original] if isinstance(action, tp.Scale) else action(grads[original], rank)
                    torch.testing.assert_close(p.grad, expected, atol=3e-5, rtol=1e-3, msg=f"{shard_name}@{rank}")
                    break
