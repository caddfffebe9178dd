"""Predefined rule tables on the self-contained model zoo: logits, chained KV-cache calls,
generation (greedy / beam / top-p) and the un-sharded save, each against the unsplit model.
Modelled on the reference's ``tests/test_transformers.py`` (three chained calls with
``past_key_values``; first generation steps' scores equal)."""
import pytest
import torch

import tensor_parallel_b200 as tp
from tensor_parallel_b200.models.bert import BertConfig, BertModel
from tensor_parallel_b200.models.bloom import BloomConfig, BloomForCausalLM
from tensor_parallel_b200.models.falcon import FalconConfig, FalconForCausalLM
from tensor_parallel_b200.models.generation import generate
from tensor_parallel_b200.models.gpt2 import GPT2Config, GPT2LMHeadModel
from tensor_parallel_b200.models.gpt_neox import GPTNeoXConfig, GPTNeoXForCausalLM
from tensor_parallel_b200.models.gptj import CodeGenConfig, CodeGenForCausalLM, GPTJConfig, GPTJForCausalLM
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM
from tensor_parallel_b200.models.opt import OPTConfig, OPTForCausalLM
from tensor_parallel_b200.models.t5 import T5Config, T5ForConditionalGeneration
from tensor_parallel_b200.parallel.hf import get_parallel_encoder

V = 120
DECODERS = {
    "llama": lambda: LlamaForCausalLM(LlamaConfig(vocab_size=V, hidden_size=64, intermediate_size=172, num_hidden_layers=2, num_attention_heads=8)),
    "llama_gqa": lambda: LlamaForCausalLM(LlamaConfig(vocab_size=V, hidden_size=64, intermediate_size=172, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=4)),
    "gpt2": lambda: GPT2LMHeadModel(GPT2Config(vocab_size=V, n_positions=64, n_embd=64, n_layer=2, n_head=4)),
    "opt": lambda: OPTForCausalLM(OPTConfig(vocab_size=V, hidden_size=64, num_hidden_layers=2, ffn_dim=128, num_attention_heads=4, max_position_embeddings=64)),
    "falcon": lambda: FalconForCausalLM(FalconConfig(vocab_size=V, hidden_size=64, n_layer=2, n_head=8, n_head_kv=4)),
    "bloom": lambda: BloomForCausalLM(BloomConfig(vocab_size=V, hidden_size=64, n_layer=2, n_head=8)),
    "gptj": lambda: GPTJForCausalLM(GPTJConfig(vocab_size=V, n_embd=64, n_layer=2, n_head=8, rotary_dim=4)),
    "codegen": lambda: CodeGenForCausalLM(CodeGenConfig(vocab_size=V, n_embd=64, n_layer=2, n_head=8, rotary_dim=4)),
    "gpt_neox": lambda: GPTNeoXForCausalLM(GPTNeoXConfig(vocab_size=V, hidden_size=64, num_hidden_layers=2, num_attention_heads=8)),
}


def _worlds(name):
    return [2] if name == "codegen" else [2, 3]  # codegen deals heads in units of 4 (8 heads -> 2 units)


@pytest.mark.parametrize("name", list(DECODERS))
@pytest.mark.parametrize("sharded", [False, True])
def test_decoder_forward_and_cache(name, sharded):
    torch.manual_seed(0)
    model = DECODERS[name]()
    ids = torch.randint(0, V, (3, 12))
    for world in _worlds(name):
        wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=sharded)
        assert wrapped.tensor_parallel_config is not None
        ref_past = tp_past = None
        for chunk in (ids[:, :3], ids[:, 3:4], ids[:, 4:6]):  # three chained calls: 3, 1, 2 tokens
            ref = model(input_ids=chunk, past_key_values=ref_past, use_cache=True)
            out = wrapped(input_ids=chunk, past_key_values=tp_past, use_cache=True)
            torch.testing.assert_close(out.logits, ref.logits, atol=3e-5, rtol=1e-5)
            ref_past, tp_past = ref.past_key_values, out.past_key_values
        assert isinstance(tp_past[0][0], tp.PerDeviceTensors)
        assert tp_past[0][0].shape[2] == 6


@pytest.mark.parametrize("name", ["llama_gqa", "gpt2", "falcon", "bloom"])
@pytest.mark.parametrize("mode", ["greedy", "beam", "top_p"])
def test_generate(name, mode):
    torch.manual_seed(0)
    model = DECODERS[name]()
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    prompt = torch.randint(0, V, (2, 5))
    kwargs = {"greedy": {}, "beam": {"num_beams": 3}, "top_p": {"do_sample": True, "top_p": 0.5}}[mode]
    gens = {}
    for key, m in (("ref", model), ("tp", wrapped)):
        extra = {"generator": torch.Generator().manual_seed(7)} if mode == "top_p" else {}
        gens[key] = generate(m, prompt, max_new_tokens=3, output_scores=True, **kwargs, **extra)
    for s_ref, s_tp in zip(gens["ref"][1], gens["tp"][1]):
        finite = torch.isfinite(s_ref)
        torch.testing.assert_close(s_tp[finite], s_ref[finite], atol=3e-4, rtol=1e-4)
    if mode != "top_p":
        assert torch.equal(gens["ref"][0], gens["tp"][0])


@pytest.mark.parametrize("name", list(DECODERS))
def test_training_step_matches_unsplit(name):
    """Loss, parameter gradients of TP slices and of ZeRO-3 flat shards after one backward."""
    torch.manual_seed(0)
    model = DECODERS[name]()
    ids = torch.randint(0, V, (2, 10))
    ref = model(input_ids=ids, labels=ids)
    ref.loss.backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    world = 2
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    out = wrapped(input_ids=ids, labels=ids)
    torch.testing.assert_close(out.loss, ref.loss, atol=1e-5, rtol=1e-5)
    out.loss.backward()
    cfg = wrapped.tensor_parallel_config
    checked = 0
    for rank, shard in enumerate(wrapped.module_shards):
        for shard_name, p in shard.named_parameters():
            original = shard_name.replace("tp_wrapped_module.", "")
            for pattern, action in cfg.state_rules.items():
                if pattern.search(original):
                    if isinstance(action, tp.Scale):
                        # a scaled bias b/W is added on every rank, so dL/d(b/W) is the full bias gradient
                        expected = ref_grads[original]
                    else:
                        expected = action(ref_grads[original], rank)
                    torch.testing.assert_close(p.grad, expected, atol=2e-5, rtol=1e-4, msg=f"{shard_name} rank {rank}")
                    checked += 1
                    break
    assert checked > 0
    mgr = wrapped.sharding_manager
    stacked = torch.stack([f.grad for f in mgr.flat_shards])
    for shard_name, grad in zip(mgr.sharded_param_names, mgr._combine(stacked)):
        torch.testing.assert_close(grad, ref_grads[shard_name.replace("tp_wrapped_module.", "")], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("split_cross", [True, False])
def test_t5(world, split_cross):
    from tensor_parallel_b200.parallel.families.encoders import get_t5_config

    torch.manual_seed(0)
    model = T5ForConditionalGeneration(T5Config(vocab_size=V, d_model=64, d_kv=8, d_ff=96, num_layers=2, num_heads=6,
                                                feed_forward_proj="gated-gelu", tie_word_embeddings=False))
    src, tgt = torch.randint(0, V, (3, 10)), torch.randint(0, V, (3, 5))
    ref = model(input_ids=src, labels=tgt)
    cfg = get_t5_config(model.config, ["cpu"] * world, split_cross_attention=split_cross)
    wrapped = tp.TensorParallel(model, ["cpu"] * world, tensor_parallel_config=cfg, sharded=True)
    out = wrapped(input_ids=src, labels=tgt)
    torch.testing.assert_close(out.logits, ref.logits, atol=3e-5, rtol=1e-5)
    torch.testing.assert_close(out.loss, ref.loss, atol=1e-5, rtol=1e-5)
    n_zero3 = len(wrapped.sharding_manager.sharded_param_names)
    # with cross-attention left replicated (the reference's table) ZeRO-3 also owns its q/k/v/o weights
    assert n_zero3 == (12 if split_cross else 12 + 2 * 4)
    # cached decoding: encoder output + 2 tokens, then 1 more with the cache
    r1 = model(input_ids=src, decoder_input_ids=tgt[:, :2], use_cache=True)
    r2 = model(input_ids=src, decoder_input_ids=tgt[:, 2:3], past_key_values=r1.past_key_values, use_cache=True)
    o1 = wrapped(input_ids=src, decoder_input_ids=tgt[:, :2], use_cache=True)
    o2 = wrapped(input_ids=src, decoder_input_ids=tgt[:, 2:3], past_key_values=o1.past_key_values, use_cache=True)
    torch.testing.assert_close(o2.logits, r2.logits, atol=3e-5, rtol=1e-5)
    # a cache produced by the unsplit model (plain full-head tensors) is cut per rank on the fly
    if split_cross:
        o3 = wrapped(input_ids=src, decoder_input_ids=tgt[:, 2:3], past_key_values=r1.past_key_values, use_cache=True)
        torch.testing.assert_close(o3.logits, r2.logits, atol=3e-5, rtol=1e-5)
    # parallel encoder (generate() of encoder-decoder models calls it once)
    enc = get_parallel_encoder(wrapped)(input_ids=src)
    torch.testing.assert_close(enc.last_hidden_state, model.get_encoder()(input_ids=src).last_hidden_state, atol=3e-5, rtol=1e-5)


@pytest.mark.parametrize("world", [2, 3])
def test_bert(world):
    torch.manual_seed(0)
    model = BertModel(BertConfig(vocab_size=V, hidden_size=64, num_hidden_layers=2, num_attention_heads=8, intermediate_size=128, max_position_embeddings=32))
    ids = torch.randint(0, V, (3, 10))
    mask = torch.ones(3, 10)
    mask[1, 7:] = 0
    ref = model(input_ids=ids, attention_mask=mask).last_hidden_state
    wrapped = tp.tensor_parallel(model, ["cpu"] * world, sharded=True)
    torch.testing.assert_close(wrapped(input_ids=ids, attention_mask=mask).last_hidden_state, ref, atol=3e-5, rtol=1e-5)


def test_predefined_table_lookup():
    for key in ("bloom", "t5", "bert", "gpt2", "gptj", "gpt_neox", "codegen", "llama", "opt", "RefinedWeb", "RefinedWebModel", "falcon"):
        assert key in tp.PREDEFINED_CONFIGS
    cfg = tp.find_predefined_tensor_parallel_config(LlamaConfig(num_hidden_layers=1), ["cpu", "cpu"])
    assert isinstance(cfg, tp.Config)

    class Unknown:
        model_type = "not-a-model"

    assert tp.find_predefined_tensor_parallel_config(Unknown(), ["cpu", "cpu"]) is None


@pytest.mark.parametrize("name", ["falcon", "gptj", "codegen", "gpt_neox"])
def test_parallel_blocks_use_a_single_all_reduce(name):
    """The planner merges the two "sum" sites of parallel attention+MLP blocks; fuse=False keeps the reference's two."""
    from tensor_parallel_b200.parallel import collectives as C

    torch.manual_seed(0)
    model = DECODERS[name]()
    ids = torch.randint(0, V, (2, 9))
    ref = model(input_ids=ids, labels=ids)
    calls = {"n": 0}
    original = C.ThreadAllReduce.__call__

    def counting(self, x, rank):
        if rank == 0:
            calls["n"] += 1
        return original(self, x, rank)

    C.ThreadAllReduce.__call__ = counting
    try:
        merged = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=False)
        out = merged(input_ids=ids, labels=ids)
        n_merged = calls["n"]
        calls["n"] = 0
        plain = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=False, fuse=False)
        out_plain = plain(input_ids=ids, labels=ids)
        n_plain = calls["n"]
    finally:
        C.ThreadAllReduce.__call__ = original
    layers = 2
    assert n_plain - n_merged == layers, (n_plain, n_merged)
    torch.testing.assert_close(out.logits, ref.logits, atol=3e-5, rtol=1e-5)
    torch.testing.assert_close(out_plain.logits, ref.logits, atol=3e-5, rtol=1e-5)
    out.loss.backward()


@pytest.mark.parametrize("name", list(DECODERS))
def test_bare_model_uses_the_family_table(name):
    """The reference's ``test_multipurpose_configs``: the same rule table serves the model with and without its head.
    Wrapping the bare transformer must pick the predefined table (row-parallel ``"sum"`` rules), not the automatic one."""
    torch.manual_seed(0)
    full = DECODERS[name]()
    base = next(m for n, m in full.named_children() if n in ("model", "transformer", "gpt_neox"))
    ids = torch.randint(0, V, (2, 7))
    with torch.no_grad():
        want = base(input_ids=ids)
    want = want["last_hidden_state"] if hasattr(want, "keys") else want[0]
    wrapped = tp.tensor_parallel(base, ["cpu", "cpu"])
    sums = [a for per_module in wrapped.tensor_parallel_config.output_rules.values() for a in per_module.values()
            if a == "sum" or type(a).__name__.endswith("AllReduce")]
    assert sums, "automatic config was used (it never sums partial outputs of attention / MLP blocks)"
    with torch.no_grad():
        got = wrapped(input_ids=ids)
    got = got["last_hidden_state"] if hasattr(got, "keys") else got[0]
    torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("name", ["bloom", "gpt2"])
@pytest.mark.parametrize("beams", [1, 3])
def test_generate_from_inputs_embeds(name, beams):
    """The reference's ``test_generate_inputs_embeds``: the prompt is given as embeddings; the tensor-parallel wrapper must
    produce the same step scores and tokens as the unsplit model, and the same tokens as the id prompt those embeddings
    came from."""
    torch.manual_seed(0)
    model = DECODERS[name]()
    prompt = torch.randint(0, V, (2, 5))
    table = model.transformer.word_embeddings if name == "bloom" else model.transformer.wte
    embeds = table(prompt).detach()
    kwargs = {"num_beams": beams} if beams > 1 else {}
    ref_ids, ref_scores = generate(model, inputs_embeds=embeds, max_new_tokens=3, output_scores=True, **kwargs)
    from_ids = generate(model, prompt, max_new_tokens=3, **kwargs)
    assert ref_ids.shape == (2, 3) and torch.equal(ref_ids, from_ids[:, 5:])
    wrapped = tp.tensor_parallel(model, ["cpu", "cpu"], sharded=True)
    tp_ids, tp_scores = generate(wrapped, inputs_embeds=embeds, max_new_tokens=3, output_scores=True, **kwargs)
    for a, b in zip(ref_scores, tp_scores):
        torch.testing.assert_close(b, a, atol=3e-4, rtol=1e-4)
    assert torch.equal(tp_ids, ref_ids)
    assert torch.equal(wrapped.generate(inputs_embeds=embeds, max_new_tokens=3, **kwargs), ref_ids)
