"""Serving engine (kernel-level prefill + CUDA-graph decode) against the module-level forward of the
same weights, which runs in fp32 with stock PyTorch operators."""
import pytest
import torch

import tensor_parallel_b200 as tp
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM

pytestmark = pytest.mark.gpu


def _models(kv_heads, ffn=1376):
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=ffn, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=kv_heads)
    ref = LlamaForCausalLM(cfg)          # fp32 CPU copy = oracle
    model = LlamaForCausalLM(cfg)
    model.load_state_dict(ref.state_dict())
    model = model.to(device="cuda", dtype=torch.bfloat16).eval()
    ref.load_state_dict({k: v.float().cpu() for k, v in model.state_dict().items()})  # same (bf16-rounded) weights
    return ref.eval(), model


@pytest.mark.parametrize("kv_heads,ffn", [(4, 1376), (2, 1376), (4, 344)])  # 344 is not a multiple of the 16-row SwiGLU groups
def test_engine_prefill_and_decode_logits(kv_heads, ffn):
    from tensor_parallel_b200.ops import native

    ref, model = _models(kv_heads, ffn)
    wrapped = tp.tensor_parallel(model, ["cuda:0"])
    ids = torch.randint(0, 1024, (3, 70), generator=torch.Generator().manual_seed(1))
    logits = wrapped.prefill(ids, max_new_tokens=16)
    with torch.no_grad():
        want = ref(input_ids=ids, use_cache=True)
    torch.testing.assert_close(logits.cpu(), want.logits[:, -1], atol=0.08, rtol=0.05)

    engine = wrapped._engine
    nxt = want.logits[:, -1].argmax(-1)
    past = want.past_key_values
    engine.ids[:3].copy_(nxt)
    for step in range(4):  # the first call captures the graph, later calls replay it
        engine.decode_step(3)
        with torch.no_grad():
            out = ref(input_ids=nxt[:, None], past_key_values=past, use_cache=True)
        past = out.past_key_values
        got = engine.logits_local[:3].float().cpu()
        torch.testing.assert_close(got, out.logits[:, -1], atol=0.08, rtol=0.05, msg=f"decode step {step}")
        nxt = out.logits[:, -1].argmax(-1)
        engine.ids[:3].copy_(nxt)  # keep both on the oracle's token choice
    torch.cuda.synchronize()
    native.device_state(torch.device("cuda", 0)).check_status()
    assert engine.graph is not None and engine.kernels_per_step > 0


def test_generate_uses_engine_and_host_driven_steps():
    ref, model = _models(4)
    wrapped = tp.tensor_parallel(model, ["cuda:0"])
    ids = torch.randint(0, 1024, (2, 33), generator=torch.Generator().manual_seed(2))
    out = wrapped.generate(ids, max_new_tokens=6)
    assert out.shape == (2, 39) and wrapped._engine is not None
    assert torch.equal(out[:, :33].cpu(), ids)
    # host-driven stepping reproduces generate()
    logits = wrapped.prefill(ids, max_new_tokens=6)
    tok = logits.argmax(-1).cpu().pin_memory()
    seq = [tok.clone()]
    for _ in range(5):
        tok = wrapped.decode_step(tok).clone().pin_memory()
        seq.append(tok.clone())
    assert torch.equal(torch.stack(seq, 1), out[:, 33:].cpu())


def _agreement(engine_tokens, generic_tokens, prompt_len):
    a, b = engine_tokens[:, prompt_len:].cpu(), generic_tokens[:, prompt_len:].cpu()
    return (a == b).float().mean().item()


def _teacher_forced_decode(wrapped, oracle, ids, steps=6):
    """Prefill + ``steps`` decode steps of the engine against the fp32 module-level forward, both fed the oracle's
    tokens (one flipped near-tie must not derail the comparison); returns the share of steps with the same arg-max."""
    batch = ids.shape[0]
    logits = wrapped.prefill(ids, max_new_tokens=steps + 4)
    with torch.no_grad():
        want = oracle(input_ids=ids, use_cache=True)
    torch.testing.assert_close(logits.cpu(), want.logits[:, -1], atol=0.08, rtol=0.05)
    engine = wrapped._engine
    nxt, past = want.logits[:, -1].argmax(-1), want.past_key_values
    same = 0
    for step in range(steps):
        engine.ids[:batch].copy_(nxt)
        engine.decode_step(batch)
        with torch.no_grad():
            out = oracle(input_ids=nxt[:, None], past_key_values=past, use_cache=True)
        past = out.past_key_values
        got = engine.logits_local[:batch].float().cpu()
        torch.testing.assert_close(got, out.logits[:, -1], atol=0.08, rtol=0.05, msg=f"decode step {step}")
        nxt = out.logits[:, -1].argmax(-1)
        same += int((engine.next_ids[:batch].cpu() == nxt).sum())
    return same / float(steps * batch)


def _bf16_rounded(model):
    """fp32 oracle (CPU) and bf16 CUDA copy holding exactly the same (bf16-representable) weights."""
    import copy

    served = copy.deepcopy(model).to(device="cuda", dtype=torch.bfloat16).eval()
    oracle = copy.deepcopy(model).float().eval()
    oracle.load_state_dict({k: v.float().cpu() for k, v in served.state_dict().items()})
    return oracle, served


def test_engine_serves_falcon_shaped_model():
    """Parallel attention + MLP block with two LayerNorms, grouped fused QKV, GeLU, tied head: the engine runs four
    kernels per layer and must track the fp32 module-level forward."""
    from tensor_parallel_b200.models.falcon import FalconConfig, FalconForCausalLM
    from tensor_parallel_b200.models.generation import generate

    torch.manual_seed(0)
    cfg = FalconConfig(vocab_size=1024, hidden_size=512, n_layer=3, n_head=8, n_head_kv=2)
    oracle, served = _bf16_rounded(FalconForCausalLM(cfg))
    wrapped = tp.tensor_parallel(served, ["cuda:0"])
    ids = torch.randint(0, 1024, (3, 70), generator=torch.Generator().manual_seed(1))
    assert _teacher_forced_decode(wrapped, oracle, ids) >= 0.9
    assert wrapped._engine is not None and wrapped._engine.parallel
    assert wrapped._engine.kernels_per_step <= 4 * cfg.n_layer + 8
    got = wrapped.generate(ids, max_new_tokens=10)  # free-running: the first new token, at least, is the oracle's
    ref = generate(oracle, ids, max_new_tokens=10)
    assert got.shape == ref.shape and torch.equal(got[:, :71].cpu(), ref[:, :71].cpu())
    wrapped._engine.check_status()


def test_engine_serves_opt_shaped_model():
    """Learned positions, LayerNorm with bias, biased projections, ReLU, tied head."""
    from tensor_parallel_b200.models.generation import generate
    from tensor_parallel_b200.models.opt import OPTConfig, OPTForCausalLM

    torch.manual_seed(0)
    cfg = OPTConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=3, ffn_dim=1024, num_attention_heads=8, max_position_embeddings=256)
    model = OPTForCausalLM(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("bias"):
                p.normal_(0.0, 0.05)
            if "layer_norm.weight" in name:
                p.add_(0.1 * torch.randn_like(p))
    oracle, served = _bf16_rounded(model)
    wrapped = tp.tensor_parallel(served, ["cuda:0"])
    ids = torch.randint(0, 1024, (2, 70), generator=torch.Generator().manual_seed(1))
    assert _teacher_forced_decode(wrapped, oracle, ids) >= 0.9
    assert wrapped._engine is not None and not wrapped._engine.parallel
    got = wrapped.generate(ids, max_new_tokens=10)
    ref = generate(oracle, ids, max_new_tokens=10)
    assert got.shape == ref.shape and torch.equal(got[:, :71].cpu(), ref[:, :71].cpu())
    wrapped._engine.check_status()


def test_engine_serves_hugging_face_llama():
    """``transformers`` ``LlamaForCausalLM`` (GQA) wrapped by the HF-aware wrapper: greedy ``generate()`` runs on the engine
    and agrees with the stock Hugging Face loop on the fp32 model."""
    transformers = pytest.importorskip("transformers")
    from tensor_parallel_b200.ops import native

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1376, num_hidden_layers=3,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512)
    hf = transformers.LlamaForCausalLM(cfg).eval()
    oracle, served = _bf16_rounded(hf)
    wrapped = tp.tensor_parallel(served, ["cuda:0"])
    ids = torch.randint(0, 1024, (2, 40), generator=torch.Generator().manual_seed(1))
    before = native.launch_count
    got = wrapped.generate(ids.cuda(), max_new_tokens=10, do_sample=False)
    assert native.launch_count - before > 50, "greedy generate() of a Hugging Face Llama did not reach the native engine"
    ref = oracle.generate(ids, max_new_tokens=10, do_sample=False)
    assert got.shape == ref.shape and _agreement(got, ref, 40) >= 0.6  # free-running: near-ties may flip and derail a sequence
    assert torch.equal(got[:, :41].cpu(), ref[:, :41])


def test_engine_is_rebuilt_after_a_weight_update():
    """The engine owns serving-layout copies; writing to the shard's parameters must invalidate them."""
    ref, model = _models(4)
    wrapped = tp.tensor_parallel(model, ["cuda:0"])
    ids = torch.randint(0, 1024, (2, 20), generator=torch.Generator().manual_seed(3))
    first = wrapped.prefill(ids, max_new_tokens=4)
    engine = wrapped._engine
    with torch.no_grad():
        wrapped.module_shards[0].model.layers[0].mlp.gate_proj.weight.mul_(-1.0)
    second = wrapped.prefill(ids, max_new_tokens=4)
    assert wrapped._engine is not engine
    assert (first - second).abs().max().item() > 1e-3


def test_release_training_weights_keeps_serving_and_frees_memory():
    """After ``release_training_weights()`` the engine answers exactly as before from its own layout, the parameters it
    copied are gone from the device, the ones it reads in place are still there, and a rebuild is refused."""
    import gc

    _, model = _models(2)
    wrapped = tp.tensor_parallel(model, ["cuda:0"])
    ids = torch.randint(0, 1024, (2, 40), generator=torch.Generator().manual_seed(4))
    before_logits = wrapped.prefill(ids, max_new_tokens=8).clone()
    before_tokens = wrapped.generate(ids, max_new_tokens=6).clone()
    gc.collect()
    torch.cuda.synchronize()
    allocated = torch.cuda.memory_allocated()
    freed = wrapped.release_training_weights()
    shard = wrapped.module_shards[0]
    layer = shard.model.layers[0]
    total = sum(p.numel() * 2 for p in _models(2)[1].parameters())
    assert freed > 0.5 * total, (freed, total)                       # q / k / v, gate / up, norms, head
    assert allocated - torch.cuda.memory_allocated() >= 0.9 * freed  # really returned to the allocator
    assert layer.self_attn.q_proj.weight.numel() == 0 and layer.mlp.gate_proj.weight.numel() == 0
    assert layer.self_attn.o_proj.weight.numel() > 0 and layer.mlp.down_proj.weight.numel() > 0  # read in place by the engine
    torch.testing.assert_close(wrapped.prefill(ids, max_new_tokens=8), before_logits, atol=0, rtol=0)
    assert torch.equal(wrapped.generate(ids, max_new_tokens=6), before_tokens)
    with pytest.raises(RuntimeError, match="released"):
        wrapped.serving_engine(max_batch=64, max_seq=8192)
