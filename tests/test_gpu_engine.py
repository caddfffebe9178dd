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
