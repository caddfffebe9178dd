"""Training step on the GPU through the native kernels (bf16): forward, backward and fused AdamW of a
small Llama- and OPT-shaped model stay close to the same step done in fp32 with stock PyTorch."""
import pytest
import torch

import tensor_parallel_b200 as tp
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM
from tensor_parallel_b200.models.opt import OPTConfig, OPTForCausalLM

pytestmark = pytest.mark.gpu


def _build(kind):
    torch.manual_seed(0)
    if kind == "llama":
        cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4)
        return LlamaForCausalLM(cfg), LlamaForCausalLM(cfg)
    cfg = OPTConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, ffn_dim=1024, num_attention_heads=4, max_position_embeddings=128)
    return OPTForCausalLM(cfg), OPTForCausalLM(cfg)


@pytest.mark.parametrize("kind", ["llama", "opt"])
def test_bf16_native_training_step_tracks_fp32_reference(kind):
    from tensor_parallel_b200.ops import native

    ref, model = _build(kind)
    model.load_state_dict(ref.state_dict())
    model = model.to(device="cuda", dtype=torch.bfloat16)
    ref.load_state_dict({k: v.float().cpu() for k, v in model.state_dict().items()})
    ids = torch.randint(0, 512, (4, 96), generator=torch.Generator().manual_seed(1))
    before = native.launch_count
    out = model(input_ids=ids.cuda(), labels=ids.cuda())
    out.loss.backward()
    want = ref(input_ids=ids, labels=ids)
    want.loss.backward()
    assert native.launch_count - before > 20, "the native kernels were not used"
    torch.testing.assert_close(out.loss.float().cpu(), want.loss, atol=3e-2, rtol=2e-2)
    grads = dict(model.named_parameters())
    for name, p in ref.named_parameters():
        g, w = grads[name].grad.float().cpu(), p.grad
        denom = w.abs().max().item() + 1e-6
        assert (g - w).abs().max().item() / denom < 0.08, name
    opt = tp.optim.AdamW(model.parameters(), lr=1e-3)
    opt.step()
    torch.cuda.synchronize()
    native.device_state(torch.device("cuda", 0)).check_status()
    out2 = model(input_ids=ids.cuda(), labels=ids.cuda())
    assert out2.loss.item() < out.loss.item()
