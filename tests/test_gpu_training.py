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
        # bf16 gradients vs the fp32 oracle; the absolute term covers gradients that are analytically zero (key bias)
        assert (g - w).norm().item() <= 0.1 * w.norm().item() + 2e-5 * w.numel() ** 0.5, name
    opt = tp.optim.AdamW(model.parameters(), lr=1e-3)
    opt.step()
    torch.cuda.synchronize()
    native.device_state(torch.device("cuda", 0)).check_status()
    out2 = model(input_ids=ids.cuda(), labels=ids.cuda())
    assert out2.loss.item() < out.loss.item()


@pytest.mark.parametrize("vocab", [1024, 4000])
def test_fused_head_cross_entropy_single_rank(vocab):
    from tensor_parallel_b200.ops.loss import lm_head_cross_entropy, lm_head_cross_entropy_ref

    torch.manual_seed(2)
    hidden = (torch.randn(3, 50, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    weight = (torch.randn(vocab, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, vocab, (3, 50), device="cuda")
    labels[0, :7] = -100
    loss = lm_head_cross_entropy(hidden, weight, labels)
    loss.backward()
    h32, w32 = hidden.detach().float().requires_grad_(True), weight.detach().float().requires_grad_(True)
    want = lm_head_cross_entropy_ref(h32, w32, labels)
    want.backward()
    torch.testing.assert_close(loss, want, atol=2e-2, rtol=1e-2)
    for got, ref in ((hidden.grad, h32.grad), (weight.grad, w32.grad)):
        denom = ref.abs().max().item() + 1e-9
        assert (got.float() - ref).abs().max().item() / denom < 0.06
