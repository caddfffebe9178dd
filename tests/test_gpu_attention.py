"""Attention kernels against the fp32 reference ``attention_ref`` (same masking convention)."""
import pytest
import torch

from tensor_parallel_b200.ops import functional as OF

pytestmark = pytest.mark.gpu


def _native():
    from tensor_parallel_b200.ops import native

    return native


CASES = [
    # batch, sq, sk, hq, hkv, d, causal
    (2, 128, 128, 4, 4, 128, True),
    (1, 200, 200, 8, 2, 64, True),     # GQA, ragged
    (2, 77, 77, 4, 4, 64, False),      # bidirectional (encoder)
    (1, 64, 300, 4, 1, 128, True),     # chunked prefill on top of a cache (MQA)
    (1, 5, 133, 2, 2, 64, False),      # cross attention shape
    (1, 1024, 1024, 2, 2, 128, True),
]


@pytest.mark.parametrize("b,sq,sk,hq,hkv,d,causal", CASES)
def test_prefill_attention(b, sq, sk, hq, hkv, d, causal):
    nat = _native()
    torch.manual_seed(0)
    q = torch.randn(b, sq, hq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16)
    out, lse = nat.attention_forward(q, k, v, causal, None, want_lse=True)
    ref = OF.attention_ref(q.float(), k.float(), v.float(), causal)
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.isfinite(lse).all()


@pytest.mark.parametrize("kind", ["relative_fp32", "padding_bf16", "alibi_causal", "full_bf16"])
def test_prefill_attention_additive_bias(kind):
    """Score biases of the model families: T5 relative positions [1,H,Sq,Sk], padding masks [B,1,1,Sk] with -inf,
    ALiBi slopes [1,H,1,Sk] under a causal mask, and a dense per-batch bias."""
    nat = _native()
    torch.manual_seed(3)
    b, sq, sk, h, d = 2, 150, 150, 4, 64
    q = torch.randn(b, sq, h, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, sk, h, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, sk, h, d, device="cuda", dtype=torch.bfloat16)
    causal = False
    if kind == "relative_fp32":
        bias = torch.randn(1, h, sq, sk, device="cuda")
    elif kind == "padding_bf16":
        bias = torch.zeros(b, 1, 1, sk, device="cuda", dtype=torch.bfloat16)
        bias[0, :, :, 100:] = float("-inf")
        bias[1, :, :, 37:] = float("-inf")
    elif kind == "alibi_causal":
        slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625], device="cuda")
        bias = (slopes[None, :, None, None] * torch.arange(sk, device="cuda")[None, None, None, :]).to(torch.bfloat16)
        causal = True
    else:
        bias = torch.randn(b, h, sq, sk, device="cuda", dtype=torch.bfloat16)
    assert nat.attention_supported(q, k, v, bias)
    out = OF.attention(q, k, v, causal, bias=bias)
    ref = OF.attention_ref(q.float(), k.float(), v.float(), causal, bias=bias.float())
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert nat.attention_supported(q.requires_grad_(), k, v, bias)  # training with a bias runs on the native kernels too


def test_prefill_attention_reads_cache_layout():
    """k / v handed over as transposed views of a [B, H, S, D] cache (strides, no copy)."""
    nat = _native()
    torch.manual_seed(1)
    b, s, h, d = 2, 96, 4, 128
    q = torch.randn(b, s, h, d, device="cuda", dtype=torch.bfloat16)
    kc = torch.randn(b, h, 256, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(b, h, 256, d, device="cuda", dtype=torch.bfloat16)
    k, v = kc[:, :, :s].transpose(1, 2), vc[:, :, :s].transpose(1, 2)
    out, _ = nat.attention_forward(q, k, v, True, None)
    torch.testing.assert_close(out.float(), OF.attention_ref(q.float(), k.float(), v.float(), True), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hq,hkv,d", [(8, 8, 128), (8, 2, 128), (16, 1, 64), (32, 32, 128), (6, 2, 64)])
@pytest.mark.parametrize("splits", [1, 4])
def test_decode_attention_with_cache_append(hq, hkv, d, splits):
    nat = _native()
    torch.manual_seed(2)
    b, ctx, smax = 3, 201, 256
    kc = torch.zeros(b, hkv, smax, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc[:, :, :ctx] = torch.randn(b, hkv, ctx, d, device="cuda")
    vc[:, :, :ctx] = torch.randn(b, hkv, ctx, d, device="cuda")
    qkv = torch.randn(b, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
    q2, k2, v2 = qkv[:, : hq * d], qkv[:, hq * d : (hq + hkv) * d], qkv[:, (hq + hkv) * d :]
    base = torch.tensor([ctx], device="cuda", dtype=torch.int32)
    q_out = torch.empty(b, hq, d, device="cuda", dtype=torch.bfloat16)
    nat.qkv_rope_append(q2, k2, v2, q_out, kc, vc, base, b, 1, d, 10000.0)
    out = nat.attn_decode(q_out, kc, vc, base, 1, splits=splits)

    pos = torch.full((b, 1), ctx, device="cuda")
    q_ref = OF.apply_rope_ref(q2.reshape(b, 1, hq, d).float(), pos, 10000.0)
    k_new = OF.apply_rope_ref(k2.reshape(b, 1, hkv, d).float(), pos, 10000.0)
    torch.testing.assert_close(kc[:, :, ctx].float(), k_new[:, 0], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(vc[:, :, ctx], v2.reshape(b, hkv, d))
    k_all = kc[:, :, : ctx + 1].transpose(1, 2).float()
    v_all = vc[:, :, : ctx + 1].transpose(1, 2).float()
    ref = OF.attention_ref(q_out.reshape(b, 1, hq, d).float(), k_all, v_all, causal=True)
    torch.testing.assert_close(out.reshape(b, 1, hq, d).float(), ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(q_out.float(), q_ref[:, 0], atol=2e-2, rtol=2e-2)


BWD_CASES = [
    (2, 128, 128, 4, 4, 128, True),
    (1, 200, 200, 8, 2, 64, True),    # GQA, ragged
    (2, 77, 77, 4, 4, 64, False),     # bidirectional
    (1, 64, 300, 4, 1, 128, True),    # cached prefix, MQA
    (1, 37, 133, 2, 2, 64, False),    # cross attention
    (1, 384, 384, 4, 2, 128, True),   # several resident tiles and streamed steps, GQA
    (2, 300, 300, 2, 2, 64, True),    # ragged ends on both sides
    (1, 256, 512, 2, 1, 128, True),   # cached prefix over several tiles, MQA
    (1, 130, 260, 2, 2, 128, False),  # ragged cross attention
    (1, 512, 512, 2, 2, 128, False),
]


@pytest.mark.parametrize("b,sq,sk,hq,hkv,d,causal", BWD_CASES)
def test_attention_backward(b, sq, sk, hq, hkv, d, causal):
    nat = _native()
    torch.manual_seed(3)
    q = torch.randn(b, sq, hq, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(b, sq, hq, d, device="cuda", dtype=torch.bfloat16)
    out = nat.attention(q, k, v, causal)
    out.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    OF.attention_ref(qr, kr, vr, causal).backward(g.float())
    for name, got, want in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (got.float() - want).norm().item() / (want.norm().item() + 1e-9)
        assert err < 0.03, (name, err)


@pytest.mark.parametrize("interleaved,rotary_dim", [(False, 128), (False, 64), (True, 128), (True, 32)])
def test_rope_append_variants(interleaved, rotary_dim):
    """Prefill-sized append (many tokens per sequence) with full / partial and split / interleaved rotary layouts."""
    nat = _native()
    torch.manual_seed(4)
    b, s, hq, hkv, d, smax, base = 2, 37, 4, 2, 128, 64, 5
    qkv = torch.randn(b * s, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
    q2, k2, v2 = qkv[:, : hq * d], qkv[:, hq * d : (hq + hkv) * d], qkv[:, (hq + hkv) * d :]
    kc = torch.zeros(b, hkv, smax, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(b * s, hq, d, device="cuda", dtype=torch.bfloat16)
    pos0 = torch.tensor([base], device="cuda", dtype=torch.int32)
    nat.qkv_rope_append(q2, k2, v2, q_out, kc, vc, pos0, b, s, rotary_dim, 10000.0, interleaved=interleaved)
    pos = torch.arange(base, base + s, device="cuda")[None].expand(b, s)
    q_ref = OF.apply_rope_ref(q2.reshape(b, s, hq, d).float(), pos, 10000.0, rotary_dim, interleaved)
    k_ref = OF.apply_rope_ref(k2.reshape(b, s, hkv, d).float(), pos, 10000.0, rotary_dim, interleaved)
    torch.testing.assert_close(q_out.view(b, s, hq, d).float(), q_ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(kc[:, :, base : base + s].transpose(1, 2).float(), k_ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(vc[:, :, base : base + s].transpose(1, 2), v2.reshape(b, s, hkv, d))
    assert kc[:, :, :base].abs().sum().item() == 0 and kc[:, :, base + s :].abs().sum().item() == 0


@pytest.mark.parametrize("hq,hkv,d", [(8, 8, 128), (8, 2, 128), (16, 1, 64), (6, 2, 64), (8, 1, 128), (24, 1, 64)])
@pytest.mark.parametrize("splits,angle_table", [(1, False), (4, False), (4, True)])
def test_fused_decode_step_matches_separate_kernels(hq, hkv, d, splits, angle_table):
    """rope + append + attention + split merge in one launch vs the three stand-alone kernels, two steps in a row."""
    nat = _native()
    torch.manual_seed(5)
    b, ctx, smax = 3, 150, 256
    kc = torch.zeros(b, hkv, smax, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc[:, :, :ctx] = torch.randn(b, hkv, ctx, d, device="cuda")
    vc[:, :, :ctx] = torch.randn(b, hkv, ctx, d, device="cuda")
    kc2, vc2 = kc.clone(), vc.clone()
    pos = torch.tensor([ctx], device="cuda", dtype=torch.int32)
    ws = None
    angles = nat.rope_table(smax, d, 10000.0, torch.device("cuda", 0)) if angle_table else None  # looked up instead of sincosf
    for step in range(2):
        qkv = torch.randn(b, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
        q2, k2, v2 = qkv[:, : hq * d], qkv[:, hq * d : (hq + hkv) * d], qkv[:, (hq + hkv) * d :]
        q_out = torch.empty(b, hq, d, device="cuda", dtype=torch.bfloat16)
        nat.qkv_rope_append(q2, k2, v2, q_out, kc, vc, pos, b, 1, d, 10000.0)
        want = nat.attn_decode(q_out, kc, vc, pos, 1, splits=splits)
        if ws is None and splits > 1:
            ws = (torch.empty(b * hq * splits * d, device="cuda"), torch.empty(b * hq * splits * 2, device="cuda"),
                  # one counter per KV head: a launch per group of query heads; one per query head: the groups share a launch
                  torch.zeros(b * (hq if angle_table else hkv), dtype=torch.int32, device="cuda"))
        before = nat.launch_count
        got = nat.attn_decode_fused(q2, k2, v2, kc2, vc2, pos, d, 10000.0, splits=splits, workspace=ws, rope_angles=angles)
        if angle_table and (hq // hkv) in (8, 16) and (hq // hkv) > (4 if d == 128 else 8) - 1 and (hq // hkv) % (4 if d == 128 else 8) == 0:
            assert nat.launch_count - before == 1, "equal groups of query heads should share one launch"
        torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(kc2, kc)
        torch.testing.assert_close(vc2, vc)
        pos += 1


BIAS_BWD_CASES = [
    # b, sq, sk, hq, hkv, d, causal, bias shape
    (2, 96, 96, 4, 4, 64, False, (1, 4, 96, 96)),     # T5 relative-position bias: broadcast over the batch, trainable
    (2, 130, 130, 4, 2, 64, True, (1, 4, 1, 130)),    # ALiBi-like: broadcast over batch and queries
    (3, 64, 200, 2, 2, 128, False, (3, 1, 1, 200)),   # padding mask per sequence (with -inf entries), cross attention
    (1, 200, 200, 4, 4, 128, True, (1, 4, 200, 200)),
]


@pytest.mark.parametrize("b,sq,sk,hq,hkv,d,causal,bias_shape", BIAS_BWD_CASES)
def test_attention_backward_with_score_bias(b, sq, sk, hq, hkv, d, causal, bias_shape):
    """Forward and backward with an additive score bias, bias gradient included, against fp32 autograd of the same math."""
    nat = _native()
    torch.manual_seed(9)
    q = torch.randn(b, sq, hq, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, sk, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(bias_shape, device="cuda", dtype=torch.float32)
    masked = bias_shape[0] == b and bias_shape[2] == 1 and b > 1
    if masked:  # the last keys of every sequence but the first are padding
        bias = torch.zeros(bias_shape, device="cuda")
        for i in range(1, b):
            bias[i, :, :, sk - 17 * i:] = float("-inf")
    else:
        bias.requires_grad_(True)
    g = torch.randn(b, sq, hq, d, device="cuda", dtype=torch.bfloat16)
    out = nat.attention(q, k, v, causal, bias=bias)
    out.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    br = bias.detach().clone().requires_grad_(not masked)
    ref = OF.attention_ref(qr, kr, vr, causal, bias=br)
    ref.backward(g.float())
    torch.testing.assert_close(out.float(), ref.detach(), atol=3e-2, rtol=3e-2)
    checks = [("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)]
    if not masked:
        checks.append(("dbias", bias.grad, br.grad))
    for name, got, want in checks:
        err = (got.float() - want).norm().item() / (want.norm().item() + 1e-9)
        assert err < 0.03, (name, err)
