"""tcgen05 GEMM against an fp32 PyTorch reference of the same operation (bf16 inputs)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _native():
    from tensor_parallel_b200.ops import native

    return native


def _ref(x, w, bias=None, residual=None, act=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = torch.nn.functional.gelu(y)
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "silu":
        y = torch.nn.functional.silu(y)
    if residual is not None:
        y = y + residual.float()
    return y


def _check(out, ref, k):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 0.02 * scale + 1e-3 * (k ** 0.5), f"max abs err {err} vs scale {scale}"


SHAPES = [
    # tokens, features, k
    (8, 4096, 4096),     # decode: weights fill the tensor-core rows, split-K
    (16, 512, 1376),     # ragged K (21.5 k-blocks)
    (1, 256, 64),        # single k-block
    (64, 1536, 4096),
    (128, 256, 512),     # one tile, normal orientation
    (300, 1000, 520),    # ragged everything
    (2048, 4096, 1024),  # 256-wide tiles
    (1024, 1376, 4096),  # ragged N
    (500, 136, 72),
]


@pytest.mark.parametrize("tokens,features,k", SHAPES)
def test_gemm_matches_reference(tokens, features, k):
    nat = _native()
    torch.manual_seed(0)
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    out = nat.gemm_nt(x, w)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    _check(out, _ref(x, w), k)


@pytest.mark.parametrize("tokens", [8, 512])
@pytest.mark.parametrize("act", [None, "relu", "gelu", "gelu_tanh", "silu"])
def test_gemm_epilogue(tokens, act):
    nat = _native()
    torch.manual_seed(1)
    features, k = 768, 512
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(features, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(tokens, features, device="cuda", dtype=torch.bfloat16)
    out = nat.gemm_nt(x, w, bias=bias, residual=res, act=act)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    _check(out, _ref(x, w, bias, res, act), k)


@pytest.mark.parametrize("splits", [1, 2, 5])
def test_gemm_forced_split_k(splits):
    nat = _native()
    torch.manual_seed(2)
    tokens, features, k = 8, 1024, 2048
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(features, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):  # repeated calls re-use the arrival counters (epochs only grow)
        out = nat.gemm_nt(x, w, bias=bias, force_splits=splits)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    _check(out, _ref(x, w, bias), k)


@pytest.mark.parametrize("tokens,features,k", [(8, 4096, 4096), (8, 1536, 4096), (16, 1000, 1376), (40, 4096, 11008), (3, 256, 64)])
def test_gemm_stream_k_decomposition(tokens, features, k):
    """Opt-in stream-K: every CTA owns one contiguous range of (tile, k-block) units; tiles shared by several CTAs are
    summed by the last contributor.  Bias / activation / residual and the gated epilogue go through the same path."""
    native = _native()
    torch.manual_seed(tokens + features)
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(features, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(tokens, features, device="cuda", dtype=torch.bfloat16)
    native.LIB.tpb_gemm_enable_stream_k(1)
    native._plan_cache.clear()
    try:
        plan = native.gemm_plan(tokens, features, k)
        for _ in range(3):  # the per-tile counters re-arm themselves
            out = native.gemm_nt(x, w, bias=bias, residual=res, act="gelu")
        torch.cuda.synchronize()
        native.device_state(x.device).check_status()
    finally:
        native.LIB.tpb_gemm_enable_stream_k(0)
        native._plan_cache.clear()
    assert plan.stream_k == 1 or features * k < 256 * 64 * 2
    _check(out, _ref(x, w, bias, res, "gelu"), k)


def test_gemm_strided_input_and_output_views():
    nat = _native()
    torch.manual_seed(3)
    big = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16)
    x = big[:, 256:768]  # row pitch 1024, 16-byte aligned start
    w = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16) * 0.05
    out = nat.gemm_nt(x, w)
    torch.cuda.synchronize()
    _check(out, _ref(x, w), 512)


def test_linear_autograd():
    nat = _native()
    torch.manual_seed(4)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = nat.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _check(y, yr.detach(), 256)
    _check(x.grad, xr.grad, 512)
    _check(w.grad, wr.grad, 384)
    _check(b.grad, br.grad, 384)


@pytest.mark.parametrize("tokens,splits", [(8, 0), (8, 3), (40, 0), (300, 0), (2048, 0)])
def test_gemm_fused_swiglu_epilogue(tokens, splits):
    nat = _native()
    torch.manual_seed(6)
    f, k = 1376, 1024
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(f, k, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(f, k, device="cuda", dtype=torch.bfloat16) * 0.05
    out = nat.gemm_nt(x, nat.interleave_gate_up(wg, wu), act="swiglu16", force_splits=splits)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    assert out.shape == (tokens, f)
    ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    _check(out, ref, k)


def test_gemm_k_not_multiple_of_8():
    nat = _native()
    torch.manual_seed(5)
    x = torch.randn(70, 150, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(96, 150, device="cuda", dtype=torch.bfloat16) * 0.05
    out = nat.gemm_nt(x, w)
    torch.cuda.synchronize()
    _check(out, _ref(x, w), 150)
    xt = nat.transpose(x)  # [150, 70] with a padded row pitch
    assert xt.stride(0) % 8 == 0 and torch.equal(xt, x.t())


def test_transpose():
    nat = _native()
    x = torch.randn(300, 136, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(nat.transpose(x), x.t().contiguous())


@pytest.mark.parametrize("tokens,features,k", [(128, 256, 512), (300, 1000, 520), (2048, 4096, 1024), (8, 192, 136), (1000, 136, 72), (520, 1376, 264)])
@pytest.mark.parametrize("x_t,w_t", [(False, True), (True, True), (True, False)])
def test_gemm_operands_transposed_in_memory(tokens, features, k, x_t, w_t):
    """MN-major tensor-core operands: x handed over as [k, tokens] and / or w as [k, features], read in place."""
    nat = _native()
    torch.manual_seed(5)
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(features, device="cuda", dtype=torch.bfloat16)
    out = nat.gemm_nt(x.t().contiguous() if x_t else x, w.t().contiguous() if w_t else w, bias=bias, x_t=x_t, w_t=w_t)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    _check(out, _ref(x, w, bias), k)


def test_linear_backward_reads_operands_in_place():
    """dX and dW of the autograd linear against fp32 autograd; no transpose kernel is launched."""
    nat = _native()
    torch.manual_seed(6)
    x = torch.randn(3, 100, 264, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(520, 264, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    b = torch.randn(520, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(3, 100, 520, device="cuda", dtype=torch.bfloat16)
    before = nat.launch_count
    nat.linear(x, w, b).backward(g)
    torch.cuda.synchronize()
    assert nat.launch_count - before == 3  # forward, dgrad, wgrad
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    torch.nn.functional.linear(xr, wr, br).backward(g.float())
    for got, want in ((x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= 0.02 * want.abs().max().item() + 0.05, err


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("tokens,features,k,act", [(8, 1536, 4096, None), (8, 2752, 4096, "swiglu16"), (3, 256, 512, "gelu"), (40, 1000, 1024, None)])
def test_gemm_with_folded_norm(mode, tokens, features, k, act):
    """RMSNorm / LayerNorm of the token rows folded into the GEMM: statistics in the epilogue warps, norm weight
    multiplied into the GEMM weight beforehand.  Reference: fp32 norm followed by an fp32 matmul."""
    nat = _native()
    torch.manual_seed(7)
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16) * 2 + (0.5 if mode == 2 else 0.0)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    gamma = 1 + 0.1 * torch.randn(k, device="cuda")
    beta = 0.1 * torch.randn(k, device="cuda") if mode == 2 else None
    bias = torch.randn(features, device="cuda", dtype=torch.bfloat16)
    xf = x.float()
    if mode == 1:
        normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma
    else:
        normed = torch.nn.functional.layer_norm(xf, (k,), gamma, beta, 1e-5)
    ref = normed @ w.float().t() + bias.float()
    w_folded = (w.float() * gamma).to(torch.bfloat16)
    rowsum = w_folded.float().sum(1) if mode == 2 else None
    fused_bias = (bias.float() + (w.float() @ beta if beta is not None else 0)).to(torch.bfloat16)
    if act == "swiglu16":
        ref = torch.nn.functional.silu(ref[:, : features // 2]) * ref[:, features // 2 :]
        half = features // 2
        w_folded = nat.interleave_gate_up(w_folded[:half].contiguous(), w_folded[half:].contiguous())
        fused_bias = torch.stack((fused_bias[:half].reshape(-1, 16), fused_bias[half:].reshape(-1, 16)), dim=1).reshape(-1).contiguous()
        if rowsum is not None:
            rowsum = w_folded.float().sum(1)
    elif act == "gelu":
        ref = torch.nn.functional.gelu(ref)
    for _ in range(2):
        out = nat.gemm_nt(x, w_folded, bias=fused_bias, act=act, norm=(mode, 1e-5, rowsum))
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    err = (out.float() - ref).abs().max().item()
    assert err <= 0.03 * ref.abs().max().item() + 0.05, err


@pytest.mark.parametrize("tokens,features,k", [(8, 1536, 4096), (8, 2752, 4096), (8, 4000, 4096), (16, 768, 8192)])
def test_gemm_splits_k_when_few_tiles_stream_much(tokens, features, k):
    """Shard-sized decode GEMMs (few 128-row tiles, a long K) are split over K automatically."""
    nat = _native()
    torch.manual_seed(8)
    plan = nat.gemm_plan(tokens, features, k)
    assert plan.swapped and plan.k_splits > 1 and plan.grid <= 148
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(tokens, features, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        out = nat.gemm_nt(x, w, residual=res)
    torch.cuda.synchronize()
    nat.device_state(x.device).check_status()
    _check(out, _ref(x, w, None, res), k)
