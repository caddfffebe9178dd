"""Memory-bound kernels (norms, rotary embedding, activations, embedding, AdamW) against fp32
PyTorch references of the same operations."""
import pytest
import torch
import torch.nn.functional as F

from tensor_parallel_b200.ops import functional as OF

pytestmark = pytest.mark.gpu


def _native():
    from tensor_parallel_b200.ops import native

    return native


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [64, 4096, 5120, 8192])
@pytest.mark.parametrize("mode", ["rms", "layer"])
def test_norm_forward_backward(dtype, cols, mode):
    nat = _native()
    torch.manual_seed(0)
    x = torch.randn(37, cols, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda", dtype=dtype)).requires_grad_(True)
    b = (0.1 * torch.randn(cols, device="cuda", dtype=dtype)).requires_grad_(True)
    g = torch.randn(37, cols, device="cuda", dtype=dtype)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    if mode == "rms":
        y = nat.rms_norm(x, w, 1e-6)
        yr = OF.rms_norm_ref(xr, wr, 1e-6)
    else:
        y = nat.layer_norm(x, w, b, 1e-5)
        yr = F.layer_norm(xr, (cols,), wr, br, 1e-5)
    y.backward(g)
    yr.backward(g.float())
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(y.float(), yr, **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)
    wtol = dict(atol=0.25, rtol=5e-2) if dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(w.grad.float(), wr.grad, **wtol)
    if mode == "layer":
        torch.testing.assert_close(b.grad.float(), br.grad, **wtol)


def test_norm_fused_residual():
    nat = _native()
    torch.manual_seed(1)
    x = torch.randn(16, 4096, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(16, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    summed = torch.empty_like(x)
    out, _, _ = nat.norm_forward(x, w, None, 1e-6, 0, residual=r, sum_out=summed)
    h = (x.float() + r.float()).to(torch.bfloat16)
    torch.testing.assert_close(summed, h)
    torch.testing.assert_close(out.float(), OF.rms_norm_ref(h.float(), w.float(), 1e-6), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("rotary_dim", [None, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope(interleaved, rotary_dim, dtype):
    nat = _native()
    torch.manual_seed(2)
    x = torch.randn(2, 19, 4, 64, device="cuda", dtype=dtype, requires_grad=True)
    pos = torch.arange(5, 24, device="cuda")[None].expand(2, 19)
    y = nat.rope(x, pos, 10000.0, rotary_dim, interleaved)
    xr = x.detach().float().requires_grad_(True)
    yr = OF.apply_rope_ref(xr, pos, 10000.0, rotary_dim, interleaved)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    tol = dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(y.float(), yr, **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)


@pytest.mark.parametrize("name", ["relu", "gelu", "gelu_tanh", "swiglu", "geglu"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_activations(name, dtype):
    nat = _native()
    torch.manual_seed(3)
    a = torch.randn(33, 1376, device="cuda", dtype=dtype, requires_grad=True)
    b = torch.randn(33, 1376, device="cuda", dtype=dtype, requires_grad=True)
    ar, br = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    if name == "relu":
        y, yr = nat.relu(a), torch.relu(ar)
    elif name == "gelu":
        y, yr = nat.gelu(a), F.gelu(ar)
    elif name == "gelu_tanh":
        y, yr = nat.gelu(a, "tanh"), F.gelu(ar, approximate="tanh")
    elif name == "swiglu":
        y, yr = nat.swiglu(a, b), F.silu(ar) * br
    else:
        y, yr = nat.geglu(a, b), F.gelu(ar, approximate="tanh") * br
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(y.float(), yr, **tol)
    torch.testing.assert_close(a.grad.float(), ar.grad, **tol)
    if name in ("swiglu", "geglu"):
        torch.testing.assert_close(b.grad.float(), br.grad, **tol)


def test_embedding_gather():
    nat = _native()
    table = torch.randn(1000, 512, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (4, 33), device="cuda")
    assert torch.equal(nat.embedding(ids, table), table[ids])


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
def test_fused_adamw_matches_torch(pdtype):
    nat = _native()
    torch.manual_seed(4)
    n = 10_000
    p0 = torch.randn(n, device="cuda")
    ref = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p = p0.to(pdtype)
    master = p0.clone() if pdtype == torch.bfloat16 else None
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = g.clone()
        opt.step()
        nat.adamw_step(p, g, m, v, step, 1e-2, 0.9, 0.95, 1e-8, 0.1, master=master)
    target = master if master is not None else p
    torch.testing.assert_close(target, ref.detach(), atol=1e-5, rtol=1e-5)
    if pdtype == torch.bfloat16:
        torch.testing.assert_close(p.float(), ref.detach(), atol=2e-2, rtol=2e-2)
