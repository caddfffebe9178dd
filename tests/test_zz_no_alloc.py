"""Allocation-free decode attention (``tpb_attn_decode_noalloc``) against the regular entry point.

Some users of the native library cannot allocate device memory themselves - a server that gave the
whole GPU to its KV cache, an embedding host that owns every buffer - so this variant keeps its split-KV
workspace in a static device array inside the library.  The test calls it through its exported C
symbol, twice in a row with different shapes (the second call sees the first call's leftovers in the
shared workspace), and compares with ``tpb_attn_decode`` run on a workspace allocated by the test and with a plain
fp32 PyTorch attention over the same keys.  The amount of free device memory must not move across the calls.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 2 * 1024 * 1024


def _symbol():
    from tensor_parallel_b200.ops import native

    fn = native.LIB.tpb_attn_decode_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ctypes.c_float, vp]
    fn.restype = ci
    return native, fn


def _case(seed, b, hq, hkv, d, ctx, smax):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(b, hq, d, device="cuda", dtype=torch.bfloat16, generator=gen)
    kc = torch.randn(b, hkv, smax, d, device="cuda", dtype=torch.bfloat16, generator=gen)
    vc = torch.randn(b, hkv, smax, d, device="cuda", dtype=torch.bfloat16, generator=gen)
    length = torch.tensor([ctx], device="cuda", dtype=torch.int32)
    return q, kc, vc, length


def _run_noalloc(fn, q, kc, vc, length, splits):
    b, hq, d = q.shape
    out = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    code = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), length.data_ptr(), 0, b, hq, kc.shape[1], d,
              kc.shape[2], splits, 1.0 / d ** 0.5, stream)
    return code, out


def test_noalloc_decode_matches_regular_entry_point_twice():
    native, fn = _symbol()
    cases = [
        (_case(1, 4, 16, 4, 128, 300, 512), 8),   # GQA, 8 splits
        (_case(2, 2, 8, 8, 64, 77, 128), 3),      # different shape and split count: reuses the same workspace
    ]
    # one call up front: the first call per device resolves the workspace address and sets kernel attributes
    (q, kc, vc, length), splits = cases[0]
    assert _run_noalloc(fn, q, kc, vc, length, splits)[0] == 0
    torch.cuda.synchronize()
    for (q, kc, vc, length), splits in cases:
        want = native.attn_decode(q, kc, vc, length, 0, splits=splits)  # regular entry point, workspace from torch
        ctx = int(length.item())
        b, hq, d = q.shape
        rep = hq // kc.shape[1]
        keys = kc[:, :, :ctx].float().repeat_interleave(rep, dim=1)
        vals = vc[:, :, :ctx].float().repeat_interleave(rep, dim=1)
        probs = torch.softmax(torch.einsum("bhd,bhsd->bhs", q.float(), keys) / d ** 0.5, dim=-1)
        want32 = torch.einsum("bhs,bhsd->bhd", probs, vals)  # fp32 reference of the same operation
        out = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        stream = torch.cuda.current_stream().cuda_stream
        code = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), length.data_ptr(), 0, b, hq, kc.shape[1], d,
                  kc.shape[2], splits, 1.0 / d ** 0.5, stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the amount of free device memory"
        got = out
        assert code == 0
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got.float(), want32, atol=2e-2, rtol=2e-2)


def test_noalloc_rejects_sizes_beyond_its_workspace():
    _, fn = _symbol()
    b, hq, d, splits = 64, 64, 128, 16
    assert b * hq * splits * (d + 2) > SCRATCH_FLOATS
    q, kc, vc, length = _case(3, 1, 1, 1, d, 8, 16)  # pointers only need to be valid: nothing may be launched
    out = torch.zeros(1, 1, d, device="cuda", dtype=torch.bfloat16)
    code = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), length.data_ptr(), 0, b, hq, 1, d, 16, splits,
              1.0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == 7  # TPB_ERR_SIZE
    assert out.abs().sum().item() == 0
