"""Small single-kernel workloads for timing and for Nsight Compute captures.

    python -m tensor_parallel_b200.profiling <case> [--iters N]

Each case allocates a few hundred MB at most (inputs larger than the 126 MB L2 where the kernel is
memory-bound), warms up, then launches the kernel ``--iters`` times with a fresh operand each time (a
ring of buffers defeats L2 reuse) and prints the median CUDA-event time with the achieved bandwidth or
FLOP rate.  Under ``ncu -k regex:<kernel> -c 3`` the same command captures those launches.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from tensor_parallel_b200.ops import native


def _time(fn, iters: int):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i + 3)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(times)


GRAPH = False  # --graph: also time 16 launches replayed from one CUDA graph (device time without host launch gaps)


def _graph_time(fn, launches: int = 16, reps: int = 5):
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                fn(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (launches * reps)


def _timed(fn, iters: int) -> dict:
    out = {"us": _time(fn, iters)}
    if GRAPH:
        out["graph_us"] = _graph_time(fn)
    return out


def case_attn_decode_fused(batch, heads, kv_heads, ctx, iters, splits=1):
    """The serving engine's decode attention: RoPE + cache append + split-KV attention + merge in one launch."""
    d, smax, ring = 128, ctx + 64, 3
    ks = [torch.randn(batch, kv_heads, smax, d, device="cuda", dtype=torch.bfloat16) for _ in range(ring)]
    vs = [torch.randn(batch, kv_heads, smax, d, device="cuda", dtype=torch.bfloat16) for _ in range(ring)]
    qkv = torch.randn(batch, (heads + 2 * kv_heads) * d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, : heads * d], qkv[:, heads * d : (heads + kv_heads) * d], qkv[:, (heads + kv_heads) * d :]
    pos = torch.tensor([ctx], device="cuda", dtype=torch.int32)
    out = torch.empty(batch, heads, d, device="cuda", dtype=torch.bfloat16)
    ws = (torch.empty(batch * heads * splits * d, device="cuda"), torch.empty(batch * heads * splits * 2, device="cuda"),
          torch.zeros(batch * kv_heads, dtype=torch.int32, device="cuda"))
    res = _timed(lambda i: native.attn_decode_fused(q, k, v, ks[i % ring], vs[i % ring], pos, d, 10000.0, splits=splits,
                                                    workspace=ws, out=out), iters)
    best = res.get("graph_us", res["us"])
    return {**res, "tbps": 2.0 * batch * kv_heads * ctx * d * 2 / best / 1e6}


def case_gemm(tokens, features, k, iters, ring=None):
    ring = ring or max(2, int(300e6 // (features * k * 2)) + 1)
    ws = [torch.randn(features, k, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(ring)]
    x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(tokens, features, device="cuda", dtype=torch.bfloat16)
    res = _timed(lambda i: native.gemm_nt(x, ws[i % ring], out=out), iters)
    us = res.get("graph_us", res["us"])
    flops = 2.0 * tokens * features * k
    bytes_ = 2.0 * (features * k + tokens * k + tokens * features)
    return {**res, "tflops": flops / us / 1e6, "tbps": bytes_ / us / 1e6, "plan": {f: getattr(native.gemm_plan(tokens, features, k), f) for f in ("swapped", "bn", "kbox", "k_splits", "grid")}}


def case_attn_decode(batch, heads, kv_heads, ctx, iters, splits=1):
    d, smax, ring = 128, ctx + 64, 3
    ks = [torch.randn(batch, kv_heads, smax, d, device="cuda", dtype=torch.bfloat16) for _ in range(ring)]
    vs = [torch.randn(batch, kv_heads, smax, d, device="cuda", dtype=torch.bfloat16) for _ in range(ring)]
    q = torch.randn(batch, heads, d, device="cuda", dtype=torch.bfloat16)
    length = torch.tensor([ctx], device="cuda", dtype=torch.int32)
    ws = (torch.empty(batch * heads * splits * d, device="cuda"), torch.empty(batch * heads * splits * 2, device="cuda"))
    us = _time(lambda i: native.attn_decode(q, ks[i % ring], vs[i % ring], length, 0, splits=splits, workspace=ws), iters)
    return {"us": us, "tbps": 2.0 * batch * kv_heads * ctx * d * 2 / us / 1e6}


def case_attn_prefill(batch, seq, heads, d, iters):
    q, k, v = (torch.randn(batch, seq, heads, d, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    us = _time(lambda i: native.attention_forward(q, k, v, True, None), iters)
    return {"us": us, "tflops": 4.0 * batch * heads * seq * seq * d / 2 / us / 1e6}


def case_attn_backward(batch, seq, heads, d, iters):
    q, k, v, g = (torch.randn(batch, seq, heads, d, device="cuda", dtype=torch.bfloat16) for _ in range(4))
    out, lse = native.attention_forward(q, k, v, True, None, want_lse=True)
    us = _time(lambda i: native.attention_backward(q, k, v, out, g, lse, True, None), iters)
    return {"us": us, "tflops": 2.5 * 4.0 * batch * heads * seq * seq * d / 2 / us / 1e6, "note": "useful FLOPs = 2.5 x forward"}


def case_cross_entropy(rows, vocab, hidden, iters):
    from tensor_parallel_b200.ops.loss import lm_head_cross_entropy

    h = (torch.randn(rows, hidden, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(vocab, hidden, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, vocab, (rows,), device="cuda")

    def step(i):
        loss = lm_head_cross_entropy(h[None], w, labels[None])
        loss.backward()
        h.grad = w.grad = None

    us = _time(step, iters)
    return {"us": us, "tflops": 6.0 * rows * vocab * hidden / us / 1e6}


def case_norm(rows, cols, iters):
    xs = [torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    w = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(xs[0])
    us = _time(lambda i: native.norm_forward(xs[i % 3], w, None, 1e-6, 0, out=out), iters)
    return {"us": us, "tbps": 2.0 * rows * cols * 2 / us / 1e6}


def case_swiglu(rows, cols, iters):
    gus = [torch.randn(rows, 2 * cols, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    out = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: native.act_forward(gus[i % 3][:, :cols], gus[i % 3][:, cols:], 4, out=out), iters)
    return {"us": us, "tbps": 3.0 * rows * cols * 2 / us / 1e6}


def case_rope_append(batch, seq, heads, iters):
    d = 128
    qkv = torch.randn(batch * seq, 3 * heads * d, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(batch, heads, seq, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(batch * seq, heads, d, device="cuda", dtype=torch.bfloat16)
    pos = torch.zeros(1, device="cuda", dtype=torch.int32)
    w = heads * d
    us = _time(lambda i: native.qkv_rope_append(qkv[:, :w], qkv[:, w : 2 * w], qkv[:, 2 * w :], q_out, kc, vc, pos, batch, seq, d, 1e4), iters)
    return {"us": us, "tbps": 2.0 * qkv.numel() * 2 / us / 1e6}


def case_adamw(n, iters):
    p = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), p.float()
    us = _time(lambda i: native.adamw_step(p, g, m, v, i + 1, 1e-4, 0.9, 0.95, 1e-8, 0.1, master=master), iters)
    return {"us": us, "tbps": n * (2 + 2 + 3 * 4 + 2 + 3 * 4) / us / 1e6}


CASES = {
    "gemm_decode_qkv": lambda it: case_gemm(8, 12288, 4096, it),
    "gemm_decode_gate_up": lambda it: case_gemm(8, 22016, 4096, it),
    "gemm_decode_down": lambda it: case_gemm(8, 4096, 11008, it),
    "gemm_decode_o_tp8": lambda it: case_gemm(8, 4096, 512, it),
    "gemm_prefill": lambda it: case_gemm(8192, 8192, 4096, it, ring=2),
    "gemm_prefill_gate_up": lambda it: case_gemm(4096, 22016, 4096, it, ring=2),
    "attn_decode": lambda it: case_attn_decode(8, 32, 32, 2048, it),
    "attn_decode_tp8": lambda it: case_attn_decode(8, 4, 4, 2048, it, splits=8),
    "attn_decode_fused": lambda it: case_attn_decode_fused(8, 32, 32, 2048, it),
    "attn_decode_fused_tp8": lambda it: case_attn_decode_fused(8, 4, 4, 2048, it, splits=8),
    "attn_prefill": lambda it: case_attn_prefill(4, 2048, 32, 128, it),
    "attn_backward": lambda it: case_attn_backward(4, 2048, 32, 128, it),
    "head_cross_entropy": lambda it: case_cross_entropy(8192, 32000, 4096, it),
    "rmsnorm": lambda it: case_norm(32768, 4096, it),
    "swiglu": lambda it: case_swiglu(16384, 11008, it),
    "rope_append": lambda it: case_rope_append(8, 2048, 32, it),
    "adamw": lambda it: case_adamw(64 * 1024 * 1024, it),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--graph", action="store_true", help="also report the per-launch time of a replayed CUDA graph")
    args = ap.parse_args()
    global GRAPH
    GRAPH = args.graph
    for name in (sorted(CASES) if args.case == "all" else [args.case]):
        result = CASES[name](args.iters)
        torch.cuda.synchronize()
        native.device_state(torch.device("cuda", torch.cuda.current_device())).check_status()
        print(json.dumps({"case": name, **result}), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
