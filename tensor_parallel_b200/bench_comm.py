"""Micro-benchmarks of the device-side communication paths (launch under torchrun, one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m tensor_parallel_b200.bench_comm

For every case the kernel is launched ``iters`` times back to back between two CUDA events (weights rotate through
a ring so they are not L2-resident); the reported time is the max over ranks.  The decode-sized cases are also
replayed from one CUDA graph (``graph_us``: device time without host launch gaps, which is how the serving engine
runs them).  Fused paths are compared with their un-fused composition and with the roofline
``max(FLOPs / measured GEMM peak, NVLink bytes / link bandwidth)``; the stand-alone all-reduce with its variants
(peer loads / stores, NVSwitch multimem) and with NCCL.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from tensor_parallel_b200.ops import comm as C
from tensor_parallel_b200.ops import native

GEMM_PEAK_TFLOPS, LINK_GBS, HBM_GBS = 1608.0, 770.0, 6537.0


def timed(fn, iters=20, warm=3):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i + warm)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def graph_timed(fn, iters=32, replays=5):
    """Device time per launch when ``iters`` launches are replayed from one CUDA graph (max over ranks)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(4):
            fn(i)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (iters * replays)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    rc = C.make_process_comm(dev, staging_bytes=288 << 20)
    out = []

    def report(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)
        out.append(kw)

    # stand-alone all-reduce: device kernel vs NCCL
    for nbytes in (8 << 10, 64 << 10, 256 << 10, 1 << 20, 16 << 20, 128 << 20):
        n = nbytes // 2
        x = torch.randn(n, device=dev, dtype=torch.bfloat16)
        src = rc.staging_view("in", (n,), torch.bfloat16)
        src.copy_(x)
        t_dev = timed(lambda i: rc.all_reduce(src))
        t_one = timed(lambda i: rc.all_reduce(src, force_algo=0)) if nbytes <= (1 << 20) else None
        t_peer = timed(lambda i: rc.all_reduce(src, force_algo=1))
        t_nvls = timed(lambda i: rc.all_reduce(src, force_algo=4)) if rc.mc_base else None
        y = x.clone()
        t_nccl = timed(lambda i: dist.all_reduce(y))
        # below 1 MiB the eager numbers above are bound by the host (one Python call per collective on either side):
        # the same launches replayed from a CUDA graph show the device time
        g_dev = g_bar = g_nccl = None
        if nbytes <= (1 << 20):
            g_dev = graph_timed(lambda i: rc.all_reduce(src))
            g_bar = graph_timed(lambda i: rc.all_reduce(src, force_algo=0))
            try:
                g_nccl = graph_timed(lambda i: dist.all_reduce(y))
            except Exception:  # noqa: BLE001 - a NCCL build that cannot be captured: leave the column empty
                g_nccl = None
        bus = 2 * (world - 1) / world * nbytes
        report(case="all_reduce", bytes=nbytes, world=world, graph_device_us=g_dev, graph_barrier_one_shot_us=g_bar, graph_nccl_us=g_nccl, device_us=t_dev, barrier_one_shot_us=t_one, peer_two_shot_us=t_peer, nvls_two_shot_us=t_nvls,
               nccl_us=t_nccl, device_busbw_gbs=bus / t_dev / 1e3, nccl_busbw_gbs=bus / t_nccl / 1e3,
               link_roofline_us=nbytes / (LINK_GBS * 1e3))

    # row-parallel GEMM + all-reduce, decode shapes (per-rank K = full K / world)
    for name, feats, k_full in (("o_proj", 4096, 4096), ("down_proj", 4096, 11008)):
        k = (k_full // world + 7) // 8 * 8
        ring = 8
        ws = [torch.randn(feats, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(ring)]
        x = torch.randn(8, k, device=dev, dtype=torch.bfloat16)
        res = torch.zeros(8, feats, device=dev, dtype=torch.bfloat16)
        o = torch.empty(8, feats, device=dev, dtype=torch.bfloat16)
        t_local = timed(lambda i: native.gemm_nt(x, ws[i % ring], out=o))
        t_fused = timed(lambda i: rc.gemm_allreduce(x, ws[i % ring], residual=res, out=o))
        g_local = graph_timed(lambda i: native.gemm_nt(x, ws[i % ring], out=o))
        by_protocol = {}
        for label, flag in (("flagged_words", -1), ("arrival_counters", 1)):
            native.LIB.tpb_gemm_disable_flagged_exchange(flag)
            by_protocol[label] = graph_timed(lambda i: rc.gemm_allreduce(x, ws[i % ring], residual=res, out=o))
        native.LIB.tpb_gemm_disable_flagged_exchange(0)
        g_fused = graph_timed(lambda i: rc.gemm_allreduce(x, ws[i % ring], residual=res, out=o))
        stage = rc.staging_view("in", (8, feats), torch.bfloat16)

        def unfused(i):
            native.gemm_nt(x, ws[i % ring], out=stage)
            rc.all_reduce(stage)

        t_unfused = timed(unfused)
        y = torch.empty(8, feats, device=dev, dtype=torch.bfloat16)

        def nccl_path(i):
            native.gemm_nt(x, ws[i % ring], out=y)
            dist.all_reduce(y)

        t_nccl = timed(nccl_path)
        roof = max(2 * 8 * feats * k / (GEMM_PEAK_TFLOPS * 1e6), feats * k * 2 / (HBM_GBS * 1e3), 8 * feats * 4 * (world - 1) / (LINK_GBS * 1e3))
        report(case="gemm_allreduce_decode", layer=name, world=world, tokens=8, features=feats, k_local=k, local_gemm_us=t_local,
               fused_us=t_fused, gemm_then_device_allreduce_us=t_unfused, gemm_then_nccl_us=t_nccl, roofline_us=roof,
               graph_local_gemm_us=g_local, graph_fused_us=g_fused, graph_fused_by_protocol_us=by_protocol,
               fraction_of_roofline=roof / g_fused)

    # all-gather + column-parallel GEMM (prefill shape): fused vs device all-gather + GEMM
    tokens, hidden, feats = 4096, 4096, 4096
    cols = hidden // world
    xl = torch.randn(tokens, cols, device=dev, dtype=torch.bfloat16)
    w = torch.randn(feats, hidden, device=dev, dtype=torch.bfloat16) * 0.02
    o = torch.empty(tokens, feats, device=dev, dtype=torch.bfloat16)
    t_fused = timed(lambda i: rc.allgather_gemm(xl, w, out=o), iters=10)

    def ag_then_gemm(i):
        g = rc.all_gather(xl)
        full = g.permute(1, 0, 2).reshape(tokens, hidden)
        native.gemm_nt(full, w, out=o)

    t_unfused = timed(ag_then_gemm, iters=10)
    full = torch.randn(tokens, hidden, device=dev, dtype=torch.bfloat16)
    t_gemm = timed(lambda i: native.gemm_nt(full, w, out=o), iters=10)
    roof = max(2 * tokens * feats * hidden / (GEMM_PEAK_TFLOPS * 1e6), tokens * cols * 2 * (world - 1) / (LINK_GBS * 1e3))
    report(case="allgather_gemm", world=world, tokens=tokens, hidden=hidden, features=feats, fused_us=t_fused,
           allgather_then_gemm_us=t_unfused, gemm_only_us=t_gemm, roofline_us=roof, fraction_of_roofline=roof / t_fused)
    torch.cuda.synchronize()
    rc.check_status()
    dist.barrier()
    C.close_all_heaps()  # (every rank unmaps its multicast view before anyone exits)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
