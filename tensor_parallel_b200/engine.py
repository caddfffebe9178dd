"""Serving engine for Llama-shaped tensor-parallel shards: kernel-level prefill and a decode step
captured once as a CUDA graph and replayed per token.

The engine is what ``generate()`` of a tensor-parallel Llama model runs on CUDA.  It reads the
shard's own parameters (q/k/v are re-pointed at one fused buffer; gate/up are copied once into an
interleaved layout that lets the GEMM epilogue apply SwiGLU), keeps a pre-allocated head-sharded KV cache ``[batch, local_kv_heads, max_seq, head_dim]``
per layer, and per layer launches::

    rmsnorm -> qkv GEMM -> [rope + cache append + attention + split merge] -> o_proj GEMM (+ all-reduce + residual)
            -> rmsnorm -> gate/up GEMM (+ SwiGLU epilogue) -> down GEMM (+ all-reduce + residual)

(seven kernels per layer in a decode step; prefill keeps rope/append and attention as separate launches)

With several ranks the two row-parallel GEMMs push their partial tiles to every peer from the
epilogue and reduce them in the same kernel (decode), or write into symmetric memory and run the
two-shot device all-reduce (prefill); nothing goes through NCCL.  The reference reaches the same
maths through Python wrappers, host barriers and one NCCL call per collective
(``src/tensor_parallel/tensor_parallel.py:139-161``, ``src/tensor_parallel/communications.py:34-52``).
"""
from __future__ import annotations

import math
import os
from typing import List, Optional

import torch

from tensor_parallel_b200.ops import native
from tensor_parallel_b200.utils.tracing import traced


def _unwrap(module):
    return module.__dict__.get("tp_wrapped_module", module) if hasattr(module, "__dict__") else module


class LlamaEngine:
    def __init__(self, shard, comm=None, max_batch: int = 8, max_seq: int = 2560, use_graph: bool = True, embed_table=None):
        lm = _unwrap(shard)
        cfg = lm.config
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.cfg = cfg
        self.eps = cfg.rms_norm_eps
        self.theta = float(cfg.rope_theta)
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        self.hidden = cfg.hidden_size
        self.max_batch, self.max_seq = max_batch, max_seq
        self.use_graph = use_graph and not os.environ.get("TPB_NO_GRAPH")
        model = _unwrap(lm.model)
        embed = _unwrap(model.embed_tokens)
        self.device = embed.weight.device
        dev = self.device

        # full embedding table (hidden-split shards are gathered once; 2 * vocab * hidden bytes per rank)
        table = embed.weight.detach() if embed_table is None else embed_table
        if table.shape[1] != self.hidden:
            import torch.distributed as dist

            parts = [torch.empty_like(table) for _ in range(self.world)]
            dist.all_gather(parts, table.contiguous())
            table = torch.cat(parts, dim=1)
        self.embed = table.contiguous()

        self.layers = []
        for layer in model.layers:
            attn, mlp = _unwrap(layer.self_attn), _unwrap(layer.mlp)
            wq, wk, wv = attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight
            wqkv = torch.cat([wq.detach(), wk.detach(), wv.detach()], dim=0).contiguous()
            nq, nk = wq.shape[0], wk.shape[0]
            wq.data, wk.data, wv.data = wqkv[:nq], wqkv[nq : nq + nk], wqkv[nq + nk :]
            wg, wu, wd = mlp.gate_proj.weight.detach(), mlp.up_proj.weight.detach(), mlp.down_proj.weight.detach()
            ff = wg.shape[0]
            if ff % 16:  # zero rows (and the matching zero columns of down_proj) fill the last group of 16: they contribute silu(0) * 0 = 0
                pad = 16 - ff % 16
                wg, wu = (torch.cat([w, w.new_zeros(pad, w.shape[1])], dim=0) for w in (wg, wu))
                wd = torch.cat([wd, wd.new_zeros(wd.shape[0], pad)], dim=1).contiguous()
                ff += pad
            # engine-owned copy, rows interleaved [16 gate | 16 up] so that the GEMM epilogue applies SwiGLU itself
            wgu = native.interleave_gate_up(wg, wu)
            self.layers.append(dict(
                wqkv=wqkv, wo=attn.o_proj.weight.detach(), wgu=wgu, wd=wd,
                ln1=layer.input_layernorm.weight.detach(), ln2=layer.post_attention_layernorm.weight.detach(),
                nq=nq // self.head_dim, nkv=nk // self.head_dim, ff=ff,
            ))
        self.final_norm = _unwrap(model.norm).weight.detach()
        self.lm_head = _unwrap(lm.lm_head).weight.detach()
        self.vocab_local = self.lm_head.shape[0]
        self.nq, self.nkv, self.ff = self.layers[0]["nq"], self.layers[0]["nkv"], self.layers[0]["ff"]

        B, D = max_batch, self.head_dim
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.kcache = [torch.zeros(B, self.nkv, max_seq, D, **bf) for _ in self.layers]
        self.vcache = [torch.zeros(B, self.nkv, max_seq, D, **bf) for _ in self.layers]
        # static decode buffers
        self.ids = torch.zeros(B, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.x = torch.zeros(B, self.hidden, **bf)
        self.n = torch.zeros(B, self.hidden, **bf)
        self.qkv = torch.zeros(B, (self.nq + 2 * self.nkv) * D, **bf)
        self.q_rot = torch.zeros(B, self.nq, D, **bf)
        self.attn = torch.zeros(B, self.nq * D, **bf)
        self.gu = None  # the gate|up product never reaches memory (SwiGLU is applied in the GEMM epilogue)
        self.act = torch.zeros(B, self.ff, **bf)
        self.logits_local = torch.zeros(B, self.vocab_local, **bf)
        self.next_ids = torch.zeros(B, dtype=torch.int64, device=dev)
        # split the key range only when (batch x kv heads) alone cannot occupy the SMs
        self.rope_angles = native.rope_table(max_seq, D, self.theta, dev)  # (cos, sin) of every position, looked up by the decode kernel
        self.splits = 1 if B * self.nkv >= 128 else max(1, min(8, math.ceil(256 / (B * self.nkv))))
        self.attn_ws = (torch.empty(B * self.nq * self.splits * D, dtype=torch.float32, device=dev),
                        torch.empty(B * self.nq * self.splits * 2, dtype=torch.float32, device=dev),
                        torch.zeros(B * self.nkv, dtype=torch.int32, device=dev))
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_batch = 0
        self.kernels_per_step = 0

    @torch.no_grad()
    def preload(self, batch: int = 1):
        """Runs the prefill and decode paths once on this rank ALONE (no peer involved; the results are meaningless
        for a shard) so that every kernel they launch - ours and PyTorch's - is loaded on this device.  A single host
        thread that drives several GPUs calls this first: with lazy module loading the first launch of a kernel may
        synchronise the device, which must not happen behind a kernel that waits for a peer not launched yet."""
        comm, world = self.comm, self.world
        self.comm, self.world = None, 1
        try:
            for seq in (8, 72):  # few-token and many-token GEMM orientations
                self.prefill(torch.zeros(batch, min(seq, self.max_seq - 2), dtype=torch.int64, device=self.device))
            for _ in range(2):
                self._decode_body(batch)
            # the PyTorch kernels that only the multi-rank path uses (strided copies, in-place add)
            t = self.x[:batch]
            t.add_(t)
            g = self.logits_local[:batch, : max(8, self.vocab_local // 2)].contiguous()
            torch.stack([g, g]).permute(1, 0, 2).reshape(batch, -1).float().argmax(-1)
            self.pos.zero_()
            self.ids.zero_()
            torch.cuda.synchronize(self.device)
        finally:
            self.comm, self.world = comm, world
        if comm is not None:
            native.check(native.LIB.tpb_comm_preload(), "tpb_comm_preload")

    # -- building blocks --------------------------------------------------------------------------

    def _row_parallel(self, x2d, weight, residual_out):
        """``residual_out += all-reduce(x2d @ weight.T)`` (in place)."""
        tokens = x2d.shape[0]
        if self.world == 1:
            native.gemm_nt(x2d, weight, residual=residual_out, out=residual_out)
        elif self.comm.fits_fused(tokens, weight.shape[0], weight.shape[1]) and tokens <= 64:
            self.comm.gemm_allreduce(x2d, weight, residual=residual_out, out=residual_out)
        else:
            staged = self.comm.staging_view("in", (tokens, weight.shape[0]), torch.bfloat16)
            native.gemm_nt(x2d, weight, out=staged)
            reduced = self.comm.all_reduce(staged)
            residual_out.add_(reduced)

    def _layer(self, i, x, n, qkv, q_rot, attn, gu, act, batch, seq, decode: bool):
        L = self.layers[i]
        D = self.head_dim
        native.norm_forward(x, L["ln1"], None, self.eps, 0, out=n)
        native.gemm_nt(n, L["wqkv"], out=qkv)
        nq_w, nk_w = self.nq * D, self.nkv * D
        q2, k2, v2 = qkv[:, :nq_w], qkv[:, nq_w : nq_w + nk_w], qkv[:, nq_w + nk_w :]
        if decode:
            # RoPE, cache append, split-KV attention and the split merge: one launch
            native.attn_decode_fused(q2, k2, v2, self.kcache[i][:batch], self.vcache[i][:batch], self.pos, D, self.theta,
                                     splits=self.splits, workspace=self.attn_ws, out=attn.view(batch, self.nq, D),
                                     rope_angles=self.rope_angles)
        else:
            native.qkv_rope_append(q2, k2, v2, q_rot, self.kcache[i], self.vcache[i], self.pos, batch, seq, D, self.theta)
            total = self._prefill_base + seq
            k = self.kcache[i][:batch, :, :total].transpose(1, 2)
            v = self.vcache[i][:batch, :, :total].transpose(1, 2)
            out, _ = native.attention_forward(q_rot.view(batch, seq, self.nq, D), k, v, True, None)
            attn = out.view(batch * seq, self.nq * D)
        self._row_parallel(attn, L["wo"], x)
        native.norm_forward(x, L["ln2"], None, self.eps, 0, out=n)
        native.gemm_nt(n, L["wgu"], out=act, act="swiglu16")  # gate/up projection with SwiGLU in the epilogue
        self._row_parallel(act, L["wd"], x)

    def _head(self, x, n, logits_local, batch):
        native.norm_forward(x, self.final_norm, None, self.eps, 0, out=n)
        native.gemm_nt(n, self.lm_head, out=logits_local)
        if self.world == 1:
            return logits_local[:batch]
        gathered = self.comm.all_gather(logits_local[:batch].contiguous())  # [world, batch, vocab_local]
        return gathered.permute(1, 0, 2).reshape(batch, self.world * self.vocab_local)

    # -- prefill ----------------------------------------------------------------------------------

    @traced("tpb.engine.prefill")
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, base: int = 0) -> torch.Tensor:
        """Run ``input_ids [batch, seq]`` through the model, fill the cache from position ``base`` and
        return the logits of the last position ``[batch, vocab]`` (fp32)."""
        batch, seq = input_ids.shape
        if batch > self.max_batch or base + seq > self.max_seq:
            raise ValueError("prompt does not fit the engine's cache (max_batch / max_seq)")
        dev, D = self.device, self.head_dim
        bf = dict(dtype=torch.bfloat16, device=dev)
        self._prefill_base = base
        self.pos.fill_(base)
        tokens = batch * seq
        x = native.embedding(input_ids.to(dev).reshape(-1), self.embed)
        n = torch.empty(tokens, self.hidden, **bf)
        qkv = torch.empty(tokens, (self.nq + 2 * self.nkv) * D, **bf)
        q_rot = torch.empty(tokens, self.nq, D, **bf)
        gu = None
        act = torch.empty(tokens, self.ff, **bf)
        for i in range(len(self.layers)):
            self._layer(i, x, n, qkv, q_rot, None, gu, act, batch, seq, decode=False)
        last = x.view(batch, seq, self.hidden)[:, -1].contiguous()
        n_last = torch.empty_like(last)
        logits_local = torch.empty(batch, self.vocab_local, **bf)
        logits = self._head(last, n_last, logits_local, batch)
        self.pos.fill_(base + seq)
        return logits.float()

    # -- decode -----------------------------------------------------------------------------------

    def _decode_body(self, batch: int):
        before = native.launch_count
        native.embedding(self.ids[:batch], self.embed, out=self.x[:batch])
        x, n = self.x[:batch], self.n[:batch]
        for i in range(len(self.layers)):
            self._layer(i, x, n, self.qkv[:batch], self.q_rot[:batch], self.attn[:batch], None, self.act[:batch],
                        batch, 1, decode=True)
        logits = self._head(x, n, self.logits_local[:batch], batch)
        torch.argmax(logits.float(), dim=-1, out=self.next_ids[:batch])
        self.ids[:batch].copy_(self.next_ids[:batch])
        self.pos.add_(1)
        self.kernels_per_step = native.launch_count - before

    @traced("tpb.engine.decode_step")
    @torch.no_grad()
    def decode_step(self, batch: int):
        """One greedy token for every sequence: consumes ``self.ids``, leaves the new ids in ``self.ids``
        / ``self.next_ids`` and advances the cache position.  Captured once per batch size."""
        if not self.use_graph:
            self._decode_body(batch)
            return
        if self.graph is None or self.graph_batch != batch:
            state = self._graph_warmup(batch)
            torch.cuda.synchronize(self.device)
            self._graph_capture(batch, state)
        self.graph.replay()

    # The capture is split in two so that a single host thread can drive several ranks: warm every rank up (the
    # warm-up steps really run and wait for their peers), synchronise all devices, then capture every rank.
    def _graph_warmup(self, batch: int):
        state = (self.pos.clone(), self.ids.clone())
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up outside capture (allocations, plan cache, smem attributes)
                self._decode_body(batch)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        return state

    def _graph_capture(self, batch: int, state):
        if self.comm is not None and (self.comm._call & 1):
            self.comm._call += 1  # keep the workspace alternation phase identical on every replay
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._decode_body(batch)
        self.graph_batch = batch
        self.pos.copy_(state[0])
        self.ids.copy_(state[1])

    def step_from_host(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step driven from the host: pinned int64 ``[batch]`` ids in, next ids out (pinned)."""
        batch = token_ids_host.shape[0]
        self.ids[:batch].copy_(token_ids_host, non_blocking=True)
        self.decode_step(batch)
        if out_host is None:
            out_host = torch.empty(batch, dtype=torch.int64).pin_memory()
        out_host.copy_(self.next_ids[:batch], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy generation: prefill + ``max_new_tokens - 1`` graph-replayed decode steps."""
        batch = input_ids.shape[0]
        logits = self.prefill(input_ids)
        first = logits.argmax(-1)
        out = [first]
        self.ids[:batch].copy_(first)
        for _ in range(max_new_tokens - 1):
            self.decode_step(batch)
            out.append(self.next_ids[:batch].clone())
        return torch.cat([input_ids.to(self.device), torch.stack(out, dim=1)], dim=1)


class EngineGroup:
    """The engines of all ranks of a single-process model (one shard per GPU, all driven by the calling thread).

    Every call enqueues the rank's work on that rank's GPU and moves on: the fused GEMM + all-reduce kernels and the
    device collectives wait (bounded) for their peers on the GPU, never on the host, so one thread can feed all GPUs.
    The only host synchronisation points are the ones the caller asks for (reading a result).

    The decode step is launched kernel by kernel here, not replayed from CUDA graphs: when one thread replayed rank 0's
    graph and then rank 1's, rank 1's graph did not start before rank 0's had run to its end (every peer wait of rank 0
    hit its time limit; measured on two B200s, and the same when each graph was replayed from a host thread of its
    own), whereas eager launches of the same kernels in the same order overlap as expected.  One process per GPU (:class:`LlamaEngine` with a graph per process) remains the fast path."""

    def __init__(self, shards, comms, max_batch: int = 8, max_seq: int = 2560):
        tables = [_unwrap(_unwrap(_unwrap(s).model).embed_tokens).weight.detach() for s in shards]
        hidden = _unwrap(shards[0]).config.hidden_size
        self.engines: List[LlamaEngine] = []
        for shard, comm, own in zip(shards, comms, tables):
            table = own
            if own.shape[1] != hidden:  # hidden-split embedding: every rank keeps a full copy for the lookup kernel
                table = torch.cat([t.to(own.device) for t in tables], dim=1).contiguous()
            with torch.cuda.device(own.device):
                engine = LlamaEngine(shard, comm, max_batch=max_batch, max_seq=max_seq, use_graph=False, embed_table=table)
                engine.preload()
                self.engines.append(engine)
        first = self.engines[0]
        self.max_batch, self.max_seq, self.world, self.device = first.max_batch, first.max_seq, len(self.engines), first.device
        self.comm = first.comm

    @property
    def graph(self):
        return self.engines[0].graph

    @property
    def kernels_per_step(self):
        return self.engines[0].kernels_per_step

    def _each(self, fn):
        out = []
        for e in self.engines:
            with torch.cuda.device(e.device):
                out.append(fn(e))
        return out

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, base: int = 0) -> torch.Tensor:
        ids = input_ids.cpu().pin_memory() if not input_ids.is_cuda else input_ids
        return self._each(lambda e: e.prefill(ids, base))[0]

    @torch.no_grad()
    def decode_step(self, batch: int):
        self._each(lambda e: e._decode_body(batch))

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        batch = input_ids.shape[0]
        ids = input_ids.cpu().pin_memory() if not input_ids.is_cuda else input_ids
        firsts = self._each(lambda e: e.prefill(ids).argmax(-1))  # every rank holds the same gathered logits
        for e, f in zip(self.engines, firsts):
            e.ids[:batch].copy_(f)
        out = [firsts[0]]
        lead = self.engines[0]
        for _ in range(max_new_tokens - 1):
            self.decode_step(batch)
            out.append(lead.next_ids[:batch].clone())
        return torch.cat([input_ids.to(lead.device), torch.stack(out, dim=1)], dim=1)

    def step_from_host(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        batch = token_ids_host.shape[0]
        for e in self.engines:
            e.ids[:batch].copy_(token_ids_host, non_blocking=True)
        self.decode_step(batch)
        lead = self.engines[0]
        if out_host is None:
            out_host = torch.empty(batch, dtype=torch.int64).pin_memory()
        out_host.copy_(lead.next_ids[:batch], non_blocking=True)
        torch.cuda.current_stream(lead.device).synchronize()
        return out_host
