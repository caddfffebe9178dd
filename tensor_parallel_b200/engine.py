"""Serving engine for decoder shards: kernel-level prefill and a decode step captured once as a CUDA
graph and replayed per token.

The engine is what ``generate()`` of a tensor-parallel causal LM runs on CUDA.  It is built from a
:class:`~tensor_parallel_b200.engine_spec.DecoderSpec` (Llama / Mistral / Qwen2, OPT, Falcon - the
self-contained models and the Hugging Face classes alike), keeps its weights in a serving layout of its own
and a pre-allocated head-sharded KV cache ``[batch, local_kv_heads, max_seq, head_dim]`` per layer.

Serving layout (engine-owned copies; the shard's parameters are left untouched):

* ``wqkv``: q | k | v rows concatenated, multiplied by the weight of the norm in front of them.  The norm itself
  never runs as a kernel of its own in a decode step: the GEMM computes every token's statistics in its epilogue
  warps while the weights stream and applies them to the accumulators.
* the MLP input projection likewise (gate / up rows interleaved in groups of 16 so that the GEMM epilogue applies
  SwiGLU), the head with the final norm folded in.
* parallel blocks (Falcon): ``[wo | w_down]`` concatenated along K, so that attention output and MLP activation go
  through ONE row-parallel GEMM and one all-reduce per layer.

Kernels per layer of a decode step::

    sequential block   qkv GEMM(+norm) -> [rope + cache append + attention + split merge] -> o_proj GEMM(+all-reduce
                       +residual) -> MLP-in GEMM(+norm +activation) -> MLP-out GEMM(+all-reduce +residual)          = 5
    parallel block     qkv GEMM(+norm) -> attention -> MLP-in GEMM(+norm +activation) -> [o | down] GEMM(+all-reduce
                       +residual)                                                                                   = 4

With several ranks the row-parallel GEMMs push their partial tiles to every peer from the epilogue and reduce
them in the same kernel (decode), or write into symmetric memory and run the device all-reduce (prefill);
nothing goes through NCCL.  The reference reaches the same maths through Python wrappers, host barriers and
one NCCL call per collective (``src/tensor_parallel/tensor_parallel.py:139-161``,
``src/tensor_parallel/communications.py:34-52``).
"""
from __future__ import annotations

import math
import os
from typing import List, Optional

import torch

from tensor_parallel_b200 import engine_spec
from tensor_parallel_b200.ops import native
from tensor_parallel_b200.parallel.actions import unit_bounds
from tensor_parallel_b200.utils.tracing import traced

_unwrap = engine_spec.unwrap
_NORM_MODE = {"rms": 1, "layernorm": 2}


def _fold(weight: torch.Tensor, gamma: Optional[torch.Tensor]) -> torch.Tensor:
    """``weight[f, k] * gamma[k]`` in fp32, rounded once to bf16."""
    if gamma is None:
        return weight.contiguous()
    return (weight.float() * gamma.float()).to(torch.bfloat16).contiguous()


def _beta_term(weight: torch.Tensor, beta: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """``weight @ beta``: what a LayerNorm bias contributes after the projection (fp32)."""
    return None if beta is None else weight.float() @ beta.float()


def _cat_bias(parts, sizes, device) -> Optional[torch.Tensor]:
    if all(p is None for p in parts):
        return None
    return torch.cat([torch.zeros(n, dtype=torch.float32, device=device) if p is None else p.float() for p, n in zip(parts, sizes)])


class DecoderEngine:
    def __init__(self, shard, comm=None, max_batch: int = 8, max_seq: int = 2560, use_graph: bool = True, embed_table=None,
                 process_group=None, replicate_embedding: bool = True, spec: Optional[engine_spec.DecoderSpec] = None,
                 pipeline_prefill: Optional[bool] = None):
        spec = spec if spec is not None else engine_spec.describe(shard, max_seq)
        if spec is None:
            raise ValueError("no serving description for this model (see tensor_parallel_b200.engine_spec)")
        self.spec = spec
        self.comm = comm
        self.process_group = process_group
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.eps, self.mode = spec.eps, _NORM_MODE[spec.norm]
        self.theta, self.head_dim, self.hidden = spec.rope_theta, spec.head_dim, spec.hidden
        self.max_batch, self.max_seq = max_batch, max_seq
        self.use_graph = use_graph and not os.environ.get("TPB_NO_GRAPH")
        # two half-batches in flight during prefill, the all-reduce of one under the GEMMs of the other (one process per
        # GPU only: a single thread that drives every rank launches the ranks' kernels one after the other)
        self.pipeline_prefill = (use_graph if pipeline_prefill is None else pipeline_prefill) and os.environ.get("TPB_PREFILL_PIPELINE", "1") != "0"
        self._side_stream: Optional[torch.cuda.Stream] = None
        self.device = dev = spec.embed.device
        self._versions = tuple(t._version for t in spec.parameters())
        D, H = self.head_dim, self.hidden
        ln = spec.norm == "layernorm"

        # -- embedding ----------------------------------------------------------------------------
        self.embed_split = spec.embed.shape[1] != H
        self.embed_local = spec.embed
        self.pos_local = spec.pos_embed
        self.embed = self.pos_embed = None
        if not self.embed_split:
            self.embed, self.pos_embed = spec.embed, spec.pos_embed
        elif embed_table is not None:
            self.embed, self.pos_embed = embed_table
            self.embed_split = False
        elif replicate_embedding:
            # hidden-split shards gathered once: every rank looks whole rows up (2 * vocab * hidden bytes per rank);
            # replicate_embedding=False keeps the slices and all-gathers [tokens, hidden / world] per call instead
            self.embed = self._gather_columns(spec.embed)
            self.pos_embed = None if spec.pos_embed is None else self._gather_columns(spec.pos_embed)
            self.embed_split = False
        self.col_lo = unit_bounds(H, self.world, self.rank)[0]  # first hidden column of this rank's slice (hidden-split tensors)

        # -- layers ---------------------------------------------------------------------------------
        self.layers = []
        gated = spec.layers[0].w_gate is not None
        self.gated, self.parallel = gated, spec.parallel_block
        self.act = "swiglu16" if gated else spec.act
        if gated and spec.act != "silu":
            raise ValueError("gated MLPs are served with the SiLU gate only")
        for L in spec.layers:
            nq, nk = L.wq.shape[0] // D, L.wk.shape[0] // D
            wqkv_raw = torch.cat([L.wq, L.wk, L.wv], dim=0)
            wqkv = _fold(wqkv_raw, L.ln1_w)
            bqkv = _cat_bias([L.bq, L.bk, L.bv], [L.wq.shape[0], L.wk.shape[0], L.wv.shape[0]], dev)
            beta = _beta_term(wqkv_raw, L.ln1_b)
            if beta is not None:
                bqkv = beta if bqkv is None else bqkv + beta
            ln2_w = L.ln2_w if L.ln2_w is not None else L.ln1_w
            ln2_b = L.ln2_b if L.ln2_w is not None else L.ln1_b
            ff = L.w_up.shape[0]
            w_down, b1 = L.w_down, None
            if gated:
                wg, wu = L.w_gate, L.w_up
                bg = None if L.b_gate is None else L.b_gate.float()
                bu = None if L.b_up is None else L.b_up.float()
                bt_g, bt_u = _beta_term(wg, ln2_b), _beta_term(wu, ln2_b)
                if bt_g is not None:
                    bg = bt_g if bg is None else bg + bt_g
                    bu = bt_u if bu is None else bu + bt_u
                if ff % 16:  # zero rows (and the matching zero columns of the down projection) fill the last group of 16: silu(0) * 0 = 0
                    pad = 16 - ff % 16
                    wg, wu = (torch.cat([w, w.new_zeros(pad, w.shape[1])], dim=0) for w in (wg, wu))
                    w_down = torch.cat([w_down, w_down.new_zeros(w_down.shape[0], pad)], dim=1)
                    if bg is not None:
                        bg, bu = (torch.cat([b, b.new_zeros(pad)]) for b in (bg, bu))
                    ff += pad
                # rows interleaved [16 gate | 16 up] so that the GEMM epilogue applies SwiGLU itself
                w1 = native.interleave_gate_up(_fold(wg, ln2_w), _fold(wu, ln2_w))
                if bg is not None:
                    b1 = torch.stack((bg.reshape(-1, 16), bu.reshape(-1, 16)), dim=1).reshape(-1)
            else:
                w1 = _fold(L.w_up, ln2_w)
                b1 = None if L.b_up is None else L.b_up.float()
                bt = _beta_term(L.w_up, ln2_b)
                if bt is not None:
                    b1 = bt if b1 is None else b1 + bt
            entry = dict(
                wqkv=wqkv, bqkv=None if bqkv is None else bqkv.to(torch.bfloat16),
                sqkv=wqkv.float().sum(1) if ln else None,
                w1=w1, b1=None if b1 is None else b1.to(torch.bfloat16), s1=w1.float().sum(1) if ln else None,
                nq=nq, nkv=nk, ff=ff,
            )
            if self.parallel:
                entry["wcat"] = torch.cat([L.wo, w_down], dim=1).contiguous()
                both = [b for b in (L.bo, L.b_down) if b is not None]
                entry["bcat"] = None if not both else sum(b.float() for b in both).to(torch.bfloat16)
            else:
                entry["wo"], entry["bo"] = L.wo, L.bo
                entry["wd"], entry["bd"] = (w_down if w_down is L.w_down else w_down.contiguous()), L.b_down
            self.layers.append(entry)
        self.nq, self.nkv, self.ff = self.layers[0]["nq"], self.layers[0]["nkv"], self.layers[0]["ff"]

        # -- head -----------------------------------------------------------------------------------
        self.head_split = spec.head_split if self.world > 1 else "vocab"
        gamma, beta = spec.final_ln_w, spec.final_ln_b
        if self.head_split == "hidden":  # tied head: this rank multiplies its column slice of the normalised state
            lo, hi = self.col_lo, self.col_lo + spec.head_w.shape[1]
            gamma, beta = gamma[lo:hi], None if beta is None else beta[lo:hi]
        self.lm_head = _fold(spec.head_w, gamma)
        bhead = _beta_term(spec.head_w, beta)
        self.head_bias = None if bhead is None else bhead.to(torch.bfloat16)
        self.head_rowsum = self.lm_head.float().sum(1) if ln else None
        self.vocab_local = self.lm_head.shape[0]

        # -- cache and static decode buffers ----------------------------------------------------------
        B = max_batch
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.kcache = [torch.zeros(B, self.nkv, max_seq, D, **bf) for _ in self.layers]
        self.vcache = [torch.zeros(B, self.nkv, max_seq, D, **bf) for _ in self.layers]
        self.ids = torch.zeros(B, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.x = torch.zeros(B, H, **bf)
        self.qkv = torch.zeros(B, (self.nq + 2 * self.nkv) * D, **bf)
        cat_cols = self.nq * D + (self.ff if self.parallel else 0)
        self.cat = torch.zeros(B, cat_cols, **bf)       # attention output (| MLP activation of a parallel block)
        self.act_buf = None if self.parallel else torch.zeros(B, self.ff, **bf)
        self.n = torch.zeros(B, H, **bf) if B > 64 else None  # normalised rows, only when a step has too many for the fold
        self.logits_local = torch.zeros(B, self.vocab_local, **bf)
        self.next_ids = torch.zeros(B, dtype=torch.int64, device=dev)
        self.rope_angles = native.rope_table(max_seq, spec.rotary_dim, self.theta, dev) if spec.rotary_dim else None
        # split the key range only when (batch x kv heads) alone cannot occupy the SMs
        # (a KV head's query heads run in groups of up to 4 (head_dim 128) or 8 (64) per CTA, all groups in one launch)
        ctas = B * self.nkv * math.ceil(self.nq / self.nkv / (4 if D == 128 else 8))
        self.splits = 1 if ctas >= 128 else max(1, min(8, math.ceil(256 / ctas)))
        self.attn_ws = (torch.empty(B * self.nq * self.splits * D, dtype=torch.float32, device=dev),
                        torch.empty(B * self.nq * self.splits * 2, dtype=torch.float32, device=dev),
                        torch.zeros(B * self.nq, dtype=torch.int32, device=dev))  # one arrival counter per group of query heads
        self.status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_batch = 0
        self.kernels_per_step = 0
        self._prefill_base = 0

    # -- helpers ------------------------------------------------------------------------------------

    def _gather_columns(self, local: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        parts = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(parts, local.contiguous(), group=self.process_group)
        return torch.cat(parts, dim=1).contiguous()

    def stale(self) -> bool:
        """True when a tensor the serving layout was derived from has been written to since (an optimizer step, a
        ``load_state_dict``, a merged adapter): the engine must be rebuilt."""
        if self._versions is None:  # the source weights were released: nothing left to watch
            return False
        return tuple(t._version for t in self.spec.parameters()) != self._versions

    def _own_tensors(self):
        seen = [self.embed, self.embed_local, self.pos_embed, self.pos_local, self.lm_head, self.head_bias, self.head_rowsum]
        for entry in self.layers:
            seen.extend(entry.values())
        return [t for t in seen if isinstance(t, torch.Tensor)]

    @torch.no_grad()
    def release_source_weights(self, shard) -> int:
        """Serving only: frees every parameter of ``shard`` on this device whose values the engine holds in its own
        layout (q / k / v behind the fused, norm-folded ``wqkv``; gate / up behind the interleaved ``w1``; the head behind
        its folded copy ...) - about two thirds of a Llama shard.  Parameters the engine reads in place (row-parallel
        output projections, the embedding table) stay.  Returns the bytes freed.  Afterwards the module can no longer run
        ``forward()``, be trained or be saved, and the engine stops watching for weight updates."""
        kept = {t.untyped_storage().data_ptr() for t in self._own_tensors()}
        freed, seen = 0, set()
        for param in engine_spec.unwrap(shard).parameters():
            storage = param.untyped_storage()
            if param.device != self.device or storage.data_ptr() in kept or storage.data_ptr() in seen:
                continue
            seen.add(storage.data_ptr())
            freed += storage.nbytes()
        # the description holds views of the same storages: drop them first, then the parameters' own references
        self.spec.layers = []
        self.spec.head_w = self.spec.final_ln_w = self.spec.final_ln_b = None
        self._versions = None
        for param in engine_spec.unwrap(shard).parameters():
            if param.device == self.device and param.untyped_storage().data_ptr() in seen:
                param.data = torch.empty(0, dtype=param.dtype, device=param.device)
        torch.cuda.empty_cache()
        return freed

    def _status_tensor(self):
        return self.comm.status if self.comm is not None else native.device_state(self.device).status

    def check_status(self):
        """Raises if a kernel gave up on a wait (synchronises the device)."""
        (self.comm if self.comm is not None else native.device_state(self.device)).check_status()

    def _embed_tokens(self, ids_flat: torch.Tensor, positions: Optional[torch.Tensor], out=None):
        """Token (+ learned position) embeddings ``[tokens, hidden]``; ``positions`` are absolute cache positions."""
        if not self.embed_split:
            x = native.embedding(ids_flat, self.embed, out=out)
            if self.pos_embed is not None:
                x.add_(self.pos_embed.index_select(0, positions + self.spec.pos_offset))
            return x
        local = native.embedding(ids_flat, self.embed_local)
        if self.pos_local is not None:
            local = local + self.pos_local.index_select(0, positions + self.spec.pos_offset)
        gathered = self.comm.all_gather(local.contiguous())  # [world, tokens, hidden / world]
        x = gathered.permute(1, 0, 2).reshape(ids_flat.numel(), self.hidden)
        if out is not None:
            out.copy_(x)
            return out
        return x.contiguous()

    @torch.no_grad()
    def preload(self, batch: int = 1):
        """Runs the prefill and decode paths once on this rank ALONE (no peer involved; the results are meaningless
        for a shard) so that every kernel they launch - ours and PyTorch's - is loaded on this device.  A single host
        thread that drives several GPUs calls this first: with lazy module loading the first launch of a kernel may
        synchronise the device, which must not happen behind a kernel that waits for a peer not launched yet."""
        comm, world, head_split, embed_split = self.comm, self.world, self.head_split, self.embed_split
        self.comm, self.world, self.head_split = None, 1, "vocab"
        if embed_split:
            self.embed_split, self.embed, self.pos_embed = False, self.embed_local.repeat(1, world), None if self.pos_local is None else self.pos_local.repeat(1, world)
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
            self.comm, self.world, self.head_split = comm, world, head_split
            if embed_split:
                self.embed_split, self.embed, self.pos_embed = True, None, None
        if comm is not None:
            native.check(native.LIB.tpb_comm_preload(), "tpb_comm_preload")

    # -- building blocks --------------------------------------------------------------------------

    def _row_parallel(self, x2d, weight, bias, residual_out):
        """``residual_out += all-reduce(x2d @ weight.T) + bias`` in place (``bias`` is the shard's copy, bias / world)."""
        tokens = x2d.shape[0]
        if self.world == 1:
            native.gemm_nt(x2d, weight, bias=bias, residual=residual_out, out=residual_out)
        elif tokens <= 64 and self.comm.fits_fused(tokens, weight.shape[0], weight.shape[1]):
            self.comm.gemm_allreduce(x2d, weight, bias=bias, residual=residual_out, out=residual_out, bias_scale=float(self.world))
        else:
            staged = self.comm.staging_view("in", (tokens, weight.shape[0]), torch.bfloat16)
            native.gemm_nt(x2d, weight, out=staged)
            residual_out.add_(self.comm.all_reduce(staged))
            if bias is not None:
                residual_out.add_(bias * self.world)

    def _projection(self, x, n, weight, bias, rowsum, out, act=None):
        """``act(norm(x) @ weight.T + bias)`` where ``weight`` already carries the norm weight: for up to 64 tokens the
        GEMM normalises on the fly, otherwise ``n`` holds the rows normalised (without weight) by a kernel in front."""
        if n is None:
            return native.gemm_nt(x, weight, bias=bias, act=act, out=out, norm=(self.mode, self.eps, rowsum))
        return native.gemm_nt(n, weight, bias=bias, act=act, out=out)

    def _layer(self, i, x, n, qkv, q_rot, cat, act_buf, batch, seq, decode: bool):
        L = self.layers[i]
        D, spec = self.head_dim, self.spec
        fold = n is None
        if not fold:
            native.norm_forward(x, None, None, self.eps, self.mode - 1, out=n)
        self._projection(x, n, L["wqkv"], L["bqkv"], L["sqkv"], qkv)
        nq_w, nk_w = self.nq * D, self.nkv * D
        q2, k2, v2 = qkv[:, :nq_w], qkv[:, nq_w : nq_w + nk_w], qkv[:, nq_w + nk_w :]
        attn = cat[:, :nq_w]
        if decode:
            # RoPE, cache append, split-KV attention and the split merge: one launch
            native.attn_decode_fused(q2, k2, v2, self.kcache[i][:batch], self.vcache[i][:batch], self.pos, spec.rotary_dim, self.theta,
                                     interleaved=spec.rope_interleaved, splits=self.splits, workspace=self.attn_ws,
                                     out=attn, rope_angles=self.rope_angles)
        else:
            native.qkv_rope_append(q2, k2, v2, q_rot, self.kcache[i], self.vcache[i], self.pos, batch, seq, spec.rotary_dim, self.theta,
                                   interleaved=spec.rope_interleaved)
            total = self._prefill_base + seq
            k = self.kcache[i][:batch, :, :total].transpose(1, 2)
            v = self.vcache[i][:batch, :, :total].transpose(1, 2)
            native.attention_forward(q_rot.view(batch, seq, self.nq, D), k, v, True, None,
                                     out=attn.unflatten(0, (batch, seq)).unflatten(2, (self.nq, D)))
        if self.parallel:
            # the MLP reads the block input as well (through its own norm weights, folded into w1; the statistics are
            # the same rows'), and both partial results leave through one row-parallel GEMM
            self._projection(x, n, L["w1"], L["b1"], L["s1"], cat[:, nq_w:], act=self.act)
            self._row_parallel(cat, L["wcat"], L["bcat"], x)
            return
        self._row_parallel(attn, L["wo"], L["bo"], x)
        if not fold:
            native.norm_forward(x, None, None, self.eps, self.mode - 1, out=n)
        self._projection(x, n, L["w1"], L["b1"], L["s1"], act_buf, act=self.act)
        self._row_parallel(act_buf, L["wd"], L["bd"], x)

    def _head(self, x, logits_local, batch):
        """Final norm + head on ``x [batch, hidden]``; returns full logits ``[batch, vocab]``."""
        n = None
        if batch > 64:  # too many rows for the in-kernel statistics
            n = native.norm_forward(x, None, None, self.eps, self.mode - 1)[0]
        if self.head_split == "hidden":
            # tied head: statistics over the whole row, contraction over this rank's column slice, partial logits summed
            lo, hi = self.col_lo, self.col_lo + self.lm_head.shape[1]
            if n is None:
                native.gemm_nt(x[:, lo:hi], self.lm_head, bias=self.head_bias, out=logits_local,
                               norm=(self.mode, self.eps, self.head_rowsum), norm_rows=x)
            else:
                native.gemm_nt(n[:, lo:hi], self.lm_head, bias=self.head_bias, out=logits_local)
            if self.comm is None:  # (preload: this rank alone)
                return logits_local[:batch]
            return self.comm.all_reduce(logits_local[:batch].contiguous())
        self._projection(x, n, self.lm_head, self.head_bias, self.head_rowsum, logits_local)
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
        positions = None
        if self.spec.pos_embed is not None:
            positions = torch.arange(base, base + seq, device=dev).repeat(batch)
        x = self._embed_tokens(input_ids.to(dev).reshape(-1), positions)
        n = torch.empty(tokens, self.hidden, **bf) if tokens > 64 else None
        qkv = torch.empty(tokens, (self.nq + 2 * self.nkv) * D, **bf)
        q_rot = torch.empty(tokens, self.nq, D, **bf)
        cat = torch.empty(tokens, self.cat.shape[1], **bf)
        act_buf = None if self.parallel else torch.empty(tokens, self.ff, **bf)
        if self._can_pipeline(batch, seq):
            self._prefill_pipelined(x, n, qkv, q_rot, cat, act_buf, batch, seq)
        else:
            for i in range(len(self.layers)):
                self._layer(i, x, n, qkv, q_rot, cat, act_buf, batch, seq, decode=False)
        last = x.view(batch, seq, self.hidden)[:, -1].contiguous()
        logits_local = torch.empty(batch, self.vocab_local, **bf)
        logits = self._head(last, logits_local, batch)
        self.pos.fill_(base + seq)
        return logits.float()

    def _can_pipeline(self, batch: int, seq: int) -> bool:
        if not self.pipeline_prefill or self.world == 1 or batch < 2 or batch * seq < 1024:
            return False
        region = -(-((batch + 1) // 2 * seq * self.hidden * 2) // 1024) * 1024
        return 2 * region <= self.comm.staging_in.numel()

    def _prefill_pipelined(self, x, n, qkv, q_rot, cat, act_buf, batch: int, seq: int):
        """All layers of a prefill with the batch cut in two halves that take turns: while the row-parallel output of
        one half is summed over the ranks (stand-alone all-reduce kernel on a side stream, in place in its own part of
        the staging buffers), the tensor cores work on the other half.  Collectives run one at a time and in the same
        order on every rank (half 0, half 1, half 0, ...).  The sum is added to the residual stream by the norm kernel
        that opens the next stage (``x += sum; n = norm(x)`` in one pass)."""
        comm, dev, D = self.comm, self.device, self.head_dim
        main = torch.cuda.current_stream(dev)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(dev, priority=-1)  # its CTAs are dispatched ahead of the queued compute kernels'
        side = self._side_stream
        cut = (batch + 1) // 2
        halves = ((0, cut), (cut, batch))
        region = -(-(cut * seq * self.hidden * 2) // 1024) * 1024
        nq_w, nk_w = self.nq * D, self.nkv * D
        # CTAs small enough to be resident beside a GEMM's (measured with a 64 MiB all-reduce beside a 8192 x 8192 x 4096 GEMM
        # at 4 ranks, through the NVSwitch: 557 / 498 / 459 us at 512 / 256 / 128 threads, the GEMM alone 437 us)
        light = 128 if (comm.mc_base and self.world >= 4) else 256
        pending = [None, None]  # per half: (event, summed rows in the staging-out buffer, bias of that projection)

        def rows(t, h):
            return None if t is None else t[halves[h][0] * seq : halves[h][1] * seq]

        def staged(h):
            count = (halves[h][1] - halves[h][0]) * seq
            return comm.staging_in[h * region : h * region + count * self.hidden * 2].view(torch.bfloat16).view(count, self.hidden)

        def reduce_async(h, bias):
            ready = torch.cuda.Event()
            ready.record(main)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                out = comm.all_reduce_staged(h * region, staged(h).shape, block_threads=light)
                done = torch.cuda.Event()
                done.record(side)
            pending[h] = (done, out, bias)

        def open_stage(h):
            """Residual stream of half ``h`` brought up to date, and its normalised rows."""
            xh, nh = rows(x, h), rows(n, h)
            if pending[h] is None:
                native.norm_forward(xh, None, None, self.eps, self.mode - 1, out=nh)
                return xh, nh
            done, red, bias = pending[h]
            pending[h] = None
            main.wait_event(done)
            if bias is None:
                native.norm_forward(xh, None, None, self.eps, self.mode - 1, residual=red, sum_out=xh, out=nh)
            else:
                xh.add_(red).add_(bias * self.world)
                native.norm_forward(xh, None, None, self.eps, self.mode - 1, out=nh)
            return xh, nh

        for i, L in enumerate(self.layers):
            for h, (b0, b1) in enumerate(halves):
                xh, nh = open_stage(h)
                qkv_h, cat_h = rows(qkv, h), rows(cat, h)
                native.gemm_nt(nh, L["wqkv"], bias=L["bqkv"], out=qkv_h)
                q2, k2, v2 = qkv_h[:, :nq_w], qkv_h[:, nq_w : nq_w + nk_w], qkv_h[:, nq_w + nk_w :]
                q_rot_h = rows(q_rot, h)
                native.qkv_rope_append(q2, k2, v2, q_rot_h, self.kcache[i][b0:b1], self.vcache[i][b0:b1], self.pos, b1 - b0, seq,
                                       self.spec.rotary_dim, self.theta, interleaved=self.spec.rope_interleaved)
                total = self._prefill_base + seq
                attn = cat_h[:, :nq_w]
                native.attention_forward(q_rot_h.view(b1 - b0, seq, self.nq, D), self.kcache[i][b0:b1, :, :total].transpose(1, 2),
                                         self.vcache[i][b0:b1, :, :total].transpose(1, 2), True, None,
                                         out=attn.unflatten(0, (b1 - b0, seq)).unflatten(2, (self.nq, D)))
                if self.parallel:
                    native.gemm_nt(nh, L["w1"], bias=L["b1"], act=self.act, out=cat_h[:, nq_w:])
                    native.gemm_nt(cat_h, L["wcat"], out=staged(h))
                    reduce_async(h, L["bcat"])
                else:
                    native.gemm_nt(attn, L["wo"], out=staged(h))
                    reduce_async(h, L["bo"])
            if not self.parallel:
                for h in range(2):
                    xh, nh = open_stage(h)
                    act_h = rows(act_buf, h)
                    native.gemm_nt(nh, L["w1"], bias=L["b1"], act=self.act, out=act_h)
                    native.gemm_nt(act_h, L["wd"], out=staged(h))
                    reduce_async(h, L["bd"])
        for h in range(2):
            done, red, bias = pending[h]
            main.wait_event(done)
            xh = rows(x, h)
            xh.add_(red)
            if bias is not None:
                xh.add_(bias * self.world)

    # -- decode -----------------------------------------------------------------------------------

    def _decode_body(self, batch: int):
        before = native.launch_count
        positions = self.pos.to(torch.int64).expand(batch) if self.spec.pos_embed is not None else None
        self._embed_tokens(self.ids[:batch], positions, out=self.x[:batch])
        x = self.x[:batch]
        for i in range(len(self.layers)):
            self._layer(i, x, self.n[:batch] if batch > 64 else None, self.qkv[:batch], None, self.cat[:batch],
                        None if self.parallel else self.act_buf[:batch], batch, 1, decode=True)
        logits = self._head(x, self.logits_local[:batch], batch)
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

    def _raise_on_status(self):
        code = int(self.status_host[0])
        if code:
            self._status_tensor().zero_()
            from tensor_parallel_b200.parallel.collectives import TPCollectiveError

            what = {1: "an mbarrier wait", 2: "a wait for a peer GPU"}.get(code, f"status {code}")
            raise TPCollectiveError(f"{what} timed out inside a kernel; the results of this step are not valid")

    def step_from_host(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step driven from the host: pinned int64 ``[batch]`` ids in, next ids out (pinned).  The kernels'
        status word travels back with the ids, so a wait that gave up raises here instead of passing stale data on."""
        batch = token_ids_host.shape[0]
        self.ids[:batch].copy_(token_ids_host, non_blocking=True)
        self.decode_step(batch)
        if out_host is None:
            out_host = torch.empty(batch, dtype=torch.int64).pin_memory()
        out_host.copy_(self.next_ids[:batch], non_blocking=True)
        self.status_host.copy_(self._status_tensor(), non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self._raise_on_status()
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
        result = torch.cat([input_ids.to(self.device), torch.stack(out, dim=1)], dim=1)
        self.status_host.copy_(self._status_tensor(), non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self._raise_on_status()
        return result


LlamaEngine = DecoderEngine  # the name the engine had while it served Llama-shaped shards only


class EngineGroup:
    """The engines of all ranks of a single-process model (one shard per GPU, all driven by the calling thread).

    Every call enqueues the rank's work on that rank's GPU and moves on: the fused GEMM + all-reduce kernels and the
    device collectives wait (bounded) for their peers on the GPU, never on the host, so one thread can feed all GPUs.
    The only host synchronisation points are the ones the caller asks for (reading a result).

    The decode step is launched kernel by kernel here, not replayed from CUDA graphs: when one thread replayed rank 0's
    graph and then rank 1's, rank 1's graph did not start before rank 0's had run to its end (every peer wait of rank 0
    hit its time limit; measured on two B200s, and the same when each graph was replayed from a host thread of its
    own), whereas eager launches of the same kernels in the same order overlap as expected.  One process per GPU
    (:class:`DecoderEngine` with a graph per process) remains the fast path."""

    def __init__(self, shards, comms, max_batch: int = 8, max_seq: int = 2560):
        specs = [engine_spec.describe(s, max_seq) for s in shards]
        if any(s is None for s in specs):
            raise ValueError("no serving description for this model")
        hidden = specs[0].hidden
        self.engines: List[DecoderEngine] = []
        for shard, comm, spec in zip(shards, comms, specs):
            table = None
            if spec.embed.shape[1] != hidden:  # hidden-split embedding: every rank keeps a full copy for the lookup kernel
                dev = spec.embed.device
                table = (torch.cat([s.embed.to(dev) for s in specs], dim=1).contiguous(),
                         None if spec.pos_embed is None else torch.cat([s.pos_embed.to(dev) for s in specs], dim=1).contiguous())
            with torch.cuda.device(spec.embed.device):
                engine = DecoderEngine(shard, comm, max_batch=max_batch, max_seq=max_seq, use_graph=False, embed_table=table, spec=spec)
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

    def stale(self) -> bool:
        return any(e.stale() for e in self.engines)

    def check_status(self):
        for e in self.engines:
            e.check_status()

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
        result = torch.cat([input_ids.to(lead.device), torch.stack(out, dim=1)], dim=1)
        for e in self.engines:
            torch.cuda.synchronize(e.device)
        self.check_status()
        return result

    def step_from_host(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        batch = token_ids_host.shape[0]
        for e in self.engines:
            e.ids[:batch].copy_(token_ids_host, non_blocking=True)
        self.decode_step(batch)
        lead = self.engines[0]
        if out_host is None:
            out_host = torch.empty(batch, dtype=torch.int64).pin_memory()
        out_host.copy_(lead.next_ids[:batch], non_blocking=True)
        for e in self.engines:
            with torch.cuda.device(e.device):
                e.status_host.copy_(e._status_tensor(), non_blocking=True)
        for e in self.engines:
            torch.cuda.current_stream(e.device).synchronize()
        for e in self.engines:
            e._raise_on_status()
        return out_host
