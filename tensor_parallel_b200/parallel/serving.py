"""``generate()`` / ``decode_step()`` for tensor-parallel models.

On CUDA, Llama-shaped shards are served by :class:`tensor_parallel_b200.engine.LlamaEngine`
(hand-written kernels, fused GEMM + all-reduce, CUDA-graph decode).  Everything else — other
families, CPU shards, beam search, sampling — goes through the generic loop in
``tensor_parallel_b200.models.generation`` with the head-sharded ``PerDeviceTensors`` cache.
"""
from __future__ import annotations

from typing import Optional

import torch


class ServingMixin:
    _engine = None

    def _engine_comm(self):
        backend = getattr(self, "_device_backend", None)
        return getattr(backend, "comm", None)

    def serving_engine(self, max_batch: int = 8, max_seq: int = 2560):
        """The kernel-level engine of this model, or ``None`` when it does not apply."""
        shard = self.module_shards[0]
        inner = shard.__dict__.get("tp_wrapped_module", shard)
        cfg = getattr(inner, "config", None)
        param = next(inner.parameters(), None)
        if getattr(cfg, "model_type", None) != "llama" or param is None or not param.is_cuda or param.dtype != torch.bfloat16:
            return None
        if type(inner).__module__ != "tensor_parallel_b200.models.llama" or not hasattr(inner, "lm_head"):
            return None  # (a bare LlamaModel without a head has nothing to generate from)
        if getattr(cfg, "tie_word_embeddings", False):
            return None  # the engine expects a vocabulary-split head; a tied head is hidden-split (the generic path serves it)
        world = getattr(self, "world_size", 1)
        eng = self._engine
        fits = eng is not None and eng.max_batch >= max_batch and eng.max_seq >= max_seq
        if eng is not None and not fits:
            max_batch, max_seq = max(max_batch, eng.max_batch), max(max_seq, eng.max_seq)
        if len(self.module_shards) > 1:
            # single process, one shard per GPU: one engine per rank on the shared symmetric heaps, one driving thread
            comms = getattr(getattr(self, "_device_backend", None), "comms", None)
            if comms is None or len(comms) != len(self.module_shards):
                return None
            if not fits:
                from tensor_parallel_b200.engine import EngineGroup

                self._engine = eng = EngineGroup(list(self.module_shards), comms, max_batch=max_batch, max_seq=max_seq)
            return eng
        comm = self._engine_comm()
        if world > 1 and comm is None:
            return None
        if not fits:
            from tensor_parallel_b200.engine import LlamaEngine

            self._engine = eng = LlamaEngine(shard, comm if world > 1 else None, max_batch=max_batch, max_seq=max_seq)
        return eng

    @torch.no_grad()
    def generate(self, input_ids: Optional[torch.Tensor] = None, max_new_tokens: int = 20, **kwargs):
        greedy = not kwargs.get("do_sample", False) and kwargs.get("num_beams", 1) == 1 and not kwargs.get("output_scores", False)
        if input_ids is not None and greedy and set(kwargs) <= {"do_sample", "num_beams", "output_scores"}:
            engine = self.serving_engine(input_ids.shape[0], input_ids.shape[1] + max_new_tokens + 4)
            if engine is not None:
                return engine.generate(input_ids, max_new_tokens)
        from tensor_parallel_b200.models.generation import generate

        return generate(self, input_ids, max_new_tokens=max_new_tokens, **kwargs)

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, max_new_tokens: int = 256) -> torch.Tensor:
        """Engine-backed prompt pass; returns last-position logits ``[batch, vocab]``."""
        engine = self.serving_engine(input_ids.shape[0], input_ids.shape[1] + max_new_tokens + 4)
        if engine is None:
            raise RuntimeError("prefill()/decode_step() need the CUDA serving engine (Llama-shaped bf16 shards)")
        return engine.prefill(input_ids)

    @torch.no_grad()
    def decode_step(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One greedy decode step driven from the host: copies ``token_ids_host`` (pinned CPU int64
        ``[batch]``) to the GPU, runs the captured step, and returns the next token ids on the host."""
        engine = self._engine
        if engine is None:
            raise RuntimeError("call prefill() first")
        return engine.step_from_host(token_ids_host, out_host)
