"""``generate()`` / ``decode_step()`` for tensor-parallel models.

On CUDA, bf16 shards of the families that ``tensor_parallel_b200.engine_spec`` describes (Llama / Mistral /
Qwen2, OPT, Falcon; the self-contained models and the Hugging Face classes) are served by
:class:`tensor_parallel_b200.engine.DecoderEngine` (hand-written kernels, fused GEMM + all-reduce, CUDA-graph
decode).  Everything else — other families, CPU shards, beam search, sampling — goes through the generic loop in
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
        """The kernel-level engine of this model, or ``None`` when it does not apply: the shards must be CUDA bf16
        causal LMs of a family that ``tensor_parallel_b200.engine_spec`` can describe (Llama / Mistral / Qwen2, OPT,
        Falcon - self-contained or Hugging Face classes).

        The engine keeps its own serving-layout copies of the projection weights.  It notices through the tensors'
        version counters when the shard's parameters have been written to since it was built (an optimizer step,
        ``load_state_dict``, a merged adapter) and is rebuilt then; with ZeRO-3 the flat shards are gathered first."""
        from tensor_parallel_b200 import engine_spec

        shard = self.module_shards[0]
        param = next(engine_spec.unwrap(shard).parameters(), None)
        if param is None or not param.is_cuda or param.dtype != torch.bfloat16:
            return None
        manager = getattr(self, "sharding_manager", None)
        if manager is not None:
            with torch.no_grad():
                manager.synchronize_weights(getattr(self, "all_cuda", True))
        eng = self._engine
        if eng is not None and eng.stale():
            self._engine = eng = None
        fits = eng is not None and eng.max_batch >= max_batch and eng.max_seq >= max_seq
        if fits:
            return eng
        if eng is not None and any(e._versions is None for e in getattr(eng, "engines", [eng])):
            raise RuntimeError("the training-layout weights were released (release_training_weights): the engine cannot be "
                               f"rebuilt for max_batch={max_batch}, max_seq={max_seq}; it serves up to {eng.max_batch} x {eng.max_seq}")
        if eng is not None:
            max_batch, max_seq = max(max_batch, eng.max_batch), max(max_seq, eng.max_seq)
        spec = engine_spec.describe(shard, max_seq)
        if spec is None:
            return None
        world = getattr(self, "world_size", 1)
        if len(self.module_shards) > 1:
            # single process, one shard per GPU: one engine per rank on the shared symmetric heaps, one driving thread
            comms = getattr(getattr(self, "_device_backend", None), "comms", None)
            if comms is None or len(comms) != len(self.module_shards):
                return None
            from tensor_parallel_b200.engine import EngineGroup

            self._engine = None  # (frees the old caches before the new ones are allocated)
            try:
                self._engine = EngineGroup(list(self.module_shards), comms, max_batch=max_batch, max_seq=max_seq)
            except ValueError:
                return None
            return self._engine
        comm = self._engine_comm()
        if world > 1 and comm is None:
            return None
        from tensor_parallel_b200.engine import DecoderEngine

        self._engine = None
        self._engine = DecoderEngine(shard, comm if world > 1 else None, max_batch=max_batch, max_seq=max_seq, spec=spec,
                                     process_group=getattr(self, "process_group", None))
        return self._engine

    def release_training_weights(self) -> int:
        """Serving only: once the kernel-level engine exists, frees the parameters it holds in its own layout (see
        ``DecoderEngine.release_source_weights``); returns the bytes freed on this process's devices.  The model then
        serves through ``generate`` / ``prefill`` / ``decode_step`` only."""
        eng = self._engine
        if eng is None:
            raise RuntimeError("build the engine first (serving_engine(), prefill() or generate())")
        if getattr(self, "sharding_manager", None) is not None:
            raise RuntimeError("a model created with sharded=True keeps training state in its parameters; nothing was released")
        engines = getattr(eng, "engines", [eng])
        return sum(e.release_source_weights(shard) for e, shard in zip(engines, self.module_shards))

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
            raise RuntimeError("prefill()/decode_step() need the CUDA serving engine (bf16 shards of a served family)")
        return engine.prefill(input_ids)

    @torch.no_grad()
    def decode_step(self, token_ids_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One greedy decode step driven from the host: copies ``token_ids_host`` (pinned CPU int64
        ``[batch]``) to the GPU, runs the captured step, and returns the next token ids on the host."""
        engine = self._engine
        if engine is None:
            raise RuntimeError("call prefill() first")
        return engine.step_from_host(token_ids_host, out_host)
