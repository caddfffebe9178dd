"""Hugging Face integration: a ``PreTrainedModel`` that holds a :class:`TensorParallel` as
``wrapped_model`` so ``generate()``, ``save_pretrained()`` and ``Trainer`` keep working.

State-dict keys carry the ``wrapped_model.`` prefix in the sharded layout and lose it in the
un-sharded one.  Generation helpers that only inspect the model are delegated to shard 0; the
KV cache stays head-sharded across calls and beam search reorders it per rank.
Reference: ``src/tensor_parallel/pretrained_model.py:21-162``.
"""
from __future__ import annotations

import logging
from typing import Any, Dict, Optional, Sequence

import torch
from torch import nn
from transformers import PreTrainedModel

try:  # transformers >= 4.50 no longer mixes generation into PreTrainedModel
    from transformers import GenerationMixin
except Exception:  # pragma: no cover
    GenerationMixin = object

from tensor_parallel_b200.parallel.families import find_predefined_tensor_parallel_config
from tensor_parallel_b200.parallel.kv import PerDeviceTensors
from tensor_parallel_b200.parallel.rules import Config
from tensor_parallel_b200.parallel.runtime import TensorParallel
from tensor_parallel_b200.utils.nested import nested_map

logger = logging.getLogger(__name__)

_BASES = (PreTrainedModel,) if issubclass(PreTrainedModel, GenerationMixin) or GenerationMixin is object else (PreTrainedModel, GenerationMixin)


class TensorParallelPreTrainedModel(*_BASES):
    is_parallelizable = model_parallel = True
    _supports_sdpa = _supports_flash_attn_2 = _supports_flex_attn = _supports_attention_backend = True
    _supports_cache_class = True

    def __init__(
        self,
        module: PreTrainedModel,
        device_ids: Optional[Sequence[torch.device]] = None,
        output_device: Optional[torch.device] = None,
        output_device_index: Optional[int] = None,
        tensor_parallel_config: Optional[Config] = None,
        **kwargs,
    ):
        super().__init__(module.config)
        if hasattr(module, "_hf_hook"):
            try:
                from accelerate.hooks import remove_hook_from_module

                remove_hook_from_module(module, recurse=True)
            except ImportError:
                logger.warning("module carries accelerate hooks but accelerate is not importable; hooks left in place")
        if tensor_parallel_config is None:
            tensor_parallel_config = find_predefined_tensor_parallel_config(module.config, device_ids)
            if tensor_parallel_config is not None:
                tensor_parallel_config = _validated_or_none(module, tensor_parallel_config)
        if getattr(module, "generation_config", None) is not None:
            self.generation_config = module.generation_config
        self.wrapped_model = TensorParallel(module, device_ids, output_device, output_device_index, tensor_parallel_config, **kwargs)

    @property
    def devices(self):
        return self.wrapped_model.devices

    @property
    def tensor_parallel_config(self):
        return self.wrapped_model.tensor_parallel_config

    @property
    def device(self):  # generate() places new tensors here
        return self.wrapped_model.devices[self.wrapped_model.output_device_index] if self.wrapped_model.devices else torch.device("cpu")

    def set_preserve_shards_when_saving(self, value: bool):
        self.wrapped_model.set_preserve_shards_when_saving(value)

    def apply_sharding(self, *args, **kwargs):
        self.wrapped_model.apply_sharding(*args, **kwargs)

    def forward(self, *args, **kwargs):
        return self.wrapped_model(*args, **kwargs)

    def state_dict(self, *args, **kwargs):
        state = super().state_dict(*args, **kwargs)
        if self.wrapped_model.preserve_shards_when_saving:
            return state
        prefix = kwargs.get("prefix", "")
        head = prefix + "wrapped_model."
        for key in [k for k in state if k.startswith(head)]:
            state[prefix + key[len(head):]] = state.pop(key)
        return state

    # -- generation: plain greedy decoding of a served family runs on the kernel-level engine ----------

    _ENGINE_KWARGS = {"max_new_tokens", "max_length", "do_sample", "num_beams", "attention_mask", "use_cache", "pad_token_id",
                      "eos_token_id", "input_ids"}

    @torch.no_grad()
    def generate(self, inputs: Optional[torch.Tensor] = None, generation_config=None, **kwargs):
        """``GenerationMixin.generate`` with one shortcut: greedy decoding of a full-attention prompt on CUDA bf16 shards
        of a family the serving engine describes (``tensor_parallel_b200.engine_spec``) runs there - hand-written
        kernels, fused GEMM + all-reduce, no Python per layer - and returns what the Hugging Face loop would return
        (tokens after an end-of-sequence token are replaced by the pad token).  Everything else (sampling, beams,
        logits processors, padded prompts, streamers ...) takes the stock path through ``forward``."""
        ids = inputs if inputs is not None else kwargs.get("input_ids")
        engine_ok = (
            generation_config is None and isinstance(ids, torch.Tensor) and ids.ndim == 2 and ids.dtype in (torch.int64, torch.int32)
            and set(kwargs) <= self._ENGINE_KWARGS
            and not (kwargs.get("do_sample") if kwargs.get("do_sample") is not None else getattr(self.generation_config, "do_sample", None))
            and (kwargs.get("num_beams") or getattr(self.generation_config, "num_beams", None) or 1) == 1
            and kwargs.get("use_cache", True) is not False
            and (kwargs.get("attention_mask") is None or bool(kwargs["attention_mask"].all()))
            and getattr(self.generation_config, "repetition_penalty", None) in (None, 1.0)
        )
        if engine_ok:
            new = kwargs.get("max_new_tokens")
            if new is None:
                total = kwargs.get("max_length", getattr(self.generation_config, "max_length", None))
                new = None if total is None else total - ids.shape[1]
            engine = self.wrapped_model.serving_engine(ids.shape[0], ids.shape[1] + (new or 0) + 4) if new and new > 0 else None
            if engine is not None:
                out = engine.generate(ids, new)
                eos = kwargs.get("eos_token_id", getattr(self.generation_config, "eos_token_id", None))
                if eos is not None:
                    pad = kwargs.get("pad_token_id", getattr(self.generation_config, "pad_token_id", None))
                    eos_ids = torch.as_tensor(eos if isinstance(eos, (list, tuple)) else [eos], device=out.device)
                    pad = int(eos_ids[0]) if pad is None else pad
                    gen = out[:, ids.shape[1]:]
                    ended = torch.isin(gen, eos_ids).cumsum(1)
                    after = (ended - torch.isin(gen, eos_ids).long()) > 0  # strictly after the first end-of-sequence token
                    gen.masked_fill_(after, pad)
                    alive = (~(ended > 0)).any(0).nonzero()
                    keep = int(alive.max()) + 2 if alive.numel() else 1   # the step at which the last sequence ended
                    out = out[:, : ids.shape[1] + min(keep, gen.shape[1])]
                return out
        return super().generate(inputs, generation_config=generation_config, **kwargs)

    # -- generation plumbing: questions about the architecture go to shard 0 -------------------------

    def _shard0(self):
        return self.wrapped_model.module_shards[0]

    def _validate_model_class(self):
        fn = getattr(self._shard0(), "_validate_model_class", None)
        return fn() if fn is not None else None

    def _validate_model_kwargs(self, model_kwargs: Dict[str, Any]):
        fn = getattr(self._shard0(), "_validate_model_kwargs", None)
        return fn(model_kwargs) if fn is not None else None

    def _prepare_model_inputs(self, *args, **kwargs):
        return self._shard0()._prepare_model_inputs(*args, **kwargs)

    def prepare_inputs_for_generation(self, *args, **kwargs):
        return self._shard0().prepare_inputs_for_generation(*args, **kwargs)

    def can_generate(self) -> bool:
        if "wrapped_model" not in self._modules:  # called from PreTrainedModel.__init__
            return True
        shard = self._shard0()
        return bool(shard.can_generate()) if hasattr(shard, "can_generate") else True

    def _reorder_cache(self, past, beam_idx):
        if hasattr(past, "reorder_cache"):  # stateful cache object: siblings on other ranks mirror the call
            past.reorder_cache(beam_idx)
            return past
        from tensor_parallel_b200.models.generation import reorder_cache

        if not hasattr(self._shard0(), "_reorder_cache"):
            return reorder_cache(past, beam_idx)
        for rank, shard in enumerate(self.wrapped_model.module_shards):
            local = nested_map(lambda leaf: leaf[rank] if isinstance(leaf, PerDeviceTensors) else leaf, past)
            shard._reorder_cache(local, beam_idx.to(self.wrapped_model.devices[rank]))
        return past

    def get_encoder(self):
        cached = self.__dict__.get("_tp_encoder")
        if cached is not None:
            return cached
        tp = self.wrapped_model
        if len(tp.module_shards) == 1:
            encoder = tp.module_shards[0].get_encoder()
        else:
            encoder = ParallelEncoder(tp, [shard.get_encoder() for shard in tp.module_shards])
        self.__dict__["_tp_encoder"] = encoder
        return encoder


class ParallelEncoder(nn.Module):
    """Runs only the encoder of every shard (used by ``generate()`` of encoder-decoder models)."""

    def __init__(self, tp: TensorParallel, encoder_shards):
        super().__init__()
        self.__dict__["tp"] = tp
        self.__dict__["encoder_shards"] = list(encoder_shards)

    def forward(self, *args, **kwargs):
        tp = self.__dict__["tp"]
        tp._materialize()
        if tp.sharding_manager is not None:
            tp.sharding_manager.synchronize_weights(tp.all_cuda)
        return tp.run_shards(self.__dict__["encoder_shards"], args, kwargs)


def get_parallel_encoder(tp_model: TensorParallel):
    """``get_encoder()`` for a plain :class:`TensorParallel` over an encoder-decoder module."""
    if len(tp_model.module_shards) == 1:
        return tp_model.module_shards[0].get_encoder()
    return ParallelEncoder(tp_model, [shard.get_encoder() for shard in tp_model.module_shards])


def _validated_or_none(module: nn.Module, config: Config) -> Optional[Config]:
    """Predefined tables name per-module attributes of a particular ``transformers`` era.  If the
    installed version's modules no longer match (no state rule hits, or wrapped modules changed
    their call signature), fall back to the automatic config rather than mis-slicing."""
    names = [n for n, _ in module.named_parameters()]
    hits = sum(1 for pattern in config.state_rules for n in names if pattern.search(n))
    if hits == 0:
        logger.warning("predefined config matches no parameter of %s; using the automatic config", type(module).__name__)
        return None
    import inspect

    by_name = dict(module.named_modules())
    for pattern, mapped in config.input_rules.items():
        for name, sub in by_name.items():
            if pattern.search(name) is None:
                continue
            params = inspect.signature(sub.forward).parameters
            accepts_any = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values())
            missing = [k for k in mapped if isinstance(k, str) and k not in params]
            if missing and not accepts_any:
                logger.warning(
                    "predefined config expects %s.forward(%s=...) which this transformers version lacks; "
                    "using the automatic config", type(sub).__name__, missing[0])
                return None
            break
    return config
