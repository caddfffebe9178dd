"""Hand-tuned (Megatron-style) rule tables per model family, keyed by ``config.model_type``.

Each table splits attention by whole heads (keeping every KV group with its query heads),
makes the MLP column-then-row parallel, splits embeddings along the hidden dim and keeps the
KV cache head-sharded between decode steps.  Reference: ``src/tensor_parallel/slicing_configs.py:32-474``
(BLOOM, T5, BERT, GPT-2, GPT-NeoX, CodeGen, Llama, RefinedWeb).  GPT-J, OPT and the
``falcon`` / ``RefinedWebModel`` keys are additions.
"""
from __future__ import annotations

import logging
from typing import Callable, Dict, Optional, Sequence

import torch

from tensor_parallel_b200.parallel.families.decoders import (
    get_bloom_config,
    get_codegen_config,
    get_falcon_config,
    get_gpt2_config,
    get_gpt_neox_config,
    get_gptj_config,
    get_llama_config,
    get_opt_config,
)
from tensor_parallel_b200.parallel.families.encoders import get_bert_config, get_t5_config
from tensor_parallel_b200.parallel.rules import Config

logger = logging.getLogger(__name__)

ConfigGetter = Callable[[object, Sequence[torch.device]], Config]

PREDEFINED_CONFIGS: Dict[str, ConfigGetter] = {
    "bloom": get_bloom_config,
    "t5": get_t5_config,
    "bert": get_bert_config,
    "gpt2": get_gpt2_config,
    "gptj": get_gptj_config,
    "gpt_neox": get_gpt_neox_config,
    "codegen": get_codegen_config,
    "llama": get_llama_config,
    "mistral": get_llama_config,  # same module names and fused-free q / k / v / o, gate / up / down layout as Llama
    "qwen2": get_llama_config,    # ditto, with biases on q / k / v (the rules match weight and bias)
    "qwen3": get_llama_config,    # per-head q / k norms act on head_dim and stay whole
    "gemma": get_llama_config,    # head tied to the embedding table (handled by the table), explicit head_dim
    "gemma2": get_llama_config,
    "opt": get_opt_config,
    "RefinedWeb": get_falcon_config,
    "RefinedWebModel": get_falcon_config,
    "falcon": get_falcon_config,
}


def register_predefined_config(model_type: str, getter: ConfigGetter, overwrite: bool = False) -> None:
    """Adds a rule-table builder ``getter(model_config, devices) -> Config`` for ``model_config.model_type == model_type``.
    The reference offers no such call; its users mutate ``PREDEFINED_CONFIGS`` directly
    (``src/tensor_parallel/slicing_configs.py:465-474``), which still works here."""
    if not callable(getter):
        raise TypeError("getter must be callable as getter(model_config, devices)")
    if model_type in PREDEFINED_CONFIGS and not overwrite:
        raise ValueError(f"a predefined config for model type {model_type!r} exists already (pass overwrite=True to replace it)")
    PREDEFINED_CONFIGS[model_type] = getter


def find_predefined_tensor_parallel_config(model_config, device_ids: Optional[Sequence]) -> Optional[Config]:
    """Rule table for ``model_config.model_type`` or ``None`` (caller falls back to autoconfig)."""
    from tensor_parallel_b200.parallel.runtime import check_device_ids

    devices = check_device_ids(device_ids)
    getter = PREDEFINED_CONFIGS.get(getattr(model_config, "model_type", None))
    if getter is None:
        logger.warning("no predefined tensor-parallel config for this model type; using the automatic config")
        return None
    return getter(model_config, devices)
