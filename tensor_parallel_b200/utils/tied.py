"""Discovery of tied (aliased) parameters / buffers and of LoRA adapter modules.

Reference behaviour: ``src/tensor_parallel/utils.py:109-145`` (alias table keyed by tensor
identity; LoRA detection limited to ``peft.tuners.lora.Linear``).  Here LoRA detection is
structural as well: any module exposing ``lora_A`` / ``lora_B`` containers counts, so newer
``peft`` layouts (``peft.tuners.lora.layer``) and hand-written adapters are recognised.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List

from torch import nn


def find_tied_weight_aliases(module: nn.Module, destination=None, prefix: str = "") -> Dict[int, List[str]]:
    """Map ``id(tensor)`` -> every dotted name under which that tensor is registered."""
    table = OrderedDict() if destination is None else destination
    pending = [(prefix, module)]
    while pending:
        base, mod = pending.pop(0)
        for store in (mod._parameters, mod._buffers):
            for local_name, tensor in store.items():
                if tensor is not None:
                    table.setdefault(id(tensor), []).append(base + local_name)
        children = [(base + child_name + ".", child) for child_name, child in mod._modules.items() if child is not None]
        pending[0:0] = children  # depth-first, registration order
    return table


def check_lora(module: nn.Module) -> bool:
    """Is ``module`` a LoRA-augmented linear layer (base weight + ``lora_A`` / ``lora_B``)?"""
    defined_in = type(module).__module__ or ""
    if defined_in.startswith("peft.tuners.lora") and type(module).__name__ == "Linear":
        return True
    has_pair = isinstance(getattr(module, "lora_A", None), (nn.Module,)) and isinstance(
        getattr(module, "lora_B", None), (nn.Module,)
    )
    return bool(has_pair and hasattr(module, "weight"))
