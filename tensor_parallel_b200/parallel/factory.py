"""``tensor_parallel()``: the one-call entry point.  Reference: ``src/tensor_parallel/factory.py:17-79``."""
from __future__ import annotations

from typing import Collection, Optional, Sequence, Union

import torch
import torch.distributed
from torch import nn

from tensor_parallel_b200.parallel.rules import Config


def _is_hf_model(module) -> bool:
    try:
        from transformers import PreTrainedModel
    except Exception:
        return False
    return isinstance(module, PreTrainedModel)


def tensor_parallel(
    module: nn.Module,
    device_ids: Optional[Sequence[Union[torch.device, str]]] = None,
    tensor_parallel_config: Optional[Config] = None,
    distributed: Optional[bool] = None,
    sharded: Optional[bool] = None,
    sharded_param_names: Optional[Collection[str]] = None,
    **kwargs,
) -> nn.Module:
    """Wrap ``module`` with tensor parallelism and return an equivalent module.

    :param device_ids: devices to split over; default = every visible CUDA device.  In the
        distributed mode exactly one (this process's) device.
    :param tensor_parallel_config: custom :class:`Config`; default = the predefined table for a
        known model family, else the automatic per-layer config.
    :param distributed: one process per rank over ``torch.distributed``; default = whether a
        process group is initialised.  The result is a module in both modes.
    :param sharded: also ZeRO-3-shard the parameters tensor parallelism left whole.  ``None``
        (the default of this function, unlike the classes) means off.  Supported in both modes.
    :param sharded_param_names: explicit list of parameter names ZeRO-3 applies to.
    """
    if distributed is None:
        distributed = torch.distributed.is_available() and torch.distributed.is_initialized()
    if distributed:
        from tensor_parallel_b200.parallel.distributed import DistributedTensorParallel

        if device_ids is None:
            device_ids = [torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"]
        if len(device_ids) != 1:
            raise ValueError("distributed=True: pass exactly one device, the one this process drives")
        return DistributedTensorParallel(
            module,
            torch.device(device_ids[0]),
            tensor_parallel_config=tensor_parallel_config,
            sharded=bool(sharded),
            sharded_param_names=sharded_param_names,
            **kwargs,
        )
    common = dict(
        device_ids=device_ids,
        tensor_parallel_config=tensor_parallel_config,
        distributed=distributed,
        sharded=sharded,
        sharded_param_names=sharded_param_names,
        **kwargs,
    )
    if _is_hf_model(module):
        from tensor_parallel_b200.parallel.hf import TensorParallelPreTrainedModel

        return TensorParallelPreTrainedModel(module, **common)
    from tensor_parallel_b200.parallel.runtime import TensorParallel

    model_config = getattr(module, "config", None)
    if tensor_parallel_config is None and getattr(model_config, "model_type", None) is not None:
        # self-contained models (tensor_parallel_b200.models) carry a config with a known model_type
        from tensor_parallel_b200.parallel.families import PREDEFINED_CONFIGS
        from tensor_parallel_b200.parallel.runtime import check_device_ids

        if model_config.model_type in PREDEFINED_CONFIGS:
            common["tensor_parallel_config"] = PREDEFINED_CONFIGS[model_config.model_type](model_config, check_device_ids(device_ids))
    return TensorParallel(module, **common)
