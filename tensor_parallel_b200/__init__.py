"""B200-native automatic tensor parallelism for PyTorch.

Public API (same names as ``tensor_parallel``, reference ``src/tensor_parallel/__init__.py:6-13``)::

    import tensor_parallel_b200 as tp
    model = tp.tensor_parallel(model, ["cuda:0", "cuda:1"])
"""
from tensor_parallel_b200.parallel.actions import (
    LegacyStateAction,
    Scale,
    Split,
    SplitInChunks,
    SplitInGroupedChunks,
    StateAction,
)
from tensor_parallel_b200.parallel.checkpoint import (
    convert_state_dict,
    infer_sharded_device_map,
    load_sharded_state_dict_,
    replicated_parameter_names,
    save_tensor_parallel,
)
from tensor_parallel_b200.parallel.collectives import CollectiveOperation, TPCollectiveError
from tensor_parallel_b200.parallel.distributed import DistributedTensorParallel
from tensor_parallel_b200.parallel.factory import tensor_parallel
from tensor_parallel_b200.parallel.families import PREDEFINED_CONFIGS, find_predefined_tensor_parallel_config, register_predefined_config
from tensor_parallel_b200.utils import tracing
from tensor_parallel_b200.parallel.kv import PerDeviceTensors
from tensor_parallel_b200.parallel.legacy import Sharded
from tensor_parallel_b200.parallel.rules import Config
from tensor_parallel_b200.parallel.runtime import TensorParallel
from tensor_parallel_b200.parallel.surgery import make_distributed_shard, make_shard
from tensor_parallel_b200 import optim  # noqa: E402,F401


def __getattr__(name):
    if name == "TensorParallelPreTrainedModel":  # imports transformers lazily
        from tensor_parallel_b200.parallel.hf import TensorParallelPreTrainedModel

        return TensorParallelPreTrainedModel
    raise AttributeError(name)


__version__ = "0.1.0"
