"""Deprecated ``Sharded(model)`` spelling: applies ZeRO-3 sharding in place and returns the
same model.  Reference: ``src/tensor_parallel/legacy.py:12-20``."""
import logging

logger = logging.getLogger(__name__)


class Sharded:
    def __new__(cls, module, *args, **kwargs):
        logger.warning("tp.Sharded(model) is deprecated: pass sharded=True to tensor_parallel(), or call model.apply_sharding()")
        module.apply_sharding(*args, **kwargs)
        return module
