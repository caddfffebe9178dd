"""Carrier for a head-sharded KV cache: one tensor per rank, never replicated.

``TensorParallel.forward`` replicates every *tensor* leaf of its inputs.  A cache wrapped in
``PerDeviceTensors`` is not a tensor, so it travels by reference and each rank picks its own
element.  ``.shape`` / ``.size`` answer from element 0 so that model code can read the cached
length.  Reference: ``src/tensor_parallel/per_device_tensors.py:4-22``.
"""
from __future__ import annotations

import torch


class PerDeviceTensors:
    __slots__ = ("tensors",)

    def __init__(self, *tensors: torch.Tensor):
        self.tensors = tuple(tensors)

    def __getitem__(self, rank: int) -> torch.Tensor:
        return self.tensors[rank]

    def __len__(self) -> int:
        return len(self.tensors)

    def __iter__(self):
        return iter(self.tensors)

    @property
    def shape(self):
        return self.tensors[0].shape

    @property
    def dtype(self):
        return self.tensors[0].dtype

    def size(self, dim=None):
        return self.tensors[0].size() if dim is None else self.tensors[0].size(dim)

    def __repr__(self):
        return f"PerDeviceTensors({', '.join(str(tuple(t.shape)) + '@' + str(t.device) for t in self.tensors)})"
