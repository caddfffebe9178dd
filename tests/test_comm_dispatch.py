"""Dispatch rules of the device collectives that need no GPU: which tensors take the kernel path and which go to
the fallback collective."""
import pytest
import torch


def _comm_module():
    try:
        from tensor_parallel_b200.ops import comm
    except Exception as exc:  # the native library could not be built here
        pytest.skip(f"native library unavailable: {exc!r}")
    return comm


def test_device_all_reduce_keeps_dtype_through_the_fallback():
    comm = _comm_module()
    seen = []

    def fallback(x, rank):
        seen.append((x.dtype, rank))
        return x

    op = comm.DeviceAllReduce(comm=None, fallback=fallback)
    for dtype in (torch.float16, torch.int64, torch.float64):
        x = torch.ones(4, dtype=dtype)
        assert op(x, 1) is x
    assert seen == [(torch.float16, 1), (torch.int64, 1), (torch.float64, 1)]
    # CPU tensors of a supported dtype cannot use the kernels either
    assert op(torch.ones(4, dtype=torch.bfloat16), 0).dtype == torch.bfloat16 and len(seen) == 4
    with pytest.raises(TypeError):
        comm.DeviceAllReduce(comm=None)(torch.ones(2, dtype=torch.float16))


def test_device_wait_limit_follows_the_collective_timeout(monkeypatch):
    from tensor_parallel_b200.ops import native

    monkeypatch.delenv("TPB_DEVICE_WAIT_S", raising=False)
    monkeypatch.setenv("TENSOR_PARALLEL_TIMEOUT", "12")
    assert native.device_wait_seconds() == 12.0
    monkeypatch.setenv("TENSOR_PARALLEL_TIMEOUT", "600")
    assert native.device_wait_seconds() == 30.0
    monkeypatch.setenv("TPB_DEVICE_WAIT_S", "1.5")
    assert native.device_wait_seconds() == 1.5
