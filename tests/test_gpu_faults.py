"""Device-side failure detection without faulting the GPU: a kernel that waits for a flag nobody sets
gives up after its time limit, records a status code and terminates normally; the host turns the
status into an exception and the context stays usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_survives():
    from tensor_parallel_b200.ops import comm, native

    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    native.check(native.LIB.tpb_wait_flag_test(flag.data_ptr(), 1, status.data_ptr(), 0.25, native._stream()), "wait test")
    stop.record()
    torch.cuda.synchronize()
    assert status[0].item() == 2                      # STATUS_TIMEOUT_FLAG
    assert 200 < start.elapsed_time(stop) < 2000      # gave up after ~0.25 s, not earlier, not never
    # a flag that is already set passes immediately and leaves the status clean
    flag.fill_(5)
    status.zero_()
    native.check(native.LIB.tpb_wait_flag_test(flag.data_ptr(), 3, status.data_ptr(), 0.25, native._stream()), "wait test")
    torch.cuda.synchronize()
    assert status[0].item() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4  # context still works


def test_status_word_becomes_exception():
    from tensor_parallel_b200.ops import native

    state = native.device_state(torch.device("cuda", 0))
    state.status[0] = 2
    with pytest.raises(RuntimeError, match="timed out"):
        state.check_status()
    state.check_status()  # cleared
