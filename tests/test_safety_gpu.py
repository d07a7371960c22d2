"""The paths a healthy run never takes, exercised without faulting, trapping or
hanging the GPU: a bounded device-side wait that gives up and reports through
the status word, and a launch that the CUDA runtime refuses on the host."""
import ctypes

import pytest
import torch

from conftest import current_stream_ptr

pytestmark = pytest.mark.gpu

OK, LAUNCH_FAILED, DEVICE_TIMEOUT, INVALID_ARGUMENT = 0, 5, 6, 4
WAIT_SELFTEST = 1 << 7


def read_status(abi):
    word = ctypes.c_uint32(0xFFFFFFFF)
    status = abi.b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(current_stream_ptr()))
    return status, word.value


def test_wait_that_nothing_completes_gives_up_and_reports(abi):
    assert read_status(abi) == (OK, 0)
    outcome = torch.zeros(1, dtype=torch.int32, device="cuda")
    # 4096 polls of a barrier nobody arrives on: milliseconds, then the kernel returns by itself.
    assert abi.b200_selftest_wait_gives_up(4096, outcome.data_ptr(), current_stream_ptr()) == OK
    torch.cuda.synchronize()                       # returns: the kernel ended on its own
    assert outcome.item() == 2                     # "gave up", not "completed"
    assert read_status(abi) == (DEVICE_TIMEOUT, WAIT_SELFTEST)
    assert read_status(abi) == (OK, 0)             # reading clears the word
    assert abi.b200_status_string(DEVICE_TIMEOUT) == b"Error Device Wait Timed Out"
    # The context is intact: ordinary work runs and is correct afterwards.
    x = torch.randn(64, 256, device="cuda")
    y = torch.empty_like(x)
    assert abi.b200_softmax(0, x.data_ptr(), y.data_ptr(), 64, 256, current_stream_ptr()) == OK
    torch.testing.assert_close(y, torch.softmax(x, dim=1), atol=1e-6, rtol=1e-5)
    assert read_status(abi) == (OK, 0)


def test_wait_cap_is_bounded_by_the_abi(abi):
    assert abi.b200_selftest_wait_gives_up(0, None, current_stream_ptr()) == INVALID_ARGUMENT
    assert abi.b200_selftest_wait_gives_up((1 << 20) + 1, None, current_stream_ptr()) == INVALID_ARGUMENT


def test_a_refused_launch_does_not_poison_later_calls(abi):
    """The library owns a private CUDA runtime whose per-thread error slot nobody else clears."""
    assert abi.b200_selftest_refused_launch(current_stream_ptr()) == LAUNCH_FAILED
    x = torch.randn(32, 128, device="cuda")
    w = torch.rand(128, device="cuda") + 0.5
    y = torch.empty_like(x)
    assert abi.b200_rmsnorm(0, x.data_ptr(), w.data_ptr(), y.data_ptr(), 32, 128, 1e-6, current_stream_ptr()) == OK
    a = torch.ones(16, 128, device="cuda").t()
    b = torch.ones(16, 128, device="cuda")
    c = torch.empty(128, 128, device="cuda")
    impl = abi.b200_sgemm_impl_from_name(b"prefetch_reg")
    assert abi.b200_sgemm(impl, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 128, 16, current_stream_ptr()) == OK
    torch.cuda.synchronize()
    assert torch.equal(c, torch.full_like(c, 16.0))
    assert read_status(abi) == (OK, 0)
