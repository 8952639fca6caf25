"""The bounded waits of the kernels, exercised without a fault: a self-test kernel waits on an mbarrier
phase that cannot complete (armed for 64 bytes, 32 delivered; the one copy completes, nothing stays
in flight).  The wait has to give up after its limit, the kernel returns, the sticky device flag
reports the time-out, and clearing it restores a healthy status for whatever runs next."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_cannot_complete_gives_up_and_is_reported():
    from adafactor8bit import _native as N
    lib = N.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert N.device_status(stream) == 0
    src = torch.arange(64, dtype=torch.uint8, device="cuda")
    gave_up = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    N.check(lib.af8_selftest_bounded_wait(src.data_ptr(), 5_000_000, gave_up.data_ptr(), stream), "selftest")   # 5 ms
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert int(gave_up.item()) == 1
    assert 0.004 <= elapsed < 1.0, elapsed                   # it waited for its limit, and not much longer
    try:
        assert N.device_status(stream) == 1                   # code of a copy that never completed
        assert N.device_status(stream) == 1                   # sticky until cleared
    finally:
        N.clear_device_status(stream)
    assert N.device_status(stream) == 0
    # the context is intact: an ordinary launch still works
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum().item()) == 2048.0


def test_selftest_rejects_bad_arguments():
    from adafactor8bit import _native as N
    lib = N.lib()
    src = torch.zeros(64, dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.af8_selftest_bounded_wait(None, 1000, out.data_ptr(), None) == N.ERR_INVALID
    assert lib.af8_selftest_bounded_wait(src.data_ptr() + 4, 1000, out.data_ptr(), None) == N.ERR_INVALID
    assert lib.af8_selftest_bounded_wait(src.data_ptr(), 0, out.data_ptr(), None) == N.ERR_INVALID
    assert lib.af8_selftest_bounded_wait(src.data_ptr(), 2_000_000_000, out.data_ptr(), None) == N.ERR_INVALID
