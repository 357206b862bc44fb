"""The bounded device waits: every mbarrier wait in the tensor-core kernels gives up after a time limit, records why in a
device status word and lets the kernel unwind.  This test makes a wait run out in the safe form: a one-thread self-test
kernel waits, with a one-millisecond limit, on a barrier whose second arrival never comes.  The kernel returns by itself,
the host reads FLCE_ERR_DEVICE_TIMEOUT once, and the next real call works as usual (nothing traps, nothing is left
spinning)."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_once_and_the_context_stays_usable():
    from flce_cases import make_inputs, oracle_for, run_cuda
    from liger_kernel_b200 import _lib

    lib = _lib.lib
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.flce_b200_check_device_status(st) == 0                 # clean before
    outcome = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.flce_b200_selftest_wait_expiry(1_000_000, C.c_void_p(outcome.data_ptr()), st))
    torch.cuda.synchronize()                                          # the kernel ended by itself
    assert int(outcome.item()) == 2                                   # ... because its wait gave up, not because it completed
    rc = lib.flce_b200_check_device_status(st)
    assert rc == _lib.FLCE_ERR_DEVICE_TIMEOUT
    assert "bounded wait" in lib.flce_b200_last_error().decode() and "status 6" in lib.flce_b200_last_error().decode()
    assert lib.flce_b200_check_device_status(st) == 0                 # reported once, then cleared
    # limits outside (0, 1e8] ns are refused on the host
    assert lib.flce_b200_selftest_wait_expiry(0, C.c_void_p(outcome.data_ptr()), st) == _lib.FLCE_ERR_INVALID_ARGUMENT
    assert lib.flce_b200_selftest_wait_expiry(10**9, C.c_void_p(outcome.data_ptr()), st) == _lib.FLCE_ERR_INVALID_ARGUMENT
    # a real call right after: unaffected
    x, w, t, _, _ = make_inputs(300, 64, 1000, torch.bfloat16, seed=5)
    res = run_cuda(x, w, t)
    ora = oracle_for(x, w, t)
    assert abs(float(res["loss"]) - float(ora.loss)) <= 1e-4 * abs(float(ora.loss))
    assert lib.flce_b200_check_device_status(st) == 0
