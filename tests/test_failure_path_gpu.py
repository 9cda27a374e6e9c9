"""What a host sees when a bounded device-side wait runs out.

The wait is made to run out on purpose and harmlessly: qo_selftest_wait_timeout launches one warp that polls, at most
1024 times, a barrier that nothing arrives on, records a site code and returns.  No trap, no fault, no hang: the
context stays usable, which the test checks by running ordinary work right after."""
import ctypes as C

import pytest
import torch

import quant_ops_b200 as q
from helpers import N, abi_quantize, lib, make_inputs, stream_ptr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_timed_out_wait_is_reported_once_and_the_device_stays_usable():
    x, left, right = make_inputs(16, 4096, "bf16", 9, True)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    ref_c, ref_s = abi_quantize(xd, ld, rd, 0.9, True, "bf16")       # also creates the device status word
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK

    N.check(lib.qo_selftest_wait_timeout(stream_ptr()))
    rc = lib.qo_device_status(stream_ptr())
    assert rc == N.QO_ERR_DEVICE_TIMEOUT
    assert b"0xe00" in lib.qo_last_error().lower()
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK              # reported once, then cleared

    # the Python layer raises for the same condition
    N.check(lib.qo_selftest_wait_timeout(stream_ptr()))
    with pytest.raises(RuntimeError, match="gave up waiting"):
        q.device_status()
    q.device_status()

    # ordinary work after the timed-out kernel: same results as before, status clean
    c, s = abi_quantize(xd, ld, rd, 0.9, True, "bf16")
    assert torch.equal(c, ref_c) and torch.equal(s, ref_s)
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK


def test_status_check_waits_for_the_given_stream():
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        N.check(lib.qo_selftest_wait_timeout(C.c_void_p(side.cuda_stream)))
        with pytest.raises(RuntimeError):
            q.device_status(side)
    q.device_status()
