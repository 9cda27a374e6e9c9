"""The allocation-free GEMM entry point (qo_int4_matmul_static) against the regular one.

Some hosts of this library cannot let it allocate: once a serving process has given the GPU's memory to its own
pool there is nothing left for a late cudaMalloc, and an allocation in the middle of a step would stall the device.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import N, QD, abi_int4_matmul, lib, ptr, stream_ptr
from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_matmul(a, b, sa, sb, out_dtype="fp16"):
    t, kp = a.shape
    n = b.shape[1]
    out = torch.empty((t, n), dtype={"fp16": torch.float16, "bf16": torch.bfloat16}[out_dtype], device=a.device)
    N.check(lib.qo_int4_matmul_static(ptr(a), a.stride(0), ptr(b), b.stride(0), b.stride(1), ptr(sa), ptr(sb), ptr(out),
                                      QD[out_dtype], t, kp * 8, n, stream_ptr()))
    torch.cuda.synchronize()
    return out


def problem(t, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-8, 8, (t, k), generator=g, dtype=torch.int8)
    w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
    ap = torch.from_numpy(O.pack_int4_to_int32(a.numpy())).to(DEV)
    wp = torch.from_numpy(O.pack_int4_to_int32(w.numpy())).to(DEV)
    sa = (torch.rand(t, generator=g) * 0.1 + 0.01).to(DEV)
    sb = (torch.rand(n, generator=g) * 0.1 + 0.01).to(DEV)
    return ap, wp, sa, sb


def test_two_calls_in_a_row_match_the_regular_entry_point():
    # two different problems back to back: the second call reuses (and overwrites) the scratch of the first
    for t, k, n, seed in ((300, 4096, 520, 11), (96, 1024, 2048, 12)):
        ap, wp, sa, sb = problem(t, k, n, seed)
        for b in (wp.t(), wp.t().contiguous()):  # transposed weight view and the reference's contiguous layout
            want = abi_int4_matmul(ap, b, sa, sb, "fp16", policy=2)
            got = static_matmul(ap, b, sa, sb, "fp16")
            assert torch.equal(got, want)
            got2 = static_matmul(ap, b, sa, sb, "fp16")
            assert torch.equal(got2, want)
    # qo_device_status also reads (and would clear) the status word that lives inside the library next to the scratch
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK, lib.qo_last_error()


def test_the_call_allocates_no_device_memory():
    """Free device memory, as the driver reports it, is the same before and after a call (and after the status
    check): the scratch is part of the loaded library, nothing is allocated or freed per call."""
    ap, wp, sa, sb = problem(200, 2048, 1024, 21)
    out = torch.empty((200, 1024), dtype=torch.float16, device=DEV)

    def call():
        N.check(lib.qo_int4_matmul_static(ptr(ap), ap.stride(0), ptr(wp), 1, wp.stride(0), ptr(sa), ptr(sb), ptr(out),
                                          N.QO_F16, 200, 2048, 1024, stream_ptr()))
        torch.cuda.synchronize()

    call()  # the first call on a device resolves the addresses of the library's arrays (and loads the kernels)
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    assert lib.qo_device_status(stream_ptr()) == N.QO_OK
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes across allocation-free calls"
    want = abi_int4_matmul(ap, wp.t(), sa, sb, "fp16", policy=2)
    assert torch.equal(out, want)


def test_limits_are_reported_not_exceeded():
    limit = lib.qo_int4_matmul_static_max_bytes()
    assert limit == 8 << 20
    ap, wp, sa, sb = problem(16, 4096, 4096, 3)  # 16*4096 + 4096*4096 bytes = 16 MiB + : over the limit
    out = torch.empty(16, 4096, dtype=torch.float16, device=DEV)
    rc = lib.qo_int4_matmul_static(ptr(ap), ap.stride(0), ptr(wp), 1, wp.stride(0), ptr(sa), ptr(sb), ptr(out), N.QO_F16,
                                   16, 4096, 4096, stream_ptr())
    assert rc == N.QO_ERR_WORKSPACE and b"exceeds" in lib.qo_last_error()
    ap, wp, sa, sb = problem(8, 8, 8, 4)  # k = 8 is not a tcgen05 shape
    out = torch.empty(8, 8, dtype=torch.float16, device=DEV)
    rc = lib.qo_int4_matmul_static(ptr(ap), 1, ptr(wp), 1, 1, ptr(sa), ptr(sb), ptr(out), N.QO_F16, 8, 8, 8, stream_ptr())
    assert rc == N.QO_ERR_UNSUPPORTED
