"""CPU-side checks of the boundary: the C-ABI library loads without a GPU, exports every symbol the header declares,
and the host-only logic (argument validation, get_decompose_dim) behaves."""
import ctypes as C
import os
import re

import pytest

from helpers import golden
from quant_ops_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "quant_ops_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"QO_API\s+[\w\s\*]+?\b(qo_\w+)\s*\(", text)))


def test_header_declares_and_library_exports_the_same_symbols():
    syms = declared_symbols()
    assert len(syms) >= 18
    raw = C.CDLL(N.LIB_PATH)
    for s in syms:
        assert hasattr(raw, s), f"{s} declared in the header but not exported"
    assert sorted(N.PROTOTYPES) == syms, "python prototypes and header drifted apart"


def test_version_and_status_strings():
    assert N.lib.qo_version() >= 100
    assert N.lib.qo_status_string(0) == b"ok"
    assert b"timed out" in N.lib.qo_status_string(N.QO_ERR_DEVICE_TIMEOUT)


def test_get_decompose_dim_matches_reference_values():
    import quant_ops_b200 as q

    g = golden("decompose")
    for n, (m_ref, n_ref) in zip(g["n"], g["mn"]):
        assert q.get_decompose_dim(int(n)) == (int(m_ref), int(n_ref))
    for bad in (0, -4, 6, 14338):
        with pytest.raises(ValueError):
            q.get_decompose_dim(bad)


def test_argument_validation_needs_no_gpu():
    lib = N.lib
    one = C.c_void_p(16)
    # negative token count, row stride smaller than the row, features not divisible by 8 when packing
    assert lib.qo_flatquant_quantize(one, 16, one, one, one, one, -1, 4, 4, 1.0, N.QO_BF16, 0, N.QO_F32, None) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_flatquant_quantize(one, 8, one, one, one, one, 2, 4, 4, 1.0, N.QO_BF16, 0, N.QO_F32, None) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_flatquant_quantize(one, 15, one, one, one, one, 2, 3, 5, 1.0, N.QO_BF16, 1, N.QO_F32, None) == N.QO_ERR_INVALID_ARGUMENT
    assert b"divisible by 8" in lib.qo_last_error()
    assert lib.qo_flatquant_quantize(one, 16, one, one, one, one, 2, 4, 4, 1.0, 7, 0, N.QO_F32, None) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_int4_matmul(one, 1, one, 1, 1, one, one, one, N.QO_F16, 4, 12, 4, None, None, 0, None) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_int4_matmul(one, 1, one, 1, 1, one, one, one, N.QO_F32, 4, 8, 4, None, None, 0, None) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_pack_int4(one, one, 2, 12, None) == N.QO_ERR_INVALID_ARGUMENT
    # empty problems succeed without touching a device
    assert lib.qo_flatquant_quantize(None, 16, None, None, None, None, 0, 4, 4, 1.0, N.QO_BF16, 0, N.QO_F32, None) == N.QO_OK
    assert lib.qo_int4_matmul(None, 1, None, 1, 1, None, None, None, N.QO_F16, 0, 8, 4, None, None, 0, None) == N.QO_OK
    # kernel policies 0 .. 3 exist; the setting is per thread and is put back
    assert lib.qo_set_kernel_policy(4) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_set_kernel_policy(-1) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_set_kernel_policy(3) == N.QO_OK
    assert lib.qo_set_kernel_policy(0) == N.QO_OK


def test_compute_without_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    one = C.c_void_p(16)
    rc = N.lib.qo_flatquant_quantize(one, 16, one, one, one, one, 2, 4, 4, 1.0, N.QO_BF16, 0, N.QO_F32, None)
    assert rc == N.QO_ERR_NO_DEVICE
    with pytest.raises(N.QuantOpsError):
        N.check(rc)
