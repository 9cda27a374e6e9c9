"""Loads the two native pieces: the C-ABI library (ctypes) and the torch dispatcher binding.

Both must be present; there is no Python or CPU fallback.  A missing file raises ImportError naming the build
command, a GPU-less machine can still import the package (the library needs no driver to load) but every
compute entry point then returns QO_ERR_NO_DEVICE.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libquant_ops_b200.so")
BINDING_PATH = os.path.join(PKG, "_torch_binding.so")

QO_OK = 0
QO_ERR_INVALID_ARGUMENT, QO_ERR_UNSUPPORTED, QO_ERR_CUDA, QO_ERR_NO_DEVICE, QO_ERR_WORKSPACE, QO_ERR_DEVICE_TIMEOUT = range(1, 7)
QO_F32, QO_F16, QO_BF16 = 0, 1, 2

_i64, _int, _f32, _vp, _sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/quant_ops_b200.h one to one
PROTOTYPES = {
    "qo_version": (_int, []),
    "qo_status_string": (C.c_char_p, [_int]),
    "qo_last_error": (C.c_char_p, []),
    "qo_get_decompose_dim": (_int, [_i64, C.POINTER(_i64), C.POINTER(_i64)]),
    "qo_flatquant_quantize": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _int, _int, _f32, _int, _int, _int, _vp]),
    "qo_flatquant_transform": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _vp]),
    "qo_device_status": (_int, [_vp]),
    "qo_selftest_wait_timeout": (_int, [_vp]),
    "qo_dequantize_int4": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "qo_int4_matmul_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "qo_int4_matmul": (_int, [_vp, _i64, _vp, _i64, _i64, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp, _vp, _sz, _vp]),
    "qo_int4_matmul_static_max_bytes": (_sz, []),
    "qo_int4_matmul_static": (_int, [_vp, _i64, _vp, _i64, _i64, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    "qo_w4a4_linear_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "qo_w4a4_linear": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _i64, _f32, _int, _int, _vp, _sz, _vp]),
    "qo_w4a4_linear_gather": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, C.POINTER(_vp), _int, _i64, _i64, _int, _int, _i64, _f32, _int, _int, _vp, _sz, _vp]),
    "qo_peer_export": (_int, [_vp, _vp, C.POINTER(_i64)]),
    "qo_peer_open": (_int, [_vp, C.POINTER(_vp)]),
    "qo_peer_close": (_int, [_vp]),
    "qo_peer_copy": (_int, [_vp, _vp, _sz, _vp]),
    "qo_prepared_weights_bytes": (_sz, [_i64, _i64]),
    "qo_prepare_weights": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "qo_w4a4_linear_prepared_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "qo_w4a4_linear_prepared": (_int, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _i64, _f32, _int, _int, _vp, _sz, _vp]),
    "qo_pack_int4": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "qo_unpack_int4": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "qo_quantize_weights_int4": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "qo_flatquant_quantize_host": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _f32, _int, _int, _int]),
    "qo_kernel_launch_count": (C.c_uint64, []),
    "qo_last_quantizer_path": (_int, []),
    "qo_last_gemm_path": (_int, []),
    "qo_set_kernel_policy": (_int, [_int]),
    "qo_release_workspaces": (_int, []),
}


class QuantOpsError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"quant_ops_b200: {message} (status {status})")
        self.status = status


def _load_lib() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python quant_ops_b200/build.py` "
                          "(this package has no fallback implementation)")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load_lib()


def check(status: int) -> None:
    if status != QO_OK:
        raise QuantOpsError(status, f"{lib.qo_status_string(status).decode()}: {lib.qo_last_error().decode()}")


_binding_loaded = False


def load_torch_binding() -> None:
    """Registers torch.ops.quant_ops.* (idempotent)."""
    global _binding_loaded
    if _binding_loaded:
        return
    if not os.path.exists(BINDING_PATH):
        raise ImportError(f"{BINDING_PATH} is missing: build it with `python quant_ops_b200/build.py`")
    import torch

    torch.ops.load_library(BINDING_PATH)
    _binding_loaded = True
