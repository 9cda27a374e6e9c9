"""get_decompose_dim: the (M, N) split of a feature count used by the FlatQuant transforms.

Host integer arithmetic, same result as the reference (src/quant_ops/utils/decompose.py:11-38) for every n
that has one; n = 2 (mod 4) has none (a*a - b*b is never 2 mod 4) and raises ValueError where the reference
would loop forever.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

from . import _native


def get_decompose_dim(n: int) -> Tuple[int, int]:
    m_out, n_out = C.c_int64(), C.c_int64()
    status = _native.lib.qo_get_decompose_dim(int(n), C.byref(m_out), C.byref(n_out))
    if status != _native.QO_OK:
        raise ValueError(_native.lib.qo_last_error().decode())
    return int(m_out.value), int(n_out.value)
