"""Host-side behaviour of the Python operator layer (no GPU needed): names, fake kernels, no CPU fallback."""
import pytest
import torch

import quant_ops_b200 as q


def test_public_names_of_the_reference_are_present():
    for name in ("flatquant_dynamic_quantize", "dequantize_int4", "int4_matmul", "get_decompose_dim", "CUDA_AVAILABLE"):
        assert hasattr(q, name)
    for op in ("flatquant_dynamic_quantize", "int4_matmul"):
        assert hasattr(torch.ops.quant_ops, op)


def test_cpu_tensors_raise_instead_of_falling_back():
    x = torch.randn(4, 16)
    eye = torch.eye(4)
    with pytest.raises((NotImplementedError, RuntimeError)):
        q.flatquant_dynamic_quantize(x, eye, eye)
    with pytest.raises((NotImplementedError, RuntimeError)):
        q.int4_matmul(torch.zeros(2, 1, dtype=torch.int32), torch.zeros(1, 2, dtype=torch.int32), torch.ones(2), torch.ones(2))
    with pytest.raises((NotImplementedError, RuntimeError)):
        q.dequantize_int4(torch.zeros(2, 8, dtype=torch.int8), torch.ones(2))


def test_fake_kernels_give_the_reference_shapes_and_dtypes():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(8, 4096, device="cuda", dtype=torch.bfloat16)
        lr = torch.empty(64, 64, device="cuda", dtype=torch.bfloat16)
        c, s = q.flatquant_dynamic_quantize(x, lr, lr, 0.9, True)
        assert c.shape == (8, 512) and c.dtype == torch.int32 and s.shape == (8,) and s.dtype == torch.float32
        c, s = q.flatquant_dynamic_quantize(x, lr, lr, 1.0, False)
        assert c.shape == (8, 4096) and c.dtype == torch.int8
        w = torch.empty(512, 96, device="cuda", dtype=torch.int32)
        out = q.int4_matmul(torch.empty(8, 512, device="cuda", dtype=torch.int32), w, s, torch.empty(96, device="cuda"))
        assert out.shape == (8, 96) and out.dtype == torch.float16
        d = q.dequantize_int4(c, s, False)
        assert d.shape == (8, 4096) and d.dtype == torch.float32
        wp = torch.empty(96, 512, device="cuda", dtype=torch.int32)
        y = q.w4a4_linear(x, lr, lr, wp, torch.empty(96, device="cuda"), None, 0.9)
        assert y.shape == (8, 96) and y.dtype == torch.bfloat16
