"""Row-sharded outputs gathered without a collective kernel (quant_ops_b200.sharding.GatheredOutput): on one GPU the
"group" is this process alone, which covers the export of a buffer, the in-kernel gather and the copy-engine gather into
the rank's own buffer; mapping a peer process's buffer needs two GPUs and is checked by `bench.py --gpus N`, whose stack
record verifies every rank's rows of every gathered buffer."""
import ctypes as C
import os
import tempfile

import pytest
import torch
import torch.distributed as dist

import quant_ops_b200 as q
from helpers import N, lib, make_inputs
from oracle import w4a4_oracle as O
from quant_ops_b200 import sharding

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture()
def single_rank_group():
    created = not dist.is_initialized()
    if created:
        store = os.path.join(tempfile.mkdtemp(), "store")
        dist.init_process_group("gloo", init_method=f"file://{store}", rank=0, world_size=1)
    yield
    if created:
        dist.destroy_process_group()


def test_exported_offset_points_back_into_the_allocation():
    pool = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)
    view = pool[4096 + 256:]
    handle = C.create_string_buffer(64)
    offset = C.c_int64(-1)
    N.check(lib.qo_peer_export(C.c_void_p(view.data_ptr()), handle, C.byref(offset)))
    assert offset.value >= 4096 + 256 and (view.data_ptr() - offset.value) % 256 == 0   # the allocation's base address
    assert handle.raw != bytes(64)
    assert lib.qo_peer_export(None, handle, C.byref(offset)) == N.QO_ERR_INVALID_ARGUMENT
    assert lib.qo_peer_close(None) == N.QO_OK


def test_layer_output_lands_in_the_gathered_buffer(single_rank_group):
    tokens, k, n_out = 2048, 4096, 4096
    x, left, right = make_inputs(tokens, k, "bf16", 20280, True)
    g = torch.Generator().manual_seed(20281)
    wq, sw = O.quantize_weights((torch.randn(n_out, k, generator=g) * 0.02).numpy())
    wp, swd = torch.from_numpy(O.pack_int4_to_int32(wq)).to(DEV), torch.from_numpy(sw).to(DEV)
    xd, ld, rd = x.to(DEV), left.to(DEV), right.to(DEV)
    want = q.w4a4_linear(xd, ld, rd, wp, swd, None, 0.9, torch.bfloat16)

    dst = sharding.GatheredOutput(tokens, n_out, torch.bfloat16, torch.device(DEV))
    assert (dst.start, dst.count, dst.ptrs) == (0, tokens, [dst.full.data_ptr()])
    dst.full.fill_(-3.0)
    got = sharding.w4a4_linear_gather(xd, ld, rd, wp, swd, dst, None, 0.9)       # stored by the GEMM's epilogue
    torch.cuda.synchronize()
    assert got is dst.full and torch.equal(got, want)
    q.device_status()

    dst.full.fill_(-3.0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    dst.push_rows(want[:1000].contiguous(), 0, side)                                # copy-engine transfers, in two pieces
    dst.push_rows(want[1000:].contiguous(), 1000, side)
    side.synchronize()
    assert torch.equal(dst.full, want)
    dst.push_rows(dst.local_rows(), 0, include_self=False)                          # nobody else to send to: a no-op
    with pytest.raises(RuntimeError):
        sharding.w4a4_linear_gather(xd[:16], ld, rd, wp, swd, sharding.GatheredOutput(16, n_out, torch.bfloat16, torch.device(DEV)), None, 0.9)
    dst.close()
