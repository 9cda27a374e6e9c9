"""Row sharding of the W4A4 path across the GPUs of one box.

Every stage of the path is independent per token row (reference: src/quant_ops/ops/quantization/flatquant/ops.py:100-117,
cuda_int4_matmul_kernel.cu:114-116), so the tokens are split contiguously over one process per GPU and the int4
weights, weight scales, L and R are replicated.  Nothing on the data path communicates; `all_gather_rows` exists for
callers that need every rank to hold the full output afterwards; `GatheredOutput` + `w4a4_linear_gather` do the same
without a collective: the GEMM's epilogue stores its rows into every rank's buffer over NVLink.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(total: int, world: int, rank: int) -> Tuple[int, int]:
    """(start, count) of `rank`'s contiguous slice of `total` rows; the first `total % world` ranks get one extra."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def shard_sizes(total: int, world: int) -> List[int]:
    return [shard_rows(total, world, r)[1] for r in range(world)]


def all_gather_rows(local: torch.Tensor, total_rows: int, group: Optional[dist.ProcessGroup] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Concatenates the ranks' row slices ([rows_r, cols], slice sizes from shard_rows) into [total_rows, cols].

    `out`, if given, receives the result (a caller that gathers every step keeps one buffer instead of allocating;
    it also lets the collective run on a side stream without the allocator's cross-stream bookkeeping)."""
    world = dist.get_world_size(group)
    sizes = shard_sizes(total_rows, world)
    if local.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError(f"this rank holds {local.shape[0]} rows, its shard of {total_rows} has {sizes[dist.get_rank(group)]}")
    tail = tuple(local.shape[1:])
    if out is not None and (tuple(out.shape) != (total_rows,) + tail or out.dtype != local.dtype or not out.is_contiguous()):
        raise ValueError("out must be a contiguous [total_rows, cols] tensor of the local slice's dtype")
    if len(set(sizes)) == 1:
        if out is None:
            out = local.new_empty((total_rows,) + tail)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # uneven split (sizes differ by at most one row): pad every slice to the largest, gather, drop the padding
    widest = max(sizes)
    padded = local.new_zeros((widest,) + tail)
    padded[: local.shape[0]] = local
    gathered = local.new_empty((world * widest,) + tail)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    pieces = [gathered[r * widest: r * widest + sizes[r]] for r in range(world)]
    if out is None:
        return torch.cat(pieces, dim=0)
    torch.cat(pieces, dim=0, out=out)
    return out


def sharded_apply(fn: Callable[[torch.Tensor], torch.Tensor], x_full_rows: int, x_local: torch.Tensor,
                  gather: bool = False, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Runs `fn` (e.g. a W4A4Linear) on this rank's rows; optionally gathers the outputs of all ranks."""
    y = fn(x_local)
    return all_gather_rows(y, x_full_rows, group) if gather else y


# ---- all-gather fused into the layer's GEMM (one node, CUDA IPC) --------------------------------------------------------
_opened: dict = {}  # exported allocation (handle bytes) -> [base address in this process, users]


def _open_peer(handle: bytes) -> int:
    import ctypes as C

    from . import _native as nat

    entry = _opened.get(handle)
    if entry is None:
        base = C.c_void_p()
        nat.check(nat.lib.qo_peer_open(C.c_char_p(handle), C.byref(base)))
        entry = _opened[handle] = [base.value, 0]
    entry[1] += 1
    return entry[0]


def _close_peer(handle: bytes) -> None:
    import ctypes as C

    from . import _native as nat

    entry = _opened.get(handle)
    if entry is None:
        return
    entry[1] -= 1
    if entry[1] == 0:
        del _opened[handle]
        nat.check(nat.lib.qo_peer_close(C.c_void_p(entry[0])))


class GatheredOutput:
    """A layer output [total_rows, cols] that every rank of the group holds in full and that the ranks fill for one
    another: `full` is this rank's buffer, `ptrs[r]` is rank r's buffer as seen from this process.  Ranks are the
    processes of ONE node (CUDA IPC).  `close()` unmaps the peers' buffers; call it on every rank, after a barrier that
    follows the last kernel writing them, and before the buffers are freed."""

    def __init__(self, total_rows: int, cols: int, dtype: torch.dtype, device: Optional[torch.device] = None,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes as C

        from . import _native as nat

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        self.full = torch.empty(total_rows, cols, dtype=dtype, device=device if device is not None else torch.cuda.current_device())
        self.start, self.count = shard_rows(total_rows, self.world, self.rank)
        handle = C.create_string_buffer(64)
        offset = C.c_int64()
        nat.check(nat.lib.qo_peer_export(C.c_void_p(self.full.data_ptr()), handle, C.byref(offset)))
        mine = (handle.raw, int(offset.value))
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._handles: List[bytes] = []
        self.ptrs: List[int] = []
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                self.ptrs.append(self.full.data_ptr())
            else:
                self.ptrs.append(_open_peer(h) + off)
                self._handles.append(h)

    def close(self) -> None:
        for h in self._handles:
            _close_peer(h)
        self._handles = []

    def local_rows(self) -> torch.Tensor:
        """This rank's rows of its own buffer: a layer that writes its output here needs no local copy afterwards."""
        return self.full[self.start:self.start + self.count]

    def push_rows(self, local: torch.Tensor, first_row: int, stream: Optional[torch.cuda.Stream] = None,
                  include_self: bool = True) -> None:
        """Copies `local` ([rows, cols], rows first_row .. of the gathered output, contiguous) into every rank's buffer
        (this rank's too unless include_self is False, e.g. when `local` already is a view of local_rows()) with
        copy-engine transfers on `stream` (default: the current stream): they take no SM, so on a side stream they run
        beside the next layer's kernels at the NVLink rate."""
        import ctypes as C

        from . import _native as nat

        if not local.is_contiguous() or tuple(local.shape[1:]) != tuple(self.full.shape[1:]) or local.dtype != self.full.dtype:
            raise ValueError("local must be a contiguous [rows, cols] tensor of the gathered output's dtype")
        sp = C.c_void_p((stream or torch.cuda.current_stream(local.device)).cuda_stream)
        row_bytes = self.full.stride(0) * self.full.element_size()
        nbytes = local.shape[0] * row_bytes
        for r in range(self.world if include_self else self.world - 1):  # peers first, each rank starting at its neighbour
            order = (self.rank + 1 + r) % self.world
            nat.check(nat.lib.qo_peer_copy(C.c_void_p(self.ptrs[order] + first_row * row_bytes), C.c_void_p(local.data_ptr()), nbytes, sp))


def w4a4_linear_gather(x_local: torch.Tensor, left_trans: torch.Tensor, right_trans: torch.Tensor, w_packed: torch.Tensor,
                       w_scale: torch.Tensor, dst: GatheredOutput, bias: Optional[torch.Tensor] = None,
                       clip_ratio: float = 1.0, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The fused layer on this rank's rows, its outputs stored by the GEMM into every rank's `dst` buffer (rows
    dst.start .. dst.start + dst.count).  Returns dst.full, whose other rows the other ranks fill: it is complete after
    every rank's call has finished and the ranks have met (a stream synchronise, then a barrier).  Raises for shapes the
    fused kernel does not take (small token counts): gather those with all_gather_rows."""
    import ctypes as C

    from . import _native as nat

    tokens, k = x_local.shape
    if tokens != dst.count:
        raise ValueError(f"this rank holds {tokens} rows, its shard has {dst.count}")
    m, n = left_trans.shape[0], right_trans.shape[0]
    n_out = w_packed.shape[0]
    if tuple(dst.full.shape[1:]) != (n_out,) or dst.full.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("dst must be [total_rows, n_out] in float16 or bfloat16")
    qd = {torch.float16: nat.QO_F16, torch.bfloat16: nat.QO_BF16, torch.float32: nat.QO_F32}
    ptrs = (C.c_void_p * dst.world)(*dst.ptrs)
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (C.c_void_p(workspace.data_ptr()), workspace.numel() * workspace.element_size())
    stream = C.c_void_p(torch.cuda.current_stream(x_local.device).cuda_stream)
    nat.check(nat.lib.qo_w4a4_linear_gather(
        C.c_void_p(x_local.data_ptr()), x_local.stride(0), C.c_void_p(left_trans.data_ptr()), C.c_void_p(right_trans.data_ptr()),
        C.c_void_p(w_packed.data_ptr()), C.c_void_p(w_scale.data_ptr()), None if bias is None else C.c_void_p(bias.data_ptr()),
        ptrs, dst.world, dst.start, tokens, m, n, n_out, float(clip_ratio), qd[x_local.dtype], qd[dst.full.dtype],
        ws_ptr, ws_bytes, stream))
    return dst.full
