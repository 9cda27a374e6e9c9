"""Row sharding of the W4A4 path across the GPUs of one box.

Every stage of the path is independent per token row (reference: src/quant_ops/ops/quantization/flatquant/ops.py:100-117,
cuda_int4_matmul_kernel.cu:114-116), so the tokens are split contiguously over one process per GPU and the int4
weights, weight scales, L and R are replicated.  Nothing on the data path communicates; `all_gather_rows` exists for
callers that need every rank to hold the full output afterwards.
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
