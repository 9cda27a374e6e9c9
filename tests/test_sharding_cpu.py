"""Host-side logic of the multi-GPU path, run as two gloo ranks on CPU: the row partition and the optional output
gather.  The compute itself needs a GPU and is replaced here by a row-wise stand-in."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from quant_ops_b200 import sharding


def test_shard_rows_partitions_exactly():
    for total in (0, 1, 7, 8, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_rows(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        sharding.shard_rows(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(total * 3, dtype=torch.float32).reshape(total, 3)
        start, count = sharding.shard_rows(total, world, rank)
        row_fn = lambda t: t * 2 + 1  # any row-independent function: the sharded result must equal the unsharded one
        local = sharding.sharded_apply(row_fn, total, full[start:start + count], gather=False)
        assert torch.equal(local, row_fn(full)[start:start + count])
        gathered = sharding.sharded_apply(row_fn, total, full[start:start + count], gather=True)
        assert torch.equal(gathered, row_fn(full))
        keep = torch.empty(total, 3)
        assert sharding.all_gather_rows(local, total, out=keep) is keep and torch.equal(keep, row_fn(full))
        with pytest.raises(ValueError):
            sharding.all_gather_rows(local, total, out=torch.empty(total + 1, 3))
        if rank == fail_rank:  # a rank holding the wrong number of rows is reported on the host, before any collective
            with pytest.raises(ValueError):
                sharding.all_gather_rows(torch.zeros(count + 1, 3), total)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [8, 11])
def test_two_ranks_gloo(total):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, total, 1), nprocs=2, join=True)
