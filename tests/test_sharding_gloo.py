"""The multi-rank host logic (row sharding and the final all-gather) on CPU
with the gloo backend, world size 2 and 3, including ragged shards."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total_rows, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "onnx-mlir_b200"))
    from omcuda.sharding import gather_rows, shard_rows
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(total_rows * 6, dtype=torch.float32).reshape(total_rows, 2, 3)
        first, rows = shard_rows(total_rows, world, rank)
        local = full[first:first + rows] * 2.0     # the rank's "forward pass"
        out = gather_rows(local, total_rows)
        ok = bool(torch.equal(out, full * 2.0))
        # the queued form exists for even CUDA shards only and must say so
        try:
            gather_rows(local, total_rows, async_op=True)
            ok = False
        except ValueError:
            pass
        q.put((rank, ok, tuple(out.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total_rows", [(2, 8), (2, 7), (3, 10), (2, 1)])
def test_shard_and_gather(world, total_rows):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total_rows, q))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, shape in results:
        assert ok, rank
        assert shape == (total_rows, 2, 3)


def test_shard_rows_partition():
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "onnx-mlir_b200"))
    from omcuda.sharding import shard_rows
    for total in (0, 1, 7, 256, 131072):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                first, rows = shard_rows(total, world, r)
                covered += list(range(first, first + rows))
            assert covered == list(range(total))
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)
