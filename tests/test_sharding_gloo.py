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


def _f32_to_ordered(f):
    """The library's order-preserving float -> uint32 encoding (common.cuh)."""
    u = np.asarray(f, np.float32).view(np.uint32)
    return np.where(u & 0x80000000, ~u, u | 0x80000000).astype(np.uint32)


def _ordered_to_f32(u):
    u = np.asarray(u, np.uint32)
    return np.where(u & 0x80000000, u & 0x7fffffff, ~u).astype(np.uint32).view(np.float32)


def _range_worker(rank, world, port, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "onnx-mlir_b200"))
    from omcuda.sharding import reduce_ranges
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ranges of mixed sign, equal values, infinities (an empty shard)
        rng = np.random.default_rng(100 + rank)
        lo = rng.normal(0, 3, 6).astype(np.float32)
        hi = lo + np.abs(rng.normal(0, 3, 6)).astype(np.float32)
        lo[4], hi[4] = np.float32(1.5), np.float32(1.5)
        if rank == 0:
            lo[5], hi[5] = np.inf, -np.inf          # nothing seen on this rank
        enc = np.stack([_f32_to_ordered(lo), _f32_to_ordered(hi)], -1)
        t = torch.from_numpy(enc.view(np.int32).copy())
        reduce_ranges(t)
        out = t.numpy().view(np.uint32)
        q.put((rank, lo, hi, _ordered_to_f32(out[:, 0]), _ordered_to_f32(out[:, 1])))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_global_quantization_range_reduce(world):
    # The 2-word all-reduce behind omcudaEncoderSetRangeSync: every rank ends up
    # with the minimum of the minima and the maximum of the maxima, exactly.
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_range_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=120) for _ in range(world)), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want_lo = np.min([r[1] for r in results], axis=0)
    want_hi = np.max([r[2] for r in results], axis=0)
    for _, _, _, got_lo, got_hi in results:
        assert got_lo.tobytes() == want_lo.tobytes()
        assert got_hi.tobytes() == want_hi.tobytes()
