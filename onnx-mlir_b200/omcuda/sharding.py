"""Row (batch) sharding of the quantized path across the GPUs of one box.

Every output row of the path depends on one input row and the replicated
weights, so ranks take contiguous row ranges and never exchange data inside a
forward pass; the only collective is the final all-gather of output rows.
Per-tensor dynamic quantization then uses each rank's own min/max ("replica
mode"): a rank's result equals the reference's result on that rank's rows.

Global-quantization mode (optional): the encoder harness can call a hook for
every DynamicQuantizeLinear range (omcudaEncoderSetRangeSync); reduce_ranges /
make_range_sync below implement it as one 2-word all-reduce, after which every
rank quantizes with the range of the WHOLE batch and the sharded run equals
the reference's run on the whole batch bit for bit.
"""
import ctypes

import torch
import torch.distributed as dist

_INT_MIN = -0x80000000


def reduce_ranges(t, group=None):
    """t: int32 tensor [..., 2] holding, as raw bits, the order-preserving
    uint32 encodings of running {min, max} (larger encoding = larger float).
    Replaces every pair in place by {min over ranks, max over ranks}.
    Flipping the top bit turns the unsigned order into int32 order; the
    bitwise complement of the second word turns its maximum into a minimum, so
    one MIN all-reduce serves both."""
    v = t ^ _INT_MIN
    v[..., 1] = ~v[..., 1]
    dist.all_reduce(v, op=dist.ReduceOp.MIN, group=group)
    v[..., 1] = ~v[..., 1]
    t.copy_(v ^ _INT_MIN)
    return t


class _DevWords:
    """Two int32 words of device memory as a zero-copy torch tensor."""

    def __init__(self, ptr):
        self.__cuda_array_interface__ = {"shape": (2,), "typestr": "<i4",
                                         "data": (int(ptr), False), "version": 2}


RANGE_SYNC_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p)


def make_range_sync(group=None, via_host=False):
    """The omcudaRangeSyncFn for omcudaEncoderSetRangeSync.  The all-reduce is
    queued in `stream` order (NCCL on device tensors); via_host routes it
    through two host words instead (for process groups without device
    collectives, e.g. gloo in tests).  Keep the returned object alive while
    the encoder may call it."""
    def fn(_ctx, range_ptr, stream):
        with torch.cuda.stream(torch.cuda.ExternalStream(int(stream or 0))):
            t = torch.as_tensor(_DevWords(range_ptr), device="cuda")
            if via_host:
                h = t.cpu()
                reduce_ranges(h, group)
                t.copy_(h)
            else:
                reduce_ranges(t, group)
    return RANGE_SYNC_FN(fn)


def shard_rows(total_rows, world, rank):
    """Contiguous, balanced split: returns (first_row, rows) of `rank`.
    The first total_rows % world ranks hold one row more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank %r/%r" % (world, rank))
    base, extra = divmod(int(total_rows), world)
    rows = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, rows


def gather_rows(local, total_rows, group=None, out=None, async_op=False):
    """All-gathers row shards made by shard_rows back into [total_rows, ...].
    `local` is this rank's [rows, ...] tensor (CPU with gloo, CUDA with nccl).
    Ragged shards are padded to the largest shard for the collective.  `out`
    (optional, [total_rows, ...]) is filled in place when the shards are even.
    With async_op (even CUDA shards only) the collective is only queued:
    returns (out, work), and `out` is complete once work.wait() has been
    called and the current stream has reached that point."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    first, rows = shard_rows(total_rows, world, rank)
    if local.shape[0] != rows:
        raise ValueError("rank %d holds %d rows, expected %d" % (rank, local.shape[0], rows))
    max_rows = -(-int(total_rows) // world)
    tail = tuple(local.shape[1:])
    if rows == max_rows:
        padded = local.contiguous()
    else:
        padded = torch.zeros((max_rows,) + tail, dtype=local.dtype, device=local.device)
        padded[:rows] = local
    if total_rows % world == 0 and local.is_cuda:
        if out is None:
            out = torch.empty((total_rows,) + tail, dtype=local.dtype,
                              device=local.device)
        if async_op:
            return out, dist.all_gather_into_tensor(out, padded, group=group, async_op=True)
        dist.all_gather_into_tensor(out, padded, group=group)
        return out
    if async_op:
        raise ValueError("async_op needs even shards on CUDA")
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    pieces = [parts[r][:shard_rows(total_rows, world, r)[1]] for r in range(world)]
    return torch.cat(pieces, dim=0)
