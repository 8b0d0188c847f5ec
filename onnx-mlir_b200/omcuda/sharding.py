"""Row (batch) sharding of the quantized path across the GPUs of one box.

Every output row of the path depends on one input row and the replicated
weights, so ranks take contiguous row ranges and never exchange data inside a
forward pass; the only collective is the final all-gather of output rows.
Per-tensor dynamic quantization then uses each rank's own min/max ("replica
mode"): a rank's result equals the reference's result on that rank's rows.
"""
import torch
import torch.distributed as dist


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
