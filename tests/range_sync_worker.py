"""Child process of tests/test_gpu_global_quant.py: one rank of a batch-sharded
encoder run with global quantization ranges.  Ranks are separate processes on
the same GPU, in lockstep only through host-side gloo collectives (no kernel
waits on another process)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "onnx-mlir_b200"))


def main():
    rank, world, port, out_dir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    B, S, H, heads, F, nl = (int(v) for v in sys.argv[5:11])
    sync = sys.argv[11] == "global"
    import torch
    import torch.distributed as dist
    import omcuda
    from omcuda.sharding import make_range_sync, shard_rows
    from omcuda.synthetic import make_encoder
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = port
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(0)
        omcuda.init()
        layers = make_encoder(51, H, F, nl)
        x = np.random.default_rng(52).normal(size=(B, S, H)).astype(np.float32)
        first, rows = shard_rows(B, world, rank)
        enc = omcuda.Encoder(H, heads, F, layers)
        if sync:
            enc.set_range_sync(make_range_sync(via_host=True))
        y = enc.run(np.ascontiguousarray(x[first:first + rows]))
        np.save(os.path.join(out_dir, "y_%d.npy" % rank), y)
        enc.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
