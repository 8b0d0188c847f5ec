"""Global quantization ranges across ranks (omcudaEncoderSetRangeSync): a batch
sharded over two ranks, with every DynamicQuantizeLinear range all-reduced,
must equal the single-rank run on the whole batch bit for bit -- that is, the
reference's own result on the whole batch, which per-shard ranges cannot give.

The two ranks are child processes on one GPU that meet only in host-side gloo
collectives, so the test needs a single B200."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from omcuda.synthetic import make_encoder

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run_ranks(tmp_path, world, dims, mode):
    port = str(_free_port())
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "range_sync_worker.py"),
                               str(r), str(world), port, str(tmp_path)] +
                              [str(d) for d in dims] + [mode],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    return np.concatenate([np.load(os.path.join(str(tmp_path), "y_%d.npy" % r))
                           for r in range(world)], axis=0)


def test_sharded_run_with_global_ranges_equals_whole_batch(gpu, tmp_path):
    B, S, H, heads, F, nl = 6, 128, 128, 2, 256, 3
    layers = make_encoder(51, H, F, nl)
    x = np.random.default_rng(52).normal(size=(B, S, H)).astype(np.float32)
    enc = gpu.Encoder(H, heads, F, layers)
    whole = enc.run(x)
    enc.close()
    got = _run_ranks(tmp_path, 2, (B, S, H, heads, F, nl), "global")
    assert got.shape == whole.shape
    assert got.tobytes() == whole.tobytes()
    # and per-shard ranges (the default) do differ from the whole-batch run:
    # the mode is not a no-op on this data
    local = _run_ranks(tmp_path, 2, (B, S, H, heads, F, nl), "shard")
    assert local.tobytes() != whole.tobytes()
    assert np.abs(local - whole).max() < 0.1
