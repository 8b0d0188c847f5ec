"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    python bench.py --impl reference ...      # CPU arm, same metric and config

One JSON line on stdout (rank 0).  Workloads (synthetic, seeded, with the
shapes and value distributions of the reference configurations):

  mmi_4096    DynamicQuantizeLinear -> MatMulInteger -> Cast/Mul dequant,
              X f32 [4096,4096] ~ N(0,1), W int8 [4096,4096] U{-127..127};
              metric int8 TOPS (2*M*N*K per step).
  qlinear_c2  QLinearMatMul A u8 [32,512,1024] x B i8 [1024,4096] -> u8,
              per-column b_scale; metric int8 TOPS.
  bert_base   dynamic-quantized encoder, 12 layers, hidden 768, 12 heads,
              FFN 3072, seq 128, batch 32; metric sequences/s.
  bert_large  24 layers, hidden 1024, 16 heads, FFN 4096, seq 512, batch 256;
              metric sequences/s.  With N > 1 the per-rank outputs are joined
              by one NCCL all-gather inside the step.
  mmi_sweep   the 15-shape MatMulInteger sweep (M x (K,N)), per-shape list in
              the JSON line; rows of the M >= 4096 members sharded with N > 1.

A step is one pass of the workload's graph over one batch.  `value` is timed
with inputs resident in HBM; `e2e` runs the same graph through the krnl.call
entry points with pinned host buffers, host<->device copies inside the timed
region (the encoder workloads use the pipelined Submit / Wait form of the
host-tensor call: every step still copies its input in and its output out,
and those copies overlap the runs of the neighbouring steps).  With N > 1
every rank runs the workload on its own batch (weights replicated, no
data-path collective): weak scaling, the default.  `--scaling strong` keeps the
configured batch fixed and splits it over the ranks instead; every N > 1 run of
an encoder workload also appends that measurement as a "strong" object (and,
for the default workload, the M >= 4096 members of the GEMM sweep sharded by
rows as "sweep_strong").  A default N = 1 run adds an "extra" object with the
other headline kernels: the 4096^3 and QLinearMatMul GEMMs (TOP/s) and
DynamicQuantizeLinear alone (GB/s).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "onnx-mlir_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

L2_FLUSH_BYTES = 256 << 20

# dram__bytes_read.sum + dram__bytes_write.sum of the int8 GEMM kernel, bytes per
# launch, from ncu captures of this script (encoders: mean over the four GEMM
# launches of a layer).  A capture describes the kernel as it was when it was
# taken: each entry names the tile shape it was taken with, and the figure is
# reported only while the library still launches that shape.  Outputs that are
# still in the 126 MB L2 when a kernel ends are not in these counts.
NCU_GEMM_DRAM_BYTES = {
    "bert_large": (1391.2e6, "256x256 tiles, cta_group::2, f32 / bf16-plane outputs"),
    "bert_base": (7.57e6, "256x256 tiles, cta_group::2"),
    "mmi_4096": (51.85e6, "256x256 tiles, cta_group::2"),
    "qlinear_c2": (37.66e6, "256x256 tiles, cta_group::2"),
}
GEMM_TILE_IN_USE = "256x256 tiles, cta_group::2"


def ncu_traffic(workload):
    ent = NCU_GEMM_DRAM_BYTES.get(workload)
    if ent is None or not ent[1].startswith(GEMM_TILE_IN_USE):
        return None, "no ncu capture of the kernel in its present form"
    return ent[0], ("ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the "
                    "int8 GEMM, captured with: " + ent[1])


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while running."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None,
                "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ---------------------------------------------------------------------------
# GPU workloads
# ---------------------------------------------------------------------------

class GpuEnv:
    def __init__(self, local_rank):
        import torch
        import omcuda
        from omcuda import dev
        self.torch, self.m, self.dev = torch, omcuda, dev
        torch.cuda.set_device(local_rank)
        os.environ.setdefault("OMCUDA_DEVICE", str(local_rank))
        omcuda.init()
        self.stream = torch.cuda.current_stream()
        omcuda.lib().omcudaSetStream(ctypes.c_void_p(self.stream.cuda_stream))
        self.device = torch.device("cuda", local_rank)
        self.flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8,
                                     device=self.device)

    def sptr(self):
        return ctypes.c_void_p(self.stream.cuda_stream)

    def flush_l2(self):
        self.flush_buf.zero_()

    def t(self, a):
        return self.torch.from_numpy(np.ascontiguousarray(a)).to(self.device)

    def pinned(self, a):
        t = self.torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
        return t


class LinearWorkload:
    """DQL -> int8 GEMM -> dequant (mmi_4096) or QLinearMatMul (qlinear_c2)."""
    metric, unit, dtype = "MatMulInteger int8 TOPS", "TOPS", "u8*s8->s32"

    def __init__(self, env, name, seed, shape=None, e2e=True):
        self.env, self.name = env, name
        torch, dev = env.torch, env.dev
        rng = np.random.default_rng(seed)
        if name == "mmi_4096" or shape is not None:
            self.M, self.K, self.N = shape if shape is not None else (4096, 4096, 4096)
            self.kind = "dynquant"
            self.Xh = rng.normal(size=(self.M, self.K)).astype(np.float32)
            self.Wh = rng.integers(-127, 128, (self.K, self.N), dtype=np.int8)
            self.w_scale = np.float32(0.02 * 4 / 127)
        elif name == "qlinear_c2":
            self.M, self.K, self.N = 32 * 512, 1024, 4096
            self.kind = "qlinear"
            self.Ah = rng.integers(0, 256, (32, 512, self.K), dtype=np.uint8)
            self.Wh = rng.integers(-127, 128, (self.K, self.N), dtype=np.int8)
            self.bs = rng.uniform(0.001, 0.01, self.N).astype(np.float32)
        else:
            raise ValueError(name)
        M, N, K = self.M, self.N, self.K
        self.ops = 2.0 * M * N * K
        self.units = self.ops  # metric unit: int8 operations
        # resident device state
        W = env.t(self.Wh)
        nbytes, kp = dev.prepared_b_bytes(K, N)
        self.bt = torch.empty(nbytes, dtype=torch.uint8, device=env.device)
        self.colsum = torch.empty(N, dtype=torch.int32, device=env.device)
        self.pb = dev.prepare_b(W.data_ptr(), True, K, N, self.bt.data_ptr(),
                                self.colsum.data_ptr(), env.sptr())
        g = dev.GemmArgs()
        g.M, g.N, g.K = M, N, K
        g.B = self.pb
        if self.kind == "dynquant":
            self.X = env.t(self.Xh)
            self.xq = torch.empty((M, K), dtype=torch.uint8, device=env.device)
            self.xs = torch.empty(1, dtype=torch.float32, device=env.device)
            self.xz = torch.empty(1, dtype=torch.uint8, device=env.device)
            self.ws = env.t(np.array([self.w_scale], np.float32))
            self.scr = torch.zeros(dev.dql_scratch_bytes(), dtype=torch.uint8,
                                   device=env.device)
            self.Y = torch.empty((M, N), dtype=torch.float32, device=env.device)
            g.A, g.a_signed = self.xq.data_ptr(), 0
            g.a_zp, g.a_zp_len = self.xz.data_ptr(), 1
            g.epilogue = dev.EPI_DEQUANT
            g.sa, g.sb, g.sb_len = self.xs.data_ptr(), self.ws.data_ptr(), 1
            self.h2d = M * K * 4
            self.d2h = M * N * 4
            # algorithmic bytes of the GEMM launch: A + B + f32 Y
            self.gemm_bytes = M * K + K * N + 4 * M * N
        else:
            self.A = env.t(self.Ah.reshape(M, K))
            self.az = env.t(np.array([128], np.uint8))
            self.bz = env.t(np.zeros(N, np.int8))
            self.S = torch.empty(N, dtype=torch.float32, device=env.device)
            a_s = env.t(np.array([0.02], np.float32))
            y_s = env.t(np.array([0.5], np.float32))
            dev.requant_scale(a_s.data_ptr(), env.t(self.bs).data_ptr(), N,
                              y_s.data_ptr(), self.S.data_ptr(), env.sptr())
            self.rs = torch.empty(M, dtype=torch.int32, device=env.device)
            self.Y = torch.empty((M, N), dtype=torch.uint8, device=env.device)
            g.A, g.a_signed = self.A.data_ptr(), 0
            g.a_zp, g.a_zp_len = self.az.data_ptr(), 1
            g.b_zp, g.b_zp_len = self.bz.data_ptr(), N
            g.a_rowsum = self.rs.data_ptr()
            g.epilogue = dev.EPI_REQUANT
            g.sb, g.sb_len = self.S.data_ptr(), N
            g.y_zp, g.y_signed = 128, 0
            self.h2d = M * K
            self.d2h = M * N
            self.gemm_bytes = M * K + K * N + M * N + 8 * N
        g.Y = self.Y.data_ptr()
        self.g = g
        self.launches_per_step = 3
        env.torch.cuda.synchronize()
        if not e2e:
            return
        # e2e: pinned host tensors wrapped as OMTensors
        m = env.m
        if self.kind == "dynquant":
            self.hX = env.pinned(self.Xh)
            self.hY = torch.empty((M, N), dtype=torch.float32).pin_memory()
            self.oX = m.Tensor.from_numpy(self.hX.numpy())
            self.oY = m.Tensor.from_numpy(self.hY.numpy())
            self.oW = m.Tensor.from_numpy(self.Wh)
            self.oWs = m.Tensor.from_numpy(np.array(self.w_scale, np.float32))
            m.lib().omcudaRegisterConstant(self.oW.handle)
        else:
            self.hA = env.pinned(self.Ah)
            self.hY = torch.empty((32, 512, N), dtype=torch.uint8).pin_memory()
            self.oA = m.Tensor.from_numpy(self.hA.numpy())
            self.oY = m.Tensor.from_numpy(self.hY.numpy())
            self.oW = m.Tensor.from_numpy(self.Wh)
            self.oS = [m.Tensor.from_numpy(np.asarray(v)) for v in (
                np.float32(0.02), np.uint8(128), self.bs, np.zeros(N, np.int8),
                np.float32(0.5), np.uint8(128))]
            m.lib().omcudaRegisterConstant(self.oW.handle)

    def step(self, gemm_events=None):
        env, dev = self.env, self.env.dev
        if self.kind == "dynquant":
            dev.dynamic_quantize_linear(self.X.data_ptr(), self.M * self.K,
                                        self.xq.data_ptr(), self.xs.data_ptr(),
                                        self.xz.data_ptr(), self.scr.data_ptr(),
                                        env.sptr())
        else:
            dev.row_sum(self.A.data_ptr(), 0, self.M, self.K, self.rs.data_ptr(),
                        env.sptr())
        if gemm_events:
            gemm_events[0].record(env.stream)
        dev.gemm_i8(self.g, env.sptr())
        if gemm_events:
            gemm_events[1].record(env.stream)

    def step_e2e(self):
        L = self.env.m.lib()
        if self.kind == "dynquant":
            L.omcudaDynQuantLinear(self.oY.handle, self.oX.handle, self.oW.handle,
                                   self.oWs.handle, None, None, 0)
        else:
            s = self.oS
            L.omcudaQLinearMatMul(self.oY.handle, self.oA.handle, s[0].handle,
                                  s[1].handle, self.oW.handle, s[2].handle,
                                  s[3].handle, s[4].handle, s[5].handle)
        self.env.m.check()

    def config(self):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K,
                "l2": "flushed between timed iterations (256 MiB write)",
                "graph": ("DynamicQuantizeLinear->MatMulInteger->Cast/Mul"
                          if self.kind == "dynquant" else "QLinearMatMul")}


class EncoderWorkload:
    """BERT-shaped dynamic-quantized encoder through the model harness."""
    SHAPES = {
        "bert_base": dict(layers=12, H=768, heads=12, F=3072, S=128, B=32),
        "bert_large": dict(layers=24, H=1024, heads=16, F=4096, S=512, B=256),
    }
    metric, unit, dtype = "quantized BERT seq/s", "seq/s", "u8*s8->s32 + f32"

    def __init__(self, env, name, seed, world, dist):
        from omcuda.synthetic import make_encoder
        self.env, self.name, self.world, self.dist = env, name, world, dist
        c = self.SHAPES[name]
        self.c = c
        torch = env.torch
        self.layers = make_encoder(42, c["H"], c["F"], c["layers"])  # replicated
        self.enc = env.m.Encoder(c["H"], c["heads"], c["F"], self.layers)
        rng = np.random.default_rng(seed)
        shape = (c["B"], c["S"], c["H"])
        self.hX = torch.from_numpy(rng.normal(size=shape).astype(np.float32)).pin_memory()
        self.X = self.hX.to(env.device)
        self.Y = torch.empty(shape, dtype=torch.float32, device=env.device)
        self.Yall = (torch.empty((world * c["B"],) + shape[1:], dtype=torch.float32,
                                 device=env.device) if world > 1 else None)
        self.Y2 = torch.empty_like(self.Y) if world > 1 else None
        self.nstep, self.pending = 0, None
        self.overlap_gather = os.environ.get("OMCUDA_BENCH_OVERLAP_GATHER", "1") != "0"
        self.oX = env.m.Tensor.from_numpy(self.hX.numpy())
        self.hY = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.oY = env.m.Tensor.from_numpy(self.hY.numpy())
        # a second pair of pinned host tensors for the pipelined e2e loop
        self.hX2 = self.hX.clone().pin_memory()
        self.oX2 = env.m.Tensor.from_numpy(self.hX2.numpy())
        self.hY2 = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.oY2 = env.m.Tensor.from_numpy(self.hY2.numpy())
        self.units = float(c["B"])
        T = c["B"] * c["S"]
        self.h2d = T * c["H"] * 4
        self.d2h = T * c["H"] * 4
        self.launches_per_step = None
        # Algorithmic bytes of the four int8 GEMM launches of a layer (A + B +
        # output; the QKV projection writes two bf16 planes = 4 bytes per
        # element, the others f32), averaged per launch.
        H, F = c["H"], c["F"]
        shapes = [(3 * H, H), (H, H), (F, H), (H, F)]      # (N, K)
        self.gemm_bytes = sum(T * K + K * N + 4 * T * N for N, K in shapes) / 4.0
        env.torch.cuda.synchronize()

    def step(self, _ev=None):
        c = self.c
        if self.world == 1:
            self.enc.run_dev(self.X.data_ptr(), c["B"], c["S"], self.Y.data_ptr(),
                             self.env.sptr())
            return
        # N > 1: the all-gather of this step's output rows runs on NCCL's
        # stream while the next step computes (two output buffers); a step
        # waits for the gather of the step before it, finish() for the last.
        from omcuda.sharding import gather_rows
        y = self.Y if self.nstep % 2 == 0 else self.Y2
        self.nstep += 1
        self.enc.run_dev(self.X.data_ptr(), c["B"], c["S"], y.data_ptr(), self.env.sptr())
        if not self.overlap_gather:
            gather_rows(y, self.world * c["B"], out=self.Yall)
            return
        self.finish()
        _, self.pending = gather_rows(y, self.world * c["B"], out=self.Yall, async_op=True)

    def finish(self):
        """Joins the all-gather still in flight into the launching stream."""
        if self.pending is not None:
            self.pending.wait()
            self.pending = None

    def step_e2e(self):
        # pinned host in, pinned host out, both copies inside the call
        self.enc.run_into(self.oX, self.oY)
        self.last = float(self.hY[0, 0, 0])
        if self.world > 1:
            from omcuda.sharding import gather_rows
            gather_rows(self.Y, self.world * self.c["B"], out=self.Yall)

    def run_e2e(self, steps, before_each=None):
        """`steps` calls of the pipelined host-tensor API back to back: every
        call copies its input from pinned host memory and its output back,
        and the copies of one call overlap the run of its neighbours.  All
        outputs are in host memory when this returns."""
        for i in range(steps):
            if before_each is not None:
                before_each()
            x, y = (self.oX, self.oY) if i % 2 == 0 else (self.oX2, self.oY2)
            self.enc.submit(x, y)
            if self.world > 1:
                from omcuda.sharding import gather_rows
                gather_rows(self.Y, self.world * self.c["B"], out=self.Yall)
        self.enc.wait()
        self.last = float(self.hY[0, 0, 0]) + float(self.hY2[0, 0, 0])

    def config(self):
        c = self.c
        return {"workload": self.name, "layers": c["layers"], "hidden": c["H"],
                "heads": c["heads"], "ffn": c["F"], "seq_len": c["S"],
                "batch_per_gpu": c["B"],
                "parallelism": "batch sharded, weights replicated, one "
                               "all-gather of outputs per step (queued behind the "
                               "step, joined before the next step ends)" if self.world > 1
                               else "single GPU",
                "l2": "flushed between timed iterations (256 MiB write)",
                "quantization": "per-shard dynamic (each rank quantizes its own batch)"}


def run_gpu(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    env = GpuEnv(local_rank)
    is_encoder = args.workload in EncoderWorkload.SHAPES
    if is_encoder and args.scaling == "strong" and world > 1:
        return run_strong_only(args, env, world, rank, dist)
    if is_encoder:
        if args.batch:
            EncoderWorkload.SHAPES[args.workload] = dict(
                EncoderWorkload.SHAPES[args.workload], B=args.batch)
        wl = EncoderWorkload(env, args.workload, 42 + rank, world, dist)
    elif args.shape:
        M, K, N = (int(v) for v in args.shape.lower().split("x"))
        wl = LinearWorkload(env, "mmi_%dx%dx%d" % (M, K, N), 42 + rank, shape=(M, K, N))
    else:
        wl = LinearWorkload(env, args.workload, seed=42 + rank)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, extra=None):
        for _ in range(warmup):
            env.flush_l2()
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True),
                torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i in range(steps):
            env.flush_l2()
            evs[i][0].record(env.stream)
            fn() if extra is None else fn(extra[i])
            evs[i][1].record(env.stream)
        # work a step left in flight (the last all-gather) belongs to the timed region
        tail = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        tail[0].record(env.stream)
        if hasattr(wl, "finish"):
            wl.finish()
        tail[1].record(env.stream)
        barrier()
        ms = sum(a.elapsed_time(b) for a, b in evs) + tail[0].elapsed_time(tail[1])
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=env.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    gemm_evs = [(torch.cuda.Event(enable_timing=True),
                 torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    # warm-up outside the launch count and the GEMM statistics
    for _ in range(args.warmup):
        env.flush_l2()
        wl.step()
    if hasattr(wl, "finish"):
        wl.finish()
    barrier()
    launches0 = env.m.launch_count()
    if is_encoder:
        wl.enc.set_profiling(True)
    if rank == 0:
        sampler.start()
    ms = timed(lambda ev=None: wl.step(ev), args.steps, 0, extra=gemm_evs)
    clocks = sampler.stop() if rank == 0 else None
    launches = env.m.launch_count() - launches0
    if is_encoder:
        gemm_ms_total, gemm_ops_total, gemm_n = wl.enc.gemm_stats()
        wl.enc.set_profiling(False)
        gemm_ms = gemm_ms_total / max(gemm_n, 1)
        achieved = gemm_ops_total / (gemm_ms_total * 1e-3) / 1e12
        roof_extra = {"launches_timed": gemm_n, "avg_launch_ms": gemm_ms,
                      "share_of_step": gemm_ms_total / ms}
        algo_bytes = wl.gemm_bytes
    else:
        gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_evs) / args.steps
        achieved = wl.ops / (gemm_ms * 1e-3) / 1e12
        roof_extra = {"avg_launch_ms": gemm_ms}
        algo_bytes = wl.gemm_bytes
    env.m.synchronize()

    # (the pipelined encoder call pays one unoverlapped copy-in and copy-out per
    # timed block: ten steps keep that at a few per cent of the block)
    e2e_steps = max(1, min(args.steps, 10))
    if is_encoder:
        # The host-tensor API as a pipeline (Submit / Wait): one timed block
        # over all steps, bracketed by events on the launching stream; the
        # closing event is recorded after the host has seen every output.
        wl.run_e2e(2, env.flush_l2)
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record(env.stream)
        wl.run_e2e(e2e_steps, env.flush_l2)
        b1.record(env.stream)
        barrier()
        e2e_ms = b0.elapsed_time(b1)
        if world > 1:
            t = torch.tensor([e2e_ms], dtype=torch.float64, device=env.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
    else:
        e2e_ms = timed(wl.step_e2e, e2e_steps, 1)

    # Fixed-batch (strong-scaling) measurement of the same graph, and of the
    # large members of the GEMM sweep, whenever there is more than one rank.
    strong = sweep_strong = None
    if world > 1 and is_encoder:
        strong = strong_scaling_leg(env, wl, world, rank, dist, barrier)
        if args.workload == "bert_large":
            sweep_strong = sweep_strong_leg(env, world, rank, dist, barrier)
    extra = None
    if world == 1 and args.workload == "bert_large" and not args.no_extra:
        extra = extra_kernels(env, peaks)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    scale = 1e12 if wl.unit == "TOPS" else 1.0
    value = wl.units * world * args.steps / (ms * 1e-3) / scale
    e2e_value = wl.units * world * e2e_steps / (e2e_ms * 1e-3) / scale
    int8_peak = 2.0 * peaks["bf16_tflops"]
    int8_sustained = 2.0 * (peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"])
    traffic, traffic_source = ncu_traffic(args.workload)
    roofline = {
        "kernel": "gemm_i8_tc2_kernel (gemm_i8_tc_kernel where a shape has too few 256x256 tiles)", "bound": "tensor",
        "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
        "frac": achieved / int8_peak,
        # the same launches against the other two denominators a reader may
        # want, and against the HBM roof
        "frac_sustained": achieved / int8_sustained,
        "frac_nominal": achieved / 4500.0,
        "hbm_frac": algo_bytes / (gemm_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "peak_source": "frac: 2 x %s TFLOP/s bf16 cuBLAS burst (%s; an int8 figure is not "
                       "in MEASURED_PEAKS.json); frac_sustained: 2 x %s (the seconds-long "
                       "loop under the power cap, the fitting one for launches timed inside "
                       "a long step); frac_nominal: 4500 TOP/s dense int8; hbm_frac: "
                       "algorithmic bytes / launch time / %s GB/s"
                       % (peaks["bf16_tflops"], peaks["source"],
                          peaks["bf16_tflops_sustained"], peaks["hbm_gbs"]),
        "algorithmic_bytes": algo_bytes,
        "traffic": traffic, "traffic_source": traffic_source}
    roofline.update(roof_extra)
    out = {
        "metric": wl.metric, "value": value, "unit": wl.unit,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic", "config": wl.config(),
        "e2e": {"value": e2e_value, "unit": wl.unit,
                "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "steps": e2e_steps,
                "api": ("omcudaEncoderSubmit / omcudaEncoderWait, all steps in "
                        "one timed block" if is_encoder else
                        "one krnl.call-style entry per step")},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
    }
    if strong is not None:
        out["strong"] = strong
    if sweep_strong is not None:
        out["sweep_strong"] = sweep_strong
    if extra is not None:
        out["extra"] = extra
    # CPU baseline on a bounded sample of the same workload (rank 0, N=1 only).
    if world == 1 and not args.no_cpu_baseline and not args.shape and not args.batch:
        out["cpu_baseline"] = cpu_baseline(args.workload, wl, long_sample=True)
    emit(out)
    if world > 1:
        dist.destroy_process_group()



def _max_over_ranks(env, dist, world, vals):
    if world == 1:
        return [float(v) for v in vals]
    t = env.torch.tensor(list(vals), dtype=env.torch.float64, device=env.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def strong_scaling_leg(env, wl, world, rank, dist, barrier, steps=5, warmup=2):
    """The encoder at its configured batch split over the ranks (shard_rows),
    one all-gather of the output rows inside every step: the fixed-batch form
    of the multi-GPU configuration.  Also times the same batch on one GPU
    without a gather (every rank runs it at once; max over ranks), so that the
    speed-up is measured inside one run."""
    import torch
    from omcuda.sharding import gather_rows, shard_rows
    c = wl.c
    B = c["B"]
    first, b_local = shard_rows(B, world, rank)
    x = wl.X[:b_local]
    y_local = torch.empty((b_local, c["S"], c["H"]), dtype=torch.float32, device=env.device)
    y_all = wl.Y  # [B, S, H]: the gathered output
    ev = lambda: torch.cuda.Event(enable_timing=True)
    l0 = env.m.launch_count()
    rows = []
    for i in range(warmup + steps):
        env.flush_l2()
        e = (ev(), ev(), ev())
        e[0].record(env.stream)
        wl.enc.run_dev(x.data_ptr(), b_local, c["S"], y_local.data_ptr(), env.sptr())
        e[1].record(env.stream)
        gather_rows(y_local, B, out=y_all)
        e[2].record(env.stream)
        if i >= warmup:
            rows.append(e)
        if i == warmup - 1:
            barrier()
    barrier()
    launches = (env.m.launch_count() - l0) // (warmup + steps)
    step_ms = sum(a.elapsed_time(c_) for a, _, c_ in rows) / steps
    run_ms = sum(a.elapsed_time(b) for a, b, _ in rows) / steps
    gather_ms = sum(b.elapsed_time(c_) for _, b, c_ in rows) / steps
    # The same with every DynamicQuantizeLinear range all-reduced over the
    # ranks (global quantization: the sharded run then equals the whole-batch
    # run bit for bit); 4 * layers + 1 two-word NCCL all-reduces per step.
    from omcuda.sharding import make_range_sync
    wl.enc.set_range_sync(make_range_sync())
    gq = []
    for i in range(warmup + steps):
        env.flush_l2()
        a, b = ev(), ev()
        a.record(env.stream)
        wl.enc.run_dev(x.data_ptr(), b_local, c["S"], y_local.data_ptr(), env.sptr())
        gather_rows(y_local, B, out=y_all)
        b.record(env.stream)
        if i >= warmup:
            gq.append((a, b))
        if i == warmup - 1:
            barrier()
    barrier()
    wl.enc.set_range_sync(None)
    gq_ms = sum(a.elapsed_time(b) for a, b in gq) / steps
    # the whole batch on one GPU, no gather
    one = []
    for i in range(1 + 3):
        env.flush_l2()
        a, b = ev(), ev()
        a.record(env.stream)
        wl.enc.run_dev(wl.X.data_ptr(), B, c["S"], wl.Y.data_ptr(), env.sptr())
        b.record(env.stream)
        if i >= 1:
            one.append((a, b))
    barrier()
    one_ms = sum(a.elapsed_time(b) for a, b in one) / len(one)
    step_ms, run_ms, gather_ms, one_ms, gq_ms = _max_over_ranks(
        env, dist, world, [step_ms, run_ms, gather_ms, one_ms, gq_ms])
    return {"scaling": "strong", "global_batch": B, "batch_per_gpu": b_local,
            "steps": steps, "warmup": warmup,
            "value": B / (step_ms * 1e-3), "unit": "seq/s", "ms_per_step": step_ms,
            "encoder_ms": run_ms, "all_gather_ms": gather_ms,
            "all_gather_bytes_received_per_gpu": (B - b_local) * c["S"] * c["H"] * 4,
            "one_gpu_ms_per_step": one_ms, "one_gpu_value": B / (one_ms * 1e-3),
            "speedup_over_one_gpu": one_ms / step_ms,
            "efficiency": one_ms / step_ms / world,
            "gpu_launches_per_step": int(launches),
            "quantization": "per-shard ranges (a rank's result equals the reference's on "
                            "its rows)",
            "global_quant": {"ms_per_step": gq_ms, "value": B / (gq_ms * 1e-3),
                             "speedup_over_one_gpu": one_ms / gq_ms,
                             "range_all_reduces_per_step": 4 * c["layers"] + 1,
                             "quantization": "ranges all-reduced over the ranks (the "
                                             "sharded result equals the whole-batch result "
                                             "bit for bit)"},
            "timing": "CUDA events on the launching stream, max over ranks; the "
                      "gather is synchronous (the step ends when the rows have arrived)"}


def sweep_strong_leg(env, world, rank, dist, barrier, steps=3, warmup=3):
    """Members of the GEMM sweep with M >= 4096, rows split over the ranks:
    DynamicQuantizeLinear -> MatMulInteger -> dequant on M / world rows."""
    import torch
    rows = []
    for K, N in SWEEP_KN:
        for M in (4096, 16384):
            m_rank = M // world
            wl = LinearWorkload(env, "mmi_%dx%dx%d" % (M, K, N), 42 + rank,
                                shape=(m_rank, K, N), e2e=False)
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                   for _ in range(steps)]
            for _ in range(warmup):
                env.flush_l2()
                wl.step()
            barrier()
            for a, b in evs:
                env.flush_l2()
                a.record(env.stream)
                wl.step()
                b.record(env.stream)
            barrier()
            ms = sum(a.elapsed_time(b) for a, b in evs) / steps
            (ms,) = _max_over_ranks(env, dist, world, [ms])
            rows.append({"M": M, "K": K, "N": N, "rows_per_gpu": m_rank, "ms_per_step": ms,
                         "tops": 2.0 * M * N * K / ms / 1e9})
            del wl
            torch.cuda.empty_cache()
    return rows


def run_strong_only(args, env, world, rank, dist):
    """`--scaling strong`: the JSON line's value is the fixed-batch figure."""
    import torch

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()
    wl = EncoderWorkload(env, args.workload, 42 + rank, world, dist)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    launches0 = env.m.launch_count()
    st = strong_scaling_leg(env, wl, world, rank, dist, barrier, steps=args.steps,
                            warmup=args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        cfg = wl.config()
        cfg.pop("batch_per_gpu")
        cfg["parallelism"] = ("configured batch split over the GPUs, weights replicated, "
                              "one all-gather of the output rows inside every step")
        cfg.update({"global_batch": st["global_batch"], "batch_per_gpu": st["batch_per_gpu"]})
        emit({"metric": wl.metric, "value": st["value"], "unit": wl.unit, "n_gpus": world,
              "steps": args.steps, "warmup": args.warmup, "ms_per_step": st["ms_per_step"],
              "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
              "dtype": wl.dtype, "data": "synthetic", "config": cfg,
              "gpu_launches": int(env.m.launch_count() - launches0), "clocks": clocks,
              "strong": st})
    dist.destroy_process_group()


def extra_kernels(env, peaks):
    """The other headline kernels, a fraction of a second each: the 4096^3
    MatMulInteger GEMM (L2 flushed and warm), the QLinearMatMul GEMM of the
    batched configuration, and DynamicQuantizeLinear alone on 64 Mi and 512 Mi
    elements (two launches: range reduction, quantize)."""
    import torch
    dev = env.dev
    int8_peak = 2.0 * peaks["bf16_tflops"]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    out = {"timing": "CUDA events around the launch(es) on the launching stream, "
                     "mean of 10 after 3 warm-ups"}

    def time_gemm(wl, flush):
        ts = []
        for i in range(13):
            wl.step()                       # refreshes xq / rowsum; not timed
            if flush:
                env.flush_l2()
            a, b = ev(), ev()
            a.record(env.stream)
            dev.gemm_i8(wl.g, env.sptr())
            b.record(env.stream)
            if i >= 3:
                ts.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in ts) / len(ts)

    for name in ("mmi_4096", "qlinear_c2"):
        wl = LinearWorkload(env, name, 42, e2e=False)
        d = {}
        for flush in (True, False):
            ms = time_gemm(wl, flush)
            tops = wl.ops / ms / 1e9
            d["l2_flushed" if flush else "l2_warm"] = {
                "gemm_ms": ms, "tops": tops, "frac_of_2x_bf16_burst": tops / int8_peak,
                "frac_nominal": tops / 4500.0}
        d["M"], d["N"], d["K"] = wl.M, wl.N, wl.K
        out[name] = d
        del wl
        torch.cuda.empty_cache()
    dql = {}
    for n in (64 << 20, 512 << 20):
        x = torch.randn(n, dtype=torch.float32, device=env.device)
        y = torch.empty(n, dtype=torch.uint8, device=env.device)
        sc = torch.empty(1, dtype=torch.float32, device=env.device)
        zp = torch.empty(1, dtype=torch.uint8, device=env.device)
        scr = torch.zeros(dev.dql_scratch_bytes(), dtype=torch.uint8, device=env.device)
        ts = []
        for i in range(13):
            env.flush_l2()
            a, b = ev(), ev()
            a.record(env.stream)
            dev.dynamic_quantize_linear(x.data_ptr(), n, y.data_ptr(), sc.data_ptr(),
                                        zp.data_ptr(), scr.data_ptr(), env.sptr())
            b.record(env.stream)
            if i >= 3:
                ts.append((a, b))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in ts) / len(ts)
        dql["%d_Mi_elements" % (n >> 20)] = {
            "ms": ms, "gbs_at_5_bytes_per_element": 5.0 * n / ms / 1e6,
            "gbs_at_9_bytes_per_element": 9.0 * n / ms / 1e6,
            "hbm_frac_5": 5.0 * n / ms / 1e6 / peaks["hbm_gbs"],
            "hbm_frac_9": 9.0 * n / ms / 1e6 / peaks["hbm_gbs"]}
        del x, y
        torch.cuda.empty_cache()
    dql["note"] = ("5 B/element = read f32 once + write u8; a tensor larger than L2 has "
                   "to be read twice (range, then quantize): 9 B/element is what the two "
                   "launches move")
    out["dynamic_quantize_linear"] = dql
    # A store-only stream for scale: the library fill of 1 GiB.  The f32 tails
    # of the K = 1024 GEMMs are store streams (2.1 GB written per launch
    # against 0.14 GB read), and a store stream does not reach the copy figure,
    # which is half reads.
    buf = torch.empty(1 << 30, dtype=torch.uint8, device=env.device)
    ts = []
    for i in range(7):
        a, b = ev(), ev()
        a.record(env.stream)
        buf.zero_()
        b.record(env.stream)
        if i >= 2:
            ts.append((a, b))
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in ts) / len(ts)
    out["hbm_fill"] = {"bytes": 1 << 30, "ms": ms, "gbs": (1 << 30) / ms / 1e6,
                       "frac_of_copy": (1 << 30) / ms / 1e6 / peaks["hbm_gbs"],
                       "kernel": "torch zero_ (library fill), not a kernel of this package"}
    del buf
    torch.cuda.empty_cache()
    return out


SWEEP_M = (1, 16, 256, 4096, 16384)
SWEEP_KN = ((4096, 4096), (4096, 14336), (14336, 4096))


def run_sweep(args):
    """The GEMM sweep of the reference configurations: DQL -> MatMulInteger ->
    dequant at M in {1,16,256,4096,16384} x (K,N) in {(4096,4096),
    (4096,14336), (14336,4096)}; with N GPUs the rows of the M >= 4096 members
    are sharded (each rank runs M / N rows), the others run replicated.  One
    JSON line: aggregate TOPS (sum of ops / sum of times) and a per-shape list.
    Small M is bound by the read of the K*N int8 weights, so each shape also
    reports the bytes/s of that read."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    env = GpuEnv(local_rank)
    peaks = load_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = env.m.launch_count()
    rows, tot_ops, tot_ms, tot_e2e_ops, tot_e2e_ms = [], 0.0, 0.0, 0.0, 0.0
    for K, N in SWEEP_KN:
        for M in SWEEP_M:
            m_rank = M // world if (M >= 4096 and world > 1) else M
            wl = LinearWorkload(env, "mmi_%dx%dx%d" % (M, K, N), 42 + rank,
                                shape=(m_rank, K, N))
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
                    torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                   for _ in range(args.steps)]
            for _ in range(args.warmup):
                env.flush_l2()
                wl.step()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            for e in evs:
                env.flush_l2()
                e[0].record(env.stream)
                wl.step((e[1], e[2]))
                e[3].record(env.stream)
            torch.cuda.synchronize()
            ms = sum(e[0].elapsed_time(e[3]) for e in evs) / args.steps
            gemm_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
            e2e_n = 2
            wl.step_e2e()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(e2e_n):
                wl.step_e2e()
            env.m.synchronize()
            e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_n
            if world > 1:
                t = torch.tensor([ms, gemm_ms, e2e_ms], dtype=torch.float64, device=env.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms, gemm_ms, e2e_ms = (float(v) for v in t.tolist())
            mult = world if m_rank != M else 1     # sharded members: all ranks' rows
            ops = wl.ops * mult
            rows.append({"M": M, "K": K, "N": N, "rows_per_gpu": m_rank,
                         "ms_per_step": ms, "tops": ops / ms / 1e9,
                         "gemm_ms": gemm_ms, "gemm_tops": ops / gemm_ms / 1e9,
                         "gemm_frac_of_int8_peak": wl.ops / gemm_ms / 1e9 / int8_peak,
                         "weight_read_gbs": K * N / gemm_ms / 1e6,
                         "e2e_ms": e2e_ms, "e2e_tops": ops / e2e_ms / 1e9})
            tot_ops += ops
            tot_ms += ms
            tot_e2e_ops += ops
            tot_e2e_ms += e2e_ms
            del wl
            env.m.lib().omcudaForgetConstants()   # the weights' host buffer is gone
            torch.cuda.empty_cache()
    clocks = sampler.stop() if rank == 0 else None
    launches = env.m.launch_count() - launches0
    if rank == 0:
        big = [r for r in rows if r["M"] >= 4096]
        emit({
            "metric": LinearWorkload.metric, "value": tot_ops / tot_ms / 1e9, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": tot_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": LinearWorkload.dtype, "data": "synthetic",
            "config": {"workload": "mmi_sweep", "shapes": len(rows),
                       "l2": "flushed between timed iterations (256 MiB write)",
                       "graph": "DynamicQuantizeLinear->MatMulInteger->Cast/Mul",
                       "sharding": "rows of the M >= 4096 members split over the GPUs"},
            "e2e": {"value": tot_e2e_ops / tot_e2e_ms / 1e9, "unit": "TOPS",
                    "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "steps": 2},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"kernel": "gemm_i8_tc2_kernel (gemm_i8_tc_kernel where a shape has too few 256x256 tiles)", "bound": "tensor",
                         "achieved": sum(r["gemm_tops"] * r["gemm_ms"] for r in big) /
                                     sum(r["gemm_ms"] for r in big) / world,
                         "peak": int8_peak, "unit": "TOP/s",
                         "frac": sum(r["gemm_tops"] * r["gemm_ms"] for r in big) /
                                 sum(r["gemm_ms"] for r in big) / world / int8_peak,
                         "peak_source": "2 x bf16 cuBLAS burst (%s); members with M >= 4096, "
                                        "per GPU" % peaks["source"],
                         "traffic": None},
            "sweep": rows})
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(workload, wl=None, reps=1, long_sample=False):
    """Times the oracle's reference-shaped CPU code on a bounded sample: about
    a second of CPU work per repetition for the reference arm's steps, ten to
    twenty seconds in all for the baseline of the default run (long_sample)."""
    import oracle_lib
    orc = oracle_lib.Oracle(os.path.join(ROOT, "oracle", "_build", "liboracle.so"))
    # All host cores this process may run on (torchrun exports OMP_NUM_THREADS=1).
    orc.L.orc_set_threads(len(os.sched_getaffinity(0)))
    threads = orc.L.orc_max_threads()
    if workload in EncoderWorkload.SHAPES:
        c = EncoderWorkload.SHAPES[workload]
        if wl is not None:
            layer = wl.layers[0]
        else:
            from omcuda.synthetic import make_encoder
            layer = make_encoder(42, c["H"], c["F"], 1)[0]
        bs = 2 if workload == "bert_large" else 8
        if long_sample:
            bs, reps = (32, 1) if workload == "bert_large" else (c["B"], 6)
        x = np.random.default_rng(0).normal(size=(bs * c["S"], c["H"])).astype(np.float32)
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.encoder_layer(x, bs, c["S"], c["H"], c["heads"], c["F"], layer)
        dt = (time.perf_counter() - t0) / reps
        return {"value": bs / (dt * c["layers"]), "unit": "seq/s", "cores": threads,
                "kind": "port", "seconds_per_rep": dt, "sequences_timed": bs,
                "sample": "one of %d layers on %d of %d sequences (%d x %.1f s), "
                          "scaled by the layer count; oracle ops with OpenMP"
                          % (c["layers"], bs, c["B"], reps, dt)}
    shapes = {"mmi_4096": (4096, 4096, 4096), "qlinear_c2": (16384, 4096, 1024)}
    M, N, K = shapes[workload]
    rng = np.random.default_rng(0)
    rows = 256
    if long_sample:
        rows, reps = M, (2 if workload == "mmi_4096" else 3)
    A = rng.integers(0, 256, (rows, K), dtype=np.uint8)
    W = wl.Wh if wl is not None else rng.integers(-127, 128, (K, N), dtype=np.int8)
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.ref_shaped_matmul_integer(A, W, 128, threads)
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * rows * N * K / dt / 1e12, "unit": "TOPS",
            "cores": threads, "kind": "port", "seconds_per_rep": dt, "rows_timed": rows,
            "sample": "%d of %d rows of the same [K=%d,N=%d] GEMM, reference-shaped "
                      "lowering (operands widened to i32, 4x8x8 register tile, "
                      "OpenMP over rows), %d x %.2f s" % (rows, M, K, N, reps, dt)}


def run_reference(args):
    """CPU arm: the oracle's port of the reference's lowering on all host
    threads, same metric and config, each step a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_baseline(args.workload)
    cb = cpu_baseline(args.workload, reps=args.steps)
    is_encoder = args.workload in EncoderWorkload.SHAPES
    if is_encoder:
        c = EncoderWorkload.SHAPES[args.workload]
        config = {"workload": args.workload, "layers": c["layers"], "hidden": c["H"],
                  "heads": c["heads"], "ffn": c["F"], "seq_len": c["S"],
                  "batch_per_gpu": c["B"],
                  # what a step of this arm really times
                  "layers_timed": 1, "sequences_timed": cb["sequences_timed"],
                  "extrapolated": True}
        metric, dtype = EncoderWorkload.metric, EncoderWorkload.dtype
    else:
        M, N, K = {"mmi_4096": (4096, 4096, 4096),
                   "qlinear_c2": (16384, 4096, 1024)}[args.workload]
        config = {"workload": args.workload, "M": M, "N": N, "K": K,
                  "rows_timed": cb["rows_timed"], "extrapolated": cb["rows_timed"] != M}
        metric, dtype = LinearWorkload.metric, LinearWorkload.dtype
    dt = cb.pop("seconds_per_rep")
    emit({
        "impl": "reference", "metric": metric, "value": cb["value"],
        "unit": cb["unit"], "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic", "config": config,
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": cb["unit"], "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0}})


_JSON_OUT = None


def _claim_stdout():
    """Keeps stdout for the one JSON line: everything else a library prints
    there (NCCL's version banner, for one) goes to stderr instead."""
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(obj):
    _JSON_OUT.write(json.dumps(obj) + "\n")
    _JSON_OUT.flush()


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="omcuda", choices=["omcuda", "reference"])
    ap.add_argument("--workload", default="bert_large",
                    choices=["mmi_4096", "qlinear_c2", "bert_base", "bert_large",
                             "mmi_sweep"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the extra kernels of the default N = 1 run")
    ap.add_argument("--shape", type=str, default=None, metavar="MxKxN",
                    help="with --workload mmi_4096: another member of the GEMM sweep, "
                         "e.g. 1x4096x14336 (small cases for profiling)")
    ap.add_argument("--batch", type=int, default=None,
                    help="encoder workloads: a smaller batch than the configured one "
                         "(small cases for profiling; the JSON line names it)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1, encoder workloads: weak = every rank runs the configured "
                         "batch (default); strong = the configured batch is split")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "omcuda" else args.warmup
    if args.workload == "mmi_sweep":
        if args.impl == "reference":
            args.workload = "mmi_4096"   # the CPU arm times the sweep's 4096^3 member
            run_reference(args)
        else:
            run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
