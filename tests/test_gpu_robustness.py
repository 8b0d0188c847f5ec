"""GPU tests of the library's error and threading contracts: the bounded
device-side wait (a wait that gives up and returns -- nothing traps, faults or
spins without a limit) and several host threads inside the library at once."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_service_resumes(gpu, orc):
    from omcuda import dev
    L = gpu.lib()
    st = L.omcudaGetStream()
    waited = gpu.Tensor.from_numpy(np.zeros(1, np.int64)).to_device()
    dev.set_wait_limit_ns(1_000_000)  # 1 ms
    try:
        # One CTA allocates tensor memory and waits, through the same mbar_wait
        # the GEMM and attention kernels use, on a barrier nothing ever signals.
        dev.selftest_bounded_wait(waited.data_ptr, st)
        with pytest.raises(gpu.OmcudaError) as ei:
            gpu.synchronize()
        assert ei.value.code == gpu.ETIMEDOUT
        ns = int(waited.numpy()[0])
        assert 1_000_000 <= ns < 200_000_000, ns
        # The status is sticky: until it is cleared every entry point returns
        # without doing work.
        dev.selftest_bounded_wait(None, st)
        L.omcudaSynchronize()
        assert L.omcudaGetLastError() == gpu.ETIMEDOUT
        y = np.full((4, 4), 7, np.int32)
        a = np.ones((4, 16), np.uint8)
        b = np.ones((16, 4), np.int8)
        ty, ta, tb = (gpu.Tensor.from_numpy(v) for v in (y, a, b))
        L.omcudaMatMulInteger(ty.handle, ta.handle, tb.handle, None, None)
        assert (y == 7).all()
        L.omcudaClearError()
        assert L.omcudaGetLastError() == gpu.OK
    finally:
        dev.set_wait_limit_ns(0)
        L.omcudaClearError()
    # Service resumes: the kernel released its tensor memory and the status
    # word is clear, so the tensor-core GEMM runs and is bit-exact again.
    rng = np.random.default_rng(1)
    A = rng.integers(0, 256, (256, 512), dtype=np.uint8)
    B = rng.integers(-127, 128, (512, 384), dtype=np.int8)
    az = np.array(3, np.uint8)
    assert np.array_equal(gpu.matmul_integer(A, B, az, None),
                          orc.matmul_integer_2d(A, B, az.reshape(1), None))
    gpu.synchronize()


def test_concurrent_host_threads(gpu, orc):
    # Three host threads in the library at once -- two with a stream of their
    # own (omcudaSetStream), one on the shared library stream -- all using the
    # same registered constant weight (one prepared copy, cached) and the same
    # temporary sizes (pool blocks change hands between streams).  Every result
    # must equal the oracle's bit for bit.
    L = gpu.lib()
    rng = np.random.default_rng(2)
    K, N = 256, 384
    W = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bias = rng.normal(0, 0.1, N).astype(np.float32)
    w_scale = np.float32(0.011)
    tW = gpu.Tensor.from_numpy(W)
    L.omcudaRegisterConstant(tW.handle)
    iters = 12
    xs = [[rng.normal(0, 1 + t, size=(64 + 32 * (i % 3), K)).astype(np.float32)
           for i in range(iters)] for t in range(3)]
    want = [[orc.dyn_quant_linear(x, W, w_scale, bias)["Y"] for x in row] for row in xs]
    errors = []
    barrier = threading.Barrier(3)

    def worker(t):
        stream = None
        try:
            if t < 2:
                stream = L.omcudaStreamCreate()
                assert stream
                L.omcudaSetStream(stream)
            barrier.wait()
            for i, x in enumerate(xs[t]):
                if i % 2:
                    got = gpu.dyn_quant_linear(x, tW, w_scale, None, bias, 0)
                else:  # device-resident: the call returns with the work queued
                    dx = gpu.Tensor.from_numpy(x).to_device()
                    got = gpu.dyn_quant_linear(dx, tW, w_scale, None, bias, 0,
                                               device=True).numpy()
                if got.tobytes() != want[t][i].tobytes():
                    errors.append((t, i, float(np.abs(got - want[t][i]).max())))
            gpu.synchronize()
        except Exception as exc:  # noqa: BLE001 - reported by the main thread
            errors.append((t, repr(exc)))
        finally:
            if stream:
                L.omcudaSetStream(None)
                L.omcudaStreamDestroy(stream)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(3)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    L.omcudaForgetConstants()
    assert not errors, errors[:5]
