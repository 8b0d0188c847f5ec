"""The allocation-free DynamicQuantizeLinear entry point.

Some users of this library run where device memory cannot be allocated on
demand -- every byte of HBM was claimed by the hosting server's own arena, or
the allocator's device-wide synchronisation is not acceptable in their loop.
For them the library carries its reduction scratch inside its own image.  This
test calls that entry point through the C ABI twice in a row (the second call
sees the first one's leftovers in the shared scratch) and requires the very
same bytes the ordinary entry point produces, plus a refusal of inputs beyond
the stated limit.  It lives in a file collected last so that a run that stops
at the first failure has already exercised everything else.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(gpu, fn_noalloc, fn_plain, x, scratch, stream):
    d = gpu.Tensor.from_numpy(x).to_device()
    outs = []
    for which in ("noalloc", "plain"):
        y = gpu.Tensor.device_empty(x.shape, np.uint8)
        s = gpu.Tensor.device_empty((), np.float32)
        z = gpu.Tensor.device_empty((), np.uint8)
        if which == "noalloc":
            rc = fn_noalloc(d.data_ptr, x.size, y.data_ptr, s.data_ptr, z.data_ptr, stream)
        else:
            rc = fn_plain(d.data_ptr, x.size, y.data_ptr, s.data_ptr, z.data_ptr,
                          scratch.data_ptr, stream)
        assert rc == 0, gpu.lib().omcudaGetLastErrorString()
        outs.append((y.numpy(), s.numpy(), z.numpy()))
    gpu.synchronize()
    return outs


def test_no_alloc_entry_matches_the_ordinary_one_twice(gpu):
    L = gpu.lib()
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    fn_noalloc = L.omcudaDevDynamicQuantizeLinearNoAlloc
    fn_noalloc.argtypes = [vp, i64, vp, vp, vp, vp]
    fn_plain = L.omcudaDevDynamicQuantizeLinear
    fn_plain.argtypes = [vp, i64, vp, vp, vp, vp, vp]
    L.omcudaDevDqlScratchBytes.restype = i64
    L.omcudaDevDqlScratchBytes.argtypes = [i64]
    stream = L.omcudaGetStream()
    scratch = gpu.Tensor.from_numpy(
        np.zeros(L.omcudaDevDqlScratchBytes(0), np.uint8)).to_device()
    rng = np.random.default_rng(2024)
    # first call: many blocks; second call: fewer blocks and a different range,
    # so stale partial results from the first call are in the shared scratch
    for shape, sigma in (((1024, 1537), 3.0), ((37, 129), 0.25)):
        x = rng.normal(0, sigma, size=shape).astype(np.float32)
        (y1, s1, z1), (y2, s2, z2) = _run(gpu, fn_noalloc, fn_plain, x, scratch, stream)
        assert s1.tobytes() == s2.tobytes()
        assert int(z1) == int(z2)
        assert np.array_equal(y1, y2)


def test_no_alloc_entry_rejects_oversized_input(gpu):
    L = gpu.lib()
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    fn = L.omcudaDevDynamicQuantizeLinearNoAlloc
    fn.argtypes = [vp, i64, vp, vp, vp, vp]
    x = gpu.Tensor.device_empty((16,), np.float32)
    y = gpu.Tensor.device_empty((16,), np.uint8)
    s = gpu.Tensor.device_empty((), np.float32)
    z = gpu.Tensor.device_empty((), np.uint8)
    L.omcudaClearError()
    rc = fn(x.data_ptr, (1 << 31) + 1, y.data_ptr, s.data_ptr, z.data_ptr,
            L.omcudaGetStream())
    assert rc == gpu.EINVAL
    assert b"exceed the limit" in L.omcudaGetLastErrorString()
    L.omcudaClearError()
