"""Helpers for the GPU parity tests: device buffers through the library's own
pool and a GEMM driver over the device-pointer entry points."""
import ctypes

import numpy as np


class DevGemm:
    def __init__(self, omcuda):
        from omcuda import dev
        self.m = omcuda
        self.dev = dev
        self.stream = omcuda.lib().omcudaGetStream()
        omcuda.check()

    def dtensor(self, a):
        return self.m.Tensor.from_numpy(np.asarray(a)).to_device()

    def prepare(self, B):
        K, N = B.shape
        nbytes, kp = self.dev.prepared_b_bytes(K, N)
        dB = self.dtensor(B)
        bt = self.m.Tensor.device_empty((N, kp), np.uint8)
        cs = self.m.Tensor.device_empty((N,), np.int32)
        pb = self.dev.prepare_b(dB.data_ptr, B.dtype == np.int8, K, N, bt.data_ptr,
                                cs.data_ptr, self.stream)
        return pb, (dB, bt, cs)

    def matmul_integer(self, A, B, a_zp=None, b_zp=None, choice=0):
        M, K = A.shape
        N = B.shape[1]
        pb, keep = self.prepare(B)
        dA = self.dtensor(A)
        Y = self.m.Tensor.device_empty((M, N), np.int32)
        g = self.dev.GemmArgs()
        g.M, g.N, g.K = M, N, K
        g.A, g.a_signed = dA.data_ptr, int(A.dtype == np.int8)
        g.B = pb
        if a_zp is not None:
            az = self.dtensor(np.asarray(a_zp, A.dtype).reshape(-1))
            g.a_zp, g.a_zp_len = az.data_ptr, az.shape[0]
        if b_zp is not None:
            bz = self.dtensor(np.asarray(b_zp, B.dtype).reshape(-1))
            g.b_zp, g.b_zp_len = bz.data_ptr, bz.shape[0]
            rs = self.m.Tensor.device_empty((M,), np.int32)
            self.dev.row_sum(dA.data_ptr, g.a_signed, M, K, rs.data_ptr, self.stream)
            g.a_rowsum = rs.data_ptr
        g.epilogue = self.dev.EPI_I32
        g.Y = Y.data_ptr
        g.kernel_choice = choice
        self.dev.gemm_i8(g, self.stream)
        out = Y.numpy()
        self.m.synchronize()
        return out
