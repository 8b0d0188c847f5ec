"""Compiled models end to end on the GPU: built by the model builder, loaded by
the session loader (the ExecutionSession / PyRuntime interface), run through
run_main_graph(OMTensorList*), checked against the oracle; the command-line
runner's save / load / verify round trip."""
import os

import numpy as np
import pytest

from omcuda.synthetic import make_encoder

pytestmark = pytest.mark.gpu


def test_config1_model_is_bit_exact(gpu, orc, tmp_path):
    from omcuda import model_builder
    from omcuda.session import OMExecutionSession
    rng = np.random.default_rng(42)
    X = rng.normal(size=(128, 768)).astype(np.float32)
    W = rng.integers(-127, 128, (768, 768), dtype=np.int8)
    bias = rng.normal(0, 0.02, 768).astype(np.float32)
    so = model_builder.build_dyn_quant_linear_model(str(tmp_path), "config1", W,
                                                    np.float32(0.0157), bias)
    s = OMExecutionSession(so)
    want = orc.dyn_quant_linear(X, W, np.float32(0.0157), bias)["Y"]
    (y,) = s.run([X])                       # host tensors in, host tensors out
    assert y.tobytes() == want.tobytes()
    (yd,) = s.run([gpu.Tensor.from_numpy(X).to_device()])   # device in, device out
    assert isinstance(yd, gpu.Tensor) and yd.device
    assert yd.numpy().tobytes() == want.tobytes()
    # a 3-D input takes the broadcast-A path; a wrong K is refused with NULL
    X3 = rng.normal(size=(2, 5, 768)).astype(np.float32)
    (y3,) = s.run([X3])
    assert y3.tobytes() == orc.dyn_quant_linear(X3, W, np.float32(0.0157), bias)["Y"].tobytes()
    with pytest.raises(gpu.OmcudaError):
        s.run([np.zeros((4, 100), np.float32)])
    (y,) = s.run([X])                       # and the session still serves
    assert y.tobytes() == want.tobytes()
    s.close()


def test_config2_model_is_bit_exact(gpu, orc, tmp_path):
    from omcuda import model_builder
    from omcuda.session import OMExecutionSession
    rng = np.random.default_rng(43)
    A = rng.integers(0, 256, (2, 64, 1024), dtype=np.uint8)
    B = rng.integers(-127, 128, (1024, 512), dtype=np.int8)
    bs = rng.uniform(0.001, 0.01, 512).astype(np.float32)
    so = model_builder.build_qlinear_matmul_model(str(tmp_path), "config2", B, bs,
                                                  np.zeros(512, np.int8), 0.02, 128, 0.5, 128)
    s = OMExecutionSession(so)
    (y,) = s.run([A])
    want = orc.qlinear_matmul(A, 0.02, np.uint8(128), B, bs, np.zeros(512, np.int8), 0.5,
                              np.uint8(128))
    assert np.array_equal(y, want)
    s.close()


def test_encoder_model_equals_the_harness_and_chains_on_device(gpu, tmp_path):
    from omcuda import model_builder
    from omcuda.session import OMExecutionSession
    H, heads, F = 128, 2, 256
    layers = make_encoder(17, H, F, 2)
    so = model_builder.build_encoder_model(str(tmp_path), "encoder", H, heads, F, layers)
    s = OMExecutionSession(so)
    x = np.random.default_rng(18).normal(size=(3, 40, H)).astype(np.float32)
    enc = gpu.Encoder(H, heads, F, layers)
    want = enc.run(x)
    (y,) = s.run([x])
    assert np.array_equal(y, want)
    # two runs chained without leaving the device
    (d1,) = s.run([gpu.Tensor.from_numpy(x).to_device()])
    (d2,) = s.run([d1])
    assert np.array_equal(d2.numpy(), enc.run(want))
    enc.close()
    s.close()


def test_torch_tensors_pass_through_without_a_copy(gpu, orc, tmp_path):
    # Device buffers of another library (anything with __cuda_array_interface__:
    # a torch.Tensor on the GPU) go in as non-owning device OMTensors, and a
    # device result is visible to torch as a view of the same memory.
    import torch
    from omcuda import model_builder
    from omcuda.session import OMExecutionSession
    rng = np.random.default_rng(44)
    X = rng.normal(size=(64, 256)).astype(np.float32)
    W = rng.integers(-127, 128, (256, 320), dtype=np.int8)
    bias = rng.normal(0, 0.02, 320).astype(np.float32)
    so = model_builder.build_dyn_quant_linear_model(str(tmp_path), "torch_io", W,
                                                    np.float32(0.01), bias)
    s = OMExecutionSession(so)
    want = orc.dyn_quant_linear(X, W, np.float32(0.01), bias)["Y"]
    xt = torch.from_numpy(X).cuda()
    torch.cuda.synchronize()
    view = gpu.Tensor.from_cuda_array(xt)
    assert view.device and view.data_ptr == xt.data_ptr() and view.shape == (64, 256)
    (yd,) = s.run([xt])
    assert isinstance(yd, gpu.Tensor) and yd.device
    gpu.synchronize()
    yt = torch.as_tensor(yd, device="cuda")
    assert yt.data_ptr() == yd.data_ptr and tuple(yt.shape) == (64, 320)
    assert yt.cpu().numpy().tobytes() == want.tobytes()
    # the plain operator API takes them too
    xq, sc, zp = gpu.dynamic_quantize_linear(xt, device=True)
    gpu.synchronize()
    ref = orc.dynamic_quantize_linear(X)
    assert np.array_equal(torch.as_tensor(xq, device="cuda").cpu().numpy(), ref[0])
    with pytest.raises(ValueError):
        gpu.Tensor.from_cuda_array(xt.t())      # not contiguous
    del view
    s.close()


def test_command_line_runner_round_trip(gpu, tmp_path, capsys):
    from omcuda import model_builder, run_model
    rng = np.random.default_rng(44)
    W = rng.integers(-127, 128, (64, 48), dtype=np.int8)
    model_builder.build_dyn_quant_linear_model(str(tmp_path), "model", W, 0.01, None)
    ref = str(tmp_path / "ref")
    assert run_model.main(["--load-model", str(tmp_path), "--shape-info", "0:9x64",
                           "--print-signatures", "-w", "1", "-n", "3",
                           "--save-ref", ref]) == 0
    out = capsys.readouterr().out
    assert "1st warmup" in out and "3rd iteration" in out and "Statistics 1" in out
    assert os.path.exists(os.path.join(ref, "output_0.npy"))
    assert run_model.main(["--load-model", str(tmp_path), "--load-ref", ref, "--verify", "ref",
                           "--verify-every-value", "--rtol", "0", "--atol", "0",
                           "--device-resident"]) == 0
    assert "correct." in capsys.readouterr().out
    bad = np.load(os.path.join(ref, "output_0.npy"))
    bad[0, 0] += 1.0
    np.save(os.path.join(ref, "output_0.npy"), bad)
    with pytest.raises(SystemExit):
        run_model.main(["--load-model", str(tmp_path), "--load-ref", ref, "--verify", "ref",
                        "--verify-every-value", "--rtol", "0", "--atol", "0"])
