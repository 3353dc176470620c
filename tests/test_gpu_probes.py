"""The self-contained host-pointer probes (``run_*_probe``) with the checks of the reference's validation scripts
(``scripts/validate_tcgen.py:28-83``, ``validate_nvfp4.py:35-72``, ``validate_vm.py:26-36``), on a smaller set of cases."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0 import _native
from native_pi0.quantization import pack_nvfp4, swizzle_scales


def test_dense_probes_bf16_and_fp8():
    lib = _native.load()
    torch.manual_seed(17)
    for repetitions in (1, 17):
        a, b = torch.randn(128, 64).bfloat16(), torch.randn(128, 64).bfloat16()
        out = np.empty((repetitions, 128, 128), np.float32)
        assert lib.run_tcgen_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, repetitions) == 0
        for result in out:
            np.testing.assert_allclose(result, (a.float() @ b.float().T).numpy(), atol=3e-5, rtol=2e-5)
        a8, b8 = (torch.randn(128, 64) * 4).to(torch.float8_e4m3fn), (torch.randn(128, 64) * 4).to(torch.float8_e4m3fn)
        alpha = np.float32(.0123) * np.float32(.0456)
        assert lib.run_fp8_probe(a8.data_ptr(), b8.data_ptr(), out.ctypes.data, repetitions, .0123, .0456) == 0
        for result in out:
            np.testing.assert_allclose(result, (a8.float() @ b8.float().T).numpy() * alpha, atol=1e-4 * float(alpha), rtol=2e-5)
    for precision, dtype in enumerate((torch.bfloat16, torch.float8_e4m3fn)):
        alpha = np.float32(.0123) * np.float32(.0456)
        for k in (192, 1024):
            a, b = torch.randn(128, k).to(dtype), torch.randn(128, k).to(dtype)
            out = np.empty((3, 128, 128), np.float32)
            assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 3, k, precision, .0123, .0456) == 0
            for result in out:
                np.testing.assert_allclose(result, (a.float() @ b.float().T).numpy() * alpha, atol=1e-4 * float(alpha), rtol=3e-5)
        for m, n, k, workers in ((256, 384, 192, 4), (51, 2560, 1024, 16)):
            pm = (m + 127) // 128 * 128
            a = torch.zeros(pm, k, dtype=dtype)
            a[:m] = torch.randn(m, k).to(dtype)
            b = torch.randn(n, k).to(dtype)
            out = np.empty((2, pm, n), np.float32)
            assert lib.run_grid_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 2, pm, n, k, workers, precision, .0123, .0456) == 0
            for result in out:
                np.testing.assert_allclose(result, (a.float() @ b.float().T).numpy() * alpha, atol=1e-4 * float(alpha), rtol=3e-5)
    assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 1, 100, 0, 1., 1.) == 1        # K must be a multiple of 64
    assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 1, 128, 2, 1., 1.) == 1        # precision 0 or 1


def test_nvfp4_probes():
    lib = _native.load()
    rng = np.random.default_rng(11)
    for reps, case, k in ((1, "random", 64), (17, "zero", 64), (17, "varied", 64), (5, "random", 1024)):
        x, y = rng.normal(size=(128, k)), rng.normal(size=(128, k))
        if case == "zero":
            x[:] = 0
        if case == "varied":
            x *= np.exp2(np.arange(128)[:, None] % 12 - 6)
            y *= np.tile([.01, .1, 1, 10], (128, 16)).reshape(128, 64)
            x[::3, :16] = 0
        a, b = pack_nvfp4(x, global_scale=.125), pack_nvfp4(y, global_scale=.25, scale_policy="ceil")
        sa, sb = swizzle_scales(a.scales), swizzle_scales(b.scales)
        out = np.empty((reps, 128, 128), np.float32)
        alpha = float(np.float32(a.global_scale * b.global_scale))
        assert lib.run_nvfp4_probe(a.data.ctypes.data, b.data.ctypes.data, sa.ctypes.data, sb.ctypes.data, out.ctypes.data, reps, alpha, k) == 0
        expected = a.dequantize() @ b.dequantize().T
        tolerance = 1e-5 * max(1, float(np.abs(expected).max()))
        for result in out:
            np.testing.assert_allclose(result, expected, atol=tolerance, rtol=3e-5)
    for m, n, k, workers in ((256, 384, 192, 4), (51, 2560, 1024, 16)):
        a = pack_nvfp4(rng.normal(size=(m, k)), global_scale=.125, row_alignment=128)
        b = pack_nvfp4(rng.normal(size=(n, k)), global_scale=.25, scale_policy="ceil")
        sa, sb = swizzle_scales(a.scales), swizzle_scales(b.scales)
        pm = a.data.shape[0]
        out = np.empty((3, pm, n), np.float32)
        assert lib.run_nvfp4_grid_probe(a.data.ctypes.data, b.data.ctypes.data, sa.ctypes.data, sb.ctypes.data, out.ctypes.data, 3, pm, n, k,
                                        workers, float(np.float32(a.global_scale * b.global_scale))) == 0
        expected = a.dequantize() @ b.dequantize().T
        tolerance = 1e-5 * max(1, float(np.abs(expected).max()))
        for result in out:
            np.testing.assert_allclose(result[:m], expected[:m], atol=tolerance, rtol=3e-5)
            np.testing.assert_array_equal(result[m:], 0)


def test_vm_probe_lifecycle():
    lib = _native.load()
    for workers, instructions in ((1, 1), (1, 257), (16, 17), (148, 65)):
        for _ in range(2):
            out = np.zeros((workers, instructions, 16), dtype=np.int32)
            assert lib.run_vm_probe(workers, instructions, out.ctypes.data) == 0
            assert np.all(out > 0) and np.all(out == out[:, :1, :1])
    assert lib.run_vm_probe(0, 1, out.ctypes.data) == 1
    assert lib.run_vm_probe(1000, 1, out.ctypes.data) != 0
