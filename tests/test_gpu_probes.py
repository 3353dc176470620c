"""The self-contained host-pointer probes (``run_*_probe``).

They are exports of the one library here (the reference builds a separate library per probe and checks it from
``scripts/validate_tcgen.py``, ``validate_nvfp4.py`` and ``validate_vm.py``); the cases below follow those scripts'
shapes, scale factors and tolerances: every repetition of a launch must reproduce ``alpha * a @ b.T`` of the operands as
the tensor core reads them, padding rows must come back as zeros, and the VM probe must show all warps in every
instruction with one tensor-memory allocation per CTA.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0 import _native
from native_pi0.quantization import pack_nvfp4, swizzle_scales

DESCALE = (0.0123, 0.0456)
ALPHA = float(np.float32(DESCALE[0]) * np.float32(DESCALE[1]))
DENSE_TYPES = {0: torch.bfloat16, 1: torch.float8_e4m3fn}


def dense_operands(m, n, k, precision, rows=None, seed=17):
    g = torch.Generator().manual_seed(seed + m + n + k)
    kind = DENSE_TYPES[precision]
    a = torch.zeros(m, k, dtype=kind)
    a[:rows or m] = torch.randn(rows or m, k, generator=g).to(kind)
    b = torch.randn(n, k, generator=g).to(kind)
    return a, b, (a.float() @ b.float().T).numpy()


def check_slabs(out, want, atol, rtol):
    for slab in out:
        np.testing.assert_allclose(slab, want, atol=atol, rtol=rtol)


@pytest.mark.parametrize("repetitions", [1, 17])
def test_single_tile_probes(repetitions):
    lib = _native.load()
    out = np.empty((repetitions, 128, 128), np.float32)
    a, b, want = dense_operands(128, 128, 64, 0)
    assert lib.run_tcgen_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, repetitions) == 0
    check_slabs(out, want, 3e-5, 2e-5)
    a, b, want = dense_operands(128, 128, 64, 1)
    assert lib.run_fp8_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, repetitions, *DESCALE) == 0
    check_slabs(out, want * ALPHA, 1e-4 * ALPHA, 2e-5)


@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("k", [192, 1024])
def test_k_loop_probe(precision, k):
    lib = _native.load()
    a, b, want = dense_operands(128, 128, k, precision)
    out = np.empty((3, 128, 128), np.float32)
    assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 3, k, precision, *DESCALE) == 0
    check_slabs(out, want * ALPHA, 1e-4 * ALPHA, 3e-5)


@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("rows,n,k,workers", [(256, 384, 192, 4), (51, 2560, 1024, 16)])
def test_grid_probe(precision, rows, n, k, workers):
    lib = _native.load()
    m = (rows + 127) // 128 * 128
    a, b, want = dense_operands(m, n, k, precision, rows=rows)
    out = np.empty((2, m, n), np.float32)
    assert lib.run_grid_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 2, m, n, k, workers, precision, *DESCALE) == 0
    check_slabs(out, want * ALPHA, 1e-4 * ALPHA, 3e-5)
    assert not out[:, rows:].any()


def test_dense_probe_argument_errors():
    lib = _native.load()
    a, b, _ = dense_operands(128, 128, 128, 0)
    out = np.empty((1, 128, 128), np.float32)
    assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 1, 100, 0, 1., 1.) == 1      # K: a multiple of 64
    assert lib.run_k_probe(a.data_ptr(), b.data_ptr(), out.ctypes.data, 1, 128, 2, 1., 1.) == 1      # precision: 0 or 1
    assert lib.run_tcgen_probe(None, b.data_ptr(), out.ctypes.data, 1) == 1


def nvfp4_operands(rows, n, k, case, rng):
    x, y = rng.normal(size=(rows, k)), rng.normal(size=(n, k))
    if case == "zero":
        x[:] = 0
    if case == "varied":                                     # wide dynamic range across rows and blocks, some empty blocks
        x *= np.exp2(np.arange(rows)[:, None] % 12 - 6)
        y *= np.tile([.01, .1, 1, 10], (n, k // 4))
        x[::3, :16] = 0
    a = pack_nvfp4(x, global_scale=.125, row_alignment=128)
    b = pack_nvfp4(y, global_scale=.25, scale_policy="ceil")
    return a, b, a.dequantize() @ b.dequantize().T


@pytest.mark.parametrize("repetitions,case,k", [(1, "random", 64), (17, "zero", 64), (17, "varied", 64), (5, "random", 1024)])
def test_nvfp4_single_tile_probe(repetitions, case, k):
    lib = _native.load()
    a, b, want = nvfp4_operands(128, 128, k, case, np.random.default_rng(11))
    sa, sb = swizzle_scales(a.scales), swizzle_scales(b.scales)
    out = np.empty((repetitions, 128, 128), np.float32)
    alpha = float(np.float32(a.global_scale * b.global_scale))
    assert lib.run_nvfp4_probe(a.data.ctypes.data, b.data.ctypes.data, sa.ctypes.data, sb.ctypes.data, out.ctypes.data, repetitions,
                               alpha, k) == 0
    check_slabs(out, want, 1e-5 * max(1, float(np.abs(want).max())), 3e-5)


@pytest.mark.parametrize("rows,n,k,workers", [(256, 384, 192, 4), (51, 2560, 1024, 16)])
def test_nvfp4_grid_probe(rows, n, k, workers):
    lib = _native.load()
    a, b, want = nvfp4_operands(rows, n, k, "random", np.random.default_rng(12))
    sa, sb = swizzle_scales(a.scales), swizzle_scales(b.scales)
    m = a.data.shape[0]
    out = np.empty((3, m, n), np.float32)
    assert lib.run_nvfp4_grid_probe(a.data.ctypes.data, b.data.ctypes.data, sa.ctypes.data, sb.ctypes.data, out.ctypes.data, 3, m, n, k,
                                    workers, float(np.float32(a.global_scale * b.global_scale))) == 0
    check_slabs(out[:, :rows], want[:rows], 1e-5 * max(1, float(np.abs(want).max())), 3e-5)
    assert not out[:, rows:].any()


@pytest.mark.parametrize("workers,instructions", [(1, 1), (1, 257), (16, 17), (148, 65)])
def test_vm_probe_lifecycle(workers, instructions):
    lib = _native.load()
    for _ in range(2):                                       # a second launch: nothing of the first one is left behind
        slots = np.zeros((workers, instructions, 16), dtype=np.int32)
        assert lib.run_vm_probe(workers, instructions, slots.ctypes.data) == 0
        assert (slots > 0).all()
        assert (slots == slots[:, :1, :1]).all()             # one allocation per CTA, seen by every warp in every instruction
    assert lib.run_vm_probe(0, 1, slots.ctypes.data) == 1
    assert lib.run_vm_probe(10000, 1, slots.ctypes.data) != 0
