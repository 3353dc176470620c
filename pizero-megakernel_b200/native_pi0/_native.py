"""Loader and ctypes signatures of ``libpi0_native.so`` (the C ABI declared in ``include/pi0_native.h``).

There is no CPU or PyTorch fallback: if the library has not been built, importing an operator fails with
instructions to build it.  ``build()`` compiles the CUDA sources in ``../csrc`` for sm_100a with nvcc.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
LIBRARY = HERE / "libpi0_native.so"
TRACE_LIBRARY = HERE / "libpi0_trace.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC"]


def build(force=False, verbose=False):
    """Compile the CUDA extension in-tree (cross-compiles without a GPU)."""
    nvcc = os.environ.get("NVCC", "nvcc")
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    newest = max(p.stat().st_mtime for p in sources)
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < newest:
        cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIBRARY), str(CSRC / "pi0_native.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.run(cmd, check=True)
    trace_src = CSRC / "launch_trace.cpp"
    if trace_src.exists() and (force or not TRACE_LIBRARY.exists() or TRACE_LIBRARY.stat().st_mtime < trace_src.stat().st_mtime):
        cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{cuda_home}/include",
                        "-o", str(TRACE_LIBRARY), str(trace_src), "-ldl"], check=True)
    return LIBRARY


class NativeSpec(C.Structure):
    """Stage record of ``create_native_model`` (``include/pi0_native.h``)."""
    _fields_ = [("kind", C.c_int), ("handle", C.c_void_p), ("sources", C.c_int * 4), ("modes", C.c_int * 4)]


_P, _I, _F = C.c_void_p, C.c_int, C.c_float
_SIGNATURES = {
    "create_resident_fp4": [C.POINTER(_P)] + [_P] * 5 + [_I] * 4 + [_F],
    "launch_resident_fp4": [_P, _P],
    "configure_resident_fp4_bf16": [_P] * 4,
    "configure_resident_fp4_quantized": [_P] * 5 + [_F, _I],
    "configure_resident_fp4_qkv_rope": [_P, _P, _I, _P, _P, _P, _P, _I, _I, _I],
    "configure_resident_fp4_stream": [_P] * 6 + [_F, _P],
    "configure_resident_fp4_row_rms": [_P, _P, _I, _I, _F],
    "configure_resident_fp4_stream_sums": [_P, _P, _I],
    "configure_resident_fp4_row_layernorm": [_P, _P, _P, _I, _I, _F, _P],
    "configure_resident_fp4_rows": [_P, _I],
    "configure_resident_fp4_tile": [_P, _I],
    "configure_resident_fp4_weight_layout": [_P, _I],
    "resident_fp4_resources": [_P, C.POINTER(_I), _I],
    "destroy_resident_fp4": [_P],
    "create_dense": [C.POINTER(_P)] + [_P] * 5 + [_I] * 6 + [_F],
    "launch_dense": [_P, _P],
    "destroy_dense": [_P],
    "configure_dense_round_before_residual": [_P],
    "configure_dense_geglu": [_P, _P],
    "configure_dense_gelu": [_P, _I],
    "configure_dense_rms_factor": [_P, _P],
    "configure_dense_skinny": [_P],
    "configure_dense_qkv_rope": [_P] * 5 + [_I] * 3,
    "configure_dense_head_pad": [_P, _I, _I, _I],
    "configure_dense_rows": [_P, _I],
    "configure_dense_tile": [_P, _I],
    "create_norm": [C.POINTER(_P)] + [_P] * 8 + [_I] * 9 + [_F] * 2,
    "launch_norm": [_P, _P],
    "destroy_norm": [_P],
    "configure_norm_quantize_only": [_P, _I],
    "configure_norm_bf16_copy": [_P, _P],
    "configure_norm_layout": [_P, _I, _I, _I],
    "create_attention": [C.POINTER(_P)] + [_P] * 12 + [_I] * 12 + [_F],
    "launch_attention": [_P, _P],
    "destroy_attention": [_P],
    "attention_resources": [C.POINTER(_I), _I],
    "configure_attention_splits": [_P, _I],
    "configure_attention_cache": [_P, _P, _P, _I, _I],
    "configure_attention_fused_merge": [_P, _I],
    "configure_attention_fp4_output": [_P, _P, _P, _I, _I, _F],
    "configure_attention_path": [_P, _I],
    "configure_attention_head_pad": [_P, _I],
    "attention_prepare_handle": [_P, C.POINTER(_P)],
    "attention_validate": [_P],
    "configure_attention_fp4_pitch": [_P, _I],
    "attention_merge_handle": [_P, C.POINTER(_P)],
    "attention_poison_partials": [_P, _P],
    "attention_split_diagnostics": [_P, _P, _I, C.POINTER(C.c_uint)],
    "create_patch_embed": [C.POINTER(_P)] + [_P] * 5 + [_I] * 3,
    "create_token_embed": [C.POINTER(_P), _P, _P, _P, _I, _I, _I, _I, _F, _I],
    "create_linear32": [C.POINTER(_P)] + [_P] * 5 + [_I] * 9 + [_F, _F, _I],
    "configure_linear32_extra_row": [_P, _P, _P],
    "create_suffix_assemble": [C.POINTER(_P), _P, _P, _P, _I, _I, _I],
    "launch_op": [_P, _P],
    "destroy_op": [_P],
    "op_geometry": [_P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)],
    "create_native_model": [C.POINTER(_P), _I, _P, _P, _I, _I],
    "launch_native_model": [_P] * 6,
    "launch_native_model_range": [_P] * 6 + [_I] * 3,
    "enable_native_model_timings": [_P, _I],
    "read_native_model_timings": [_P, _P, C.c_size_t],
    "read_native_model_status": [_P, C.POINTER(_I), _I],
    "read_native_model_counters": [_P, _P, _P, _I, C.POINTER(_I)],
    "native_model_kernel_variant": [_P, C.POINTER(_I)],
    "run_tcgen_probe": [_P, _P, _P, _I],
    "run_fp8_probe": [_P, _P, _P, _I, _F, _F],
    "run_k_probe": [_P, _P, _P, _I, _I, _I, _F, _F],
    "run_grid_probe": [_P, _P, _P] + [_I] * 6 + [_F, _F],
    "run_nvfp4_probe": [_P] * 5 + [_I, _F, _I],
    "run_nvfp4_grid_probe": [_P] * 5 + [_I] * 5 + [_F],
    "run_vm_probe": [_I, _I, _P],
    "enable_native_model_debug": [_P, _I],
    "read_native_model_debug": [_P, C.POINTER(_I), _I],
    "set_native_model_wait_budget": [_P, C.c_ulonglong],
    "destroy_native_model": [_P],
    "create_native_linear": [C.POINTER(_P), _I, _P, _P, _P, _I, _I],
    "launch_native_linear": [_P, _P],
    "read_native_linear": [_P, _P, _I, _P],
    "destroy_native_linear": [_P],
    "quantize_nvfp4": [_P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "attention_split_noalloc": [_P, _P, _P, _P] + [_I] * 10 + [_F, _P],
}
EXPORTS = tuple(_SIGNATURES)
_cache = {}

# libpi0_trace.so: (argument types, result type); these return CUptiResult, not cudaError_t
_TRACE_SIGNATURES = {
    "begin_launch_trace": ([C.POINTER(_P)], _I),
    "end_launch_trace": ([_P, C.POINTER(_I), C.c_char_p, _I], _I),
    "launch_trace_error": ([_I], C.c_char_p),
}


def load_trace(path=None):
    """The CUPTI launch counter, a library of its own so that the engine does not link CUPTI."""
    path = Path(path) if path is not None else TRACE_LIBRARY
    key = "trace:" + str(path)
    if key not in _cache:
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run native_pi0._native.build() first")
        lib = C.CDLL(str(path))
        for name, (argtypes, restype) in _TRACE_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        _cache[key] = lib
    return _cache[key]


def load(path=None):
    """Return the ctypes library with every entry point typed.  Raises if the extension is missing."""
    path = Path(path) if path is not None else LIBRARY
    key = str(path.resolve()) if path.exists() else str(path)
    if key in _cache:
        return _cache[key]
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build the CUDA extension first (python -c 'import __graft_entry__ as g; g.build()' "
            "or native_pi0._native.build()).  This engine has no CPU fallback.")
    lib = C.CDLL(str(path))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    _cache[key] = lib
    return lib


def check(code, what):
    if code:
        raise RuntimeError(f"{what} CUDA error {code}")


def ptr(t):
    return None if t is None else t.data_ptr()


def status(lib, handle):
    """Synchronise and return the device status record of a program or operator handle."""
    values = (C.c_int * 8)()
    check(lib.read_native_model_status(handle, values, 8), "status read")
    keys = ("code", "worker", "stage", "band", "observed", "expected", "aborted", "epoch")
    return dict(zip(keys, values))
