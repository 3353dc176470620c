"""NVFP4 block-scaled GEMM operator (tcgen05 / TMEM / TMA) with fused epilogues.

Same constructor and attributes as the reference wrapper ``ResidentNVFP4``
(``native_pi0/primitives.py:12-146``): operands are ``PackedNVFP4`` matrices packed offline, the
constructor uploads them, ``forward()`` launches on the current PyTorch stream and returns the reused
output tensor.
"""
import ctypes

import numpy as np
import torch

from native_pi0 import _native
from native_pi0.quantization import swizzle_scales
from native_pi0.storage import packed_tma_buffer


_OUTPUT_KINDS = {torch.float32: "f32", torch.bfloat16: "bf16", torch.uint8: "fp4"}
_ACTIVATION_CODES = {"none": 0, "gelu": 1, "geglu": 2, "relu2": 3}          # configure_resident_fp4_quantized
_RESOURCE_KEYS = ("registers_per_thread", "static_shared_bytes", "dynamic_shared_bytes", "local_bytes_per_thread",
                  "predicted_max_ctas_per_sm", "threads_per_cta", "max_threads_per_sm", "sm_count")


def _operand_geometry(name, packed):
    """(rows, K) of a ``PackedNVFP4`` operand after checking its arrays are what the kernel consumes."""
    data, scales = packed.data, packed.scales
    if data.dtype != np.uint8 or scales.dtype != np.uint8 or data.ndim != 2 or scales.ndim != 2 or data.size == 0:
        raise ValueError(f"{name}: packed E2M1 codes and E4M3 scale codes must be non-empty 2-D uint8 arrays")
    if int(scales.max(initial=0)) > 126:
        raise ValueError(f"{name}: scale codes above 126 are not finite unsigned E4M3 values")
    rows, k = data.shape[0], 2 * data.shape[1]
    if rows % 128 or k % 64:
        raise ValueError(f"{name}: rows must be padded to 128 and K to 64 (got {rows} x {k})")
    if scales.shape != (rows, k // 16):
        raise ValueError(f"{name}: expected one scale per 16 K-elements, shape {(rows, k // 16)}, got {scales.shape}")
    return rows, k


def _epilogue_kind(output_dtype, gelu, geglu, relu2, global_scale, bias, residual):
    """Validate the requested epilogue and return (output kind, activation name)."""
    kind = _OUTPUT_KINDS.get(output_dtype)
    if kind is None:
        raise ValueError("output_dtype must be torch.float32, torch.bfloat16 or torch.uint8 (packed NVFP4)")
    chosen = [name for name, on in (("gelu", gelu), ("geglu", geglu), ("relu2", relu2)) if on]
    if len(chosen) > 1:
        raise ValueError(f"At most one output activation can be fused, got {chosen}")
    activation = chosen[0] if chosen else "none"
    fused_add = bias is not None or residual is not None
    if not np.isfinite(global_scale) or global_scale <= 0:
        raise ValueError("output_global_scale must be a positive finite number")
    if kind == "f32" and fused_add:
        raise ValueError("The FP32 epilogue stores the raw product: bias and residual need a BF16 or NVFP4 output")
    if kind != "fp4" and (activation != "none" or global_scale != 1):
        raise ValueError("Activations and an output tensor scale belong to the NVFP4 (uint8) output")
    if activation == "geglu" and fused_add:
        raise ValueError("GeGLU halves the width over interleaved gate/up columns and takes neither bias nor residual")
    return kind, activation


def narrow_tile_scales(swizzled, rows, blocks):
    """Weight scales for 32-wide output tiles: from the standard swizzled layout (128-row x 4-block atoms, ``rows`` a
    multiple of 128, ``blocks`` 16-element blocks per row, a multiple of 4) to one atom per (32-row tile, group of four
    blocks) with the tile's rows in the first 32-row sub-column and zeros elsewhere (uint8 tensor, 4x the size)."""
    atoms, groups = rows // 128, blocks // 4
    standard = swizzled.view(atoms, groups, 32, 4, 4)                       # [atom, group, row % 32, row // 32 % 4, block % 4]
    narrow = torch.zeros((atoms * 4, groups, 32, 4, 4), dtype=torch.uint8, device=swizzled.device)
    narrow[:, :, :, 0, :] = standard.permute(0, 3, 1, 2, 4).reshape(atoms * 4, groups, 32, 4)
    return narrow.reshape(-1)


class ResidentNVFP4:
    def __init__(self, library, activation, weight, *, workers=16, device="cuda",
                 output_dtype=torch.float32, bias=None, residual=None,
                 output_global_scale=1.0, output_gelu=False, output_geglu=False, output_relu2=False,
                 block_n=128, rows=None, activation_buffers=None, tiled_weight=False):
        self._handle = ctypes.c_void_p()
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("ResidentNVFP4 runs on a CUDA device")
        self.device = device if device.index is not None else torch.device("cuda", torch.cuda.current_device())
        m, k = _operand_geometry("activation", activation)
        n, weight_k = _operand_geometry("weight", weight)
        if weight_k != k:
            raise ValueError(f"activation K ({k}) and weight K ({weight_k}) differ")
        self.output_global_scale = np.float32(output_global_scale)
        kind, act = _epilogue_kind(output_dtype, output_gelu, output_geglu, output_relu2, self.output_global_scale, bias, residual)
        self.activation_global_scale, self.weight_global_scale = np.float32(activation.global_scale), np.float32(weight.global_scale)
        self.output_width = n // 2 if act == "geglu" else n
        self._library = lib = _native.load(library)
        with torch.cuda.device(self.device):
            self._upload(activation, weight, activation_buffers, bias, residual, m, n)
            if block_n == 32:
                if k % 64:
                    raise ValueError("32-wide tiles need K to be a multiple of 64")
                self.sb = narrow_tile_scales(self.sb, n, k // 16)
            if kind == "fp4":
                self.output = packed_tma_buffer((m, self.output_width // 2), device=self.device)
                atoms = ((m + 127) // 128) * ((self.output_width // 16 + 3) // 4)
                self.output_scales = torch.zeros(atoms * 512, dtype=torch.uint8, device=self.device)
            else:
                self.output, self.output_scales = torch.zeros((m, n), dtype=output_dtype, device=self.device), None
            alpha = float(self.activation_global_scale * self.weight_global_scale)
            _native.check(lib.create_resident_fp4(ctypes.byref(self._handle), self.a.data_ptr(), self.b.data_ptr(), self.sa.data_ptr(),
                                                  self.sb.data_ptr(), self.output.data_ptr(), m, n, k, workers, alpha), "Native FP4 setup")
            try:
                if kind == "fp4":
                    _native.check(lib.configure_resident_fp4_quantized(
                        self._handle, _native.ptr(self.bias), _native.ptr(self.residual), self.output.data_ptr(),
                        self.output_scales.data_ptr(), float(self.output_global_scale), _ACTIVATION_CODES[act]),
                        "Native FP4 quantized-output setup")
                elif kind == "bf16":
                    _native.check(lib.configure_resident_fp4_bf16(self._handle, _native.ptr(self.bias), _native.ptr(self.residual),
                                                                  self.output.data_ptr()), "Native FP4 epilogue setup")
                if rows is not None:
                    _native.check(lib.configure_resident_fp4_rows(self._handle, int(rows)), "Native FP4 rows")
                if block_n != 128:
                    _native.check(lib.configure_resident_fp4_tile(self._handle, int(block_n)), "Native FP4 tile")
                if tiled_weight:
                    # re-lay the packed weight tile-major: block (n tile, 256-wide K stage) = block_n contiguous 128-byte rows
                    tiled = self.b.view(n // block_n, block_n, k // 256, 128).permute(0, 2, 1, 3).contiguous()
                    self.b.copy_(tiled.view(n, k // 2))
                    _native.check(lib.configure_resident_fp4_weight_layout(self._handle, 1), "Native FP4 weight layout")
                values = (ctypes.c_int * len(_RESOURCE_KEYS))()
                _native.check(lib.resident_fp4_resources(self._handle, values, len(values)), "Native FP4 resource query")
            except Exception:
                self.close()
                raise
        self.resources = dict(zip(_RESOURCE_KEYS, values))

    def _upload(self, activation, weight, activation_buffers, bias, residual, m, n):
        """Device copies of the operands: codes in TMA-safe storage, scales in the 128x4 atom order."""
        def codes(packed):
            buffer = packed_tma_buffer(packed.data.shape, device=self.device)
            buffer.copy_(torch.from_numpy(np.ascontiguousarray(packed.data)))
            return buffer

        def scales(packed):
            return torch.from_numpy(swizzle_scales(packed.scales)).to(self.device)

        self.b, self.sb = codes(weight), scales(weight)
        if activation_buffers is None:
            self.a, self.sa = codes(activation), scales(activation)
        else:
            # A operand produced on the device by an earlier stage (packed codes + swizzled scales)
            data, swizzled = activation_buffers
            atoms = ((m + 127) // 128) * ((activation.scales.shape[1] + 3) // 4) * 512
            if tuple(data.shape) != tuple(activation.data.shape) or data.dtype != torch.uint8 or swizzled.numel() != atoms:
                raise ValueError("Bound activation buffers must match the packed activation layout")
            self.a, self.sa = data, swizzled
        self.bias = self.residual = None
        if bias is not None:
            self.bias = torch.as_tensor(bias, dtype=torch.bfloat16, device=self.device).contiguous()
            if tuple(self.bias.shape) != (n,):
                raise ValueError(f"bias must have shape ({n},)")
        if residual is not None:
            self.residual = torch.as_tensor(residual, dtype=torch.bfloat16, device=self.device).contiguous()
            if tuple(self.residual.shape) != (m, n):
                raise ValueError(f"residual must have the padded output shape ({m}, {n})")

    @property
    def handle(self):
        return self._handle

    def forward(self):
        if not self._handle.value:
            raise RuntimeError("Native FP4 instance is closed")
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device)
            _native.check(self._library.launch_resident_fp4(self._handle, stream.cuda_stream), "Native FP4 launch")
        return self.output

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self._library, self._handle)

    def close(self):
        if self._handle.value:
            with torch.cuda.device(self.device):
                _native.check(self._library.destroy_resident_fp4(self._handle), "Native FP4 teardown")
            self._handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
