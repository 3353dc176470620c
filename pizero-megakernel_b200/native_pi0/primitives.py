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


class ResidentNVFP4:
    def __init__(self, library, activation, weight, *, workers=16, device="cuda",
                 output_dtype=torch.float32, bias=None, residual=None,
                 output_global_scale=1.0, output_gelu=False, output_geglu=False, output_relu2=False,
                 block_n=128, rows=None, activation_buffers=None, tiled_weight=False):
        self._handle = ctypes.c_void_p()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("CUDA device required")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        for operand in (activation, weight):
            if (operand.data.dtype != np.uint8 or operand.data.ndim != 2 or 0 in operand.data.shape
                    or operand.scales.dtype != np.uint8 or operand.scales.ndim != 2
                    or np.any(operand.scales > 126)):
                raise ValueError("Expected packed uint8 E2M1 data and finite unsigned E4M3 scales")
        m, half_k = activation.data.shape
        n, weight_half_k = weight.data.shape
        k = 2 * half_k
        if weight_half_k != half_k or m % 128 or n % 128 or k % 64:
            raise ValueError("Packed M/N must be multiples of 128 and K a multiple of 64")
        if activation.scales.shape != (m, k // 16) or weight.scales.shape != (n, k // 16):
            raise ValueError("Scale dimensions do not match operands")
        if output_dtype not in (torch.float32, torch.bfloat16, torch.uint8):
            raise ValueError("Output must be FP32, BF16, or packed FP4 (uint8)")
        if output_dtype == torch.float32 and (bias is not None or residual is not None):
            raise ValueError("Bias/residual fusion requires BF16 or FP4 output")
        self.output_global_scale = np.float32(output_global_scale)
        self.activation_global_scale = np.float32(activation.global_scale)
        self.weight_global_scale = np.float32(weight.global_scale)
        if not np.isfinite(self.output_global_scale) or self.output_global_scale <= 0:
            raise ValueError("Output global scale must be finite and positive")
        if sum(map(bool, (output_gelu, output_geglu, output_relu2))) > 1:
            raise ValueError("Select only one output activation")
        if output_geglu and (output_gelu or bias is not None or residual is not None):
            raise ValueError("Compact GeGLU requires interleaved gate/up weights without bias/residual")
        if output_dtype != torch.uint8 and (output_gelu or output_geglu or output_relu2 or self.output_global_scale != 1):
            raise ValueError("Output activation/global scaling requires packed FP4 output")
        self._library = _native.load(library)
        alpha = np.float32(activation.global_scale * weight.global_scale)
        with torch.cuda.device(self.device):
            self.a, self.b = [packed_tma_buffer(x.shape, device=self.device).copy_(torch.from_numpy(np.ascontiguousarray(x)))
                              for x in (activation.data, weight.data)]
            self.sa, self.sb = [torch.from_numpy(swizzle_scales(x)).to(self.device)
                                for x in (activation.scales, weight.scales)]
            if activation_buffers is not None:
                # A operand produced on the device by an earlier stage (packed codes + swizzled scales)
                data, scales = activation_buffers
                if tuple(data.shape) != tuple(self.a.shape) or data.dtype != torch.uint8 or scales.numel() != self.sa.numel():
                    raise ValueError("Bound activation buffers must match the packed activation layout")
                self.a, self.sa = data, scales
            self.bias = None if bias is None else torch.as_tensor(bias, dtype=torch.bfloat16, device=self.device).contiguous()
            self.residual = None if residual is None else torch.as_tensor(residual, dtype=torch.bfloat16, device=self.device).contiguous()
            if self.bias is not None and tuple(self.bias.shape) != (n,):
                raise ValueError("Bias must have shape (N,)")
            if self.residual is not None and tuple(self.residual.shape) != (m, n):
                raise ValueError("Residual must have padded shape (M,N)")
            self.output_width = n // 2 if output_geglu else n
            if output_dtype == torch.uint8:
                self.output = packed_tma_buffer((m, self.output_width // 2), device=self.device)
                self.output_scales = torch.zeros(((m + 127) // 128) * ((self.output_width // 16 + 3) // 4) * 512,
                                                 dtype=torch.uint8, device=self.device)
            else:
                self.output = torch.zeros((m, n), dtype=output_dtype, device=self.device)
                self.output_scales = None
            lib = self._library
            _native.check(lib.create_resident_fp4(ctypes.byref(self._handle), self.a.data_ptr(), self.b.data_ptr(),
                                                  self.sa.data_ptr(), self.sb.data_ptr(), self.output.data_ptr(),
                                                  m, n, k, workers, float(alpha)), "Native FP4 setup")
            try:
                if output_dtype == torch.uint8:
                    activation_code = 3 if output_relu2 else 2 if output_geglu else int(bool(output_gelu))
                    _native.check(lib.configure_resident_fp4_quantized(
                        self._handle, _native.ptr(self.bias), _native.ptr(self.residual), self.output.data_ptr(),
                        self.output_scales.data_ptr(), float(self.output_global_scale), activation_code),
                        "Native FP4 quantized-output setup")
                elif output_dtype == torch.bfloat16:
                    _native.check(lib.configure_resident_fp4_bf16(
                        self._handle, _native.ptr(self.bias), _native.ptr(self.residual), self.output.data_ptr()),
                        "Native FP4 epilogue setup")
                if rows is not None:
                    _native.check(lib.configure_resident_fp4_rows(self._handle, int(rows)), "Native FP4 rows")
                if block_n != 128:
                    _native.check(lib.configure_resident_fp4_tile(self._handle, int(block_n)), "Native FP4 tile")
                if tiled_weight:
                    # re-lay the packed weight tile-major: block (n tile, 256-wide K stage) = block_n contiguous 128-byte rows
                    tiled = self.b.view(n // block_n, block_n, k // 256, 128).permute(0, 2, 1, 3).contiguous()
                    self.b.copy_(tiled.view(n, k // 2))
                    _native.check(lib.configure_resident_fp4_weight_layout(self._handle, 1), "Native FP4 weight layout")
                values = (ctypes.c_int * 8)()
                _native.check(lib.resident_fp4_resources(self._handle, values, 8), "Native FP4 resource query")
            except Exception:
                self.close()
                raise
        self.resources = dict(zip(("registers_per_thread", "static_shared_bytes", "dynamic_shared_bytes",
                                   "local_bytes_per_thread", "predicted_max_ctas_per_sm", "threads_per_cta",
                                   "max_threads_per_sm", "sm_count"), values))

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
