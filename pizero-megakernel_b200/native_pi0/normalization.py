"""Fused LayerNorm / RMSNorm -> NVFP4 producer.

Constructor-compatible with the reference ``ResidentNorm`` (``native_pi0/normalization.py:9-82``): BF16 input,
``precision`` ``"fp4"`` (packed NVFP4 + swizzled block scales), ``"fp8"`` (E4M3 of value / global scale), ``"bf16"`` or
``"factor"`` (only the FP32 ``1 / sqrt(mean square + eps)`` per row, for projections whose weight has the norm weight
folded in), FP32 ``gamma`` / ``beta`` / ``inverse_scale`` (an AWQ-style per-channel factor applied after the affine
part), optional fused ``residual`` add (the sum is kept in ``residual_output``).  RMSNorm gamma must already contain
``1 + w``.  Not offered: FP16 input and the ``legacy_ties`` rounding variant.
"""
import ctypes

import numpy as np
import torch

from native_pi0 import _native
from native_pi0.storage import packed_tma_buffer


class ResidentNorm:
    def __init__(self, library, inputs, *, kind="rms", precision="fp4", gamma=None, beta=None,
                 inverse_scale=None, residual=None, workers=16, epsilon=1e-6, global_scale=1.,
                 round_normalized=True, round_residual=True, legacy_ties=False, row_alignment=1,
                 quantize_only=False, scale_policy="nearest", keep_bf16=False):
        if inputs.dtype != torch.bfloat16 or inputs.ndim != 2:
            raise ValueError("Inputs must be a BF16 matrix")
        rows, width = inputs.shape
        if rows < 1 or width < 16 or width % 16 or (width > 2048 and not quantize_only):
            raise ValueError("Width must be a multiple of 16 up to 2048")
        if kind not in ("rms", "layer") or precision not in ("fp4", "fp8", "bf16", "factor"):
            raise ValueError("Unknown normalization or precision (fp4, fp8, bf16 or factor)")
        if legacy_ties:
            raise ValueError("The legacy tie-breaking variant of the quantiser is not offered")
        if precision == "factor" and (kind != "rms" or any(x is not None for x in (gamma, beta, inverse_scale, residual))):
            raise ValueError("The RMS factor output takes raw rows: no affine parameters, no residual")
        if not isinstance(row_alignment, int) or row_alignment < 1:
            raise ValueError("Invalid row alignment")
        if kind == "rms" and beta is not None:
            raise ValueError("Standard pi0 RMSNorm has no beta")
        if not np.isfinite(epsilon) or epsilon <= 0 or not np.isfinite(global_scale) or global_scale <= 0:
            raise ValueError("Epsilon and global scale must be finite and positive")
        if scale_policy not in ("nearest", "ceil"):
            raise ValueError("scale_policy must be nearest or ceil")
        if precision == "bf16" and global_scale != 1.:
            raise ValueError("BF16 normalization requires unit global scale")
        self.logical_rows = rows
        self.workers = workers
        out_rows = (rows + row_alignment - 1) // row_alignment * row_alignment
        self.device = inputs.device if inputs.is_cuda else torch.device("cuda", torch.cuda.current_device())
        self.global_scale = np.float32(global_scale)
        self.library = _native.load(library)
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            self.inputs = inputs.to(self.device).contiguous()
            self.gamma, self.beta, self.inverse_scale = [
                None if v is None else torch.as_tensor(v, dtype=torch.float32, device=self.device).contiguous()
                for v in (gamma, beta, inverse_scale)]
            for vec in (self.gamma, self.beta, self.inverse_scale):
                if vec is not None and tuple(vec.shape) != (width,):
                    raise ValueError("Affine / inverse-scale vector shape mismatch")
            self.residual = self.residual_output = None
            if residual is not None:
                self.residual = torch.as_tensor(residual, dtype=torch.bfloat16, device=self.device).contiguous()
                if self.residual.shape != self.inputs.shape:
                    raise ValueError("Residual shape mismatch")
                self.residual_output = torch.empty_like(self.inputs)
            if precision == "factor":
                self.output, self.output_scales = torch.zeros(out_rows, dtype=torch.float32, device=self.device), None
            elif precision == "fp8":
                self.output, self.output_scales = torch.zeros((out_rows, width), dtype=torch.float8_e4m3fn, device=self.device), None
            elif precision == "fp4":
                self.output = packed_tma_buffer((out_rows, width // 2), device=self.device)
                self.output_scales = torch.zeros(((out_rows + 127) // 128) * ((width // 16 + 3) // 4) * 512,
                                                 dtype=torch.uint8, device=self.device)
            else:
                self.output = torch.zeros((out_rows, width), dtype=torch.bfloat16, device=self.device)
                self.output_scales = None
            self.normalized = torch.zeros((out_rows, width), dtype=torch.bfloat16, device=self.device) if keep_bf16 else None
            code = self.library.create_norm(
                ctypes.byref(self.handle), self.inputs.data_ptr(), _native.ptr(self.residual), _native.ptr(self.gamma), _native.ptr(self.beta),
                _native.ptr(self.inverse_scale), _native.ptr(self.residual_output), self.output.data_ptr(), _native.ptr(self.output_scales),
                rows, width, workers, 0, {"fp4": 4, "fp8": 8, "bf16": 16, "factor": 17}[precision], int(kind == "layer"),
                int(round_normalized), int(round_residual), 0, float(epsilon), float(self.global_scale))
            _native.check(code, "Native norm setup")
            try:
                if quantize_only:
                    _native.check(self.library.configure_norm_quantize_only(self.handle, int(scale_policy == "ceil")), "Native norm mode")
                if keep_bf16:
                    _native.check(self.library.configure_norm_bf16_copy(self.handle, self.normalized.data_ptr()), "Native norm copy")
            except Exception:
                self.close()
                raise

    def forward(self):
        if not self.handle.value:
            raise RuntimeError("Normalization instance is closed")
        with torch.cuda.device(self.device):
            _native.check(self.library.launch_norm(self.handle, torch.cuda.current_stream(self.device).cuda_stream),
                          "Native norm launch")
        return self.output

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.library, self.handle)

    def close(self):
        if self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.library.destroy_norm(self.handle), "Native norm teardown")
            self.handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
