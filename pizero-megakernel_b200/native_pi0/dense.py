"""Resident BF16 / FP8 projections on tcgen05 with the BF16 model's fused epilogues.

Constructor-compatible with the reference ``ResidentDense`` (``native_pi0/dense.py:8-129``): ``inputs [M, K]`` and
``weights [N, K]`` in BF16 or FP8 E4M3 are copied into buffers padded to multiples of 128 (rows) and 64 (K), unless
the caller binds padded buffers itself; ``forward()`` launches on the current stream and returns the logical
``[M, N]`` view of the reused output.  ``alpha`` is the product of the static FP8 descales.  Epilogue options (BF16
operands and BF16 output unless noted): ``bias`` / ``residual`` (any output type; added in FP32, residual first),
``round_before_residual``, ``geglu_output`` (compact ``[M, N/2]`` from interleaved gate/up rows of the weight),
``gelu``, ``rms_factors`` (FP32 ``[M_pad]`` row factors), ``skinny`` (at most 64 rows) and ``rope`` + ``kv_cache``
(fused QKV epilogue: rotate-half RoPE on the Q heads and the K head, K and V rows appended to the cache).

One layout difference from the reference: with ``rope`` the kernel rotates ADJACENT column pairs, so this wrapper
stores the rows of every Q head and of the K head of the weight in the order (0, 128, 1, 129, ...); the rotated Q in
the output and K in the cache are in that same pair order.  Attention over them is unaffected (a dot product does not
care about a common permutation); ``head_order`` gives the permutation for anyone who wants to read Q or K directly.
"""
import ctypes
import math

import torch

from native_pi0 import _native

_HEAD = 256


def head_order(device=None):
    """Index vector p with stored[:, j] = standard[:, p[j]] inside one 256-wide rotated head."""
    half = torch.arange(_HEAD // 2, device=device)
    return torch.stack((half, half + _HEAD // 2), dim=1).reshape(-1)


def _round_up(value, multiple):
    return (value + multiple - 1) // multiple * multiple


class ResidentDense:
    def __init__(self, library, inputs, weights, *, alpha=1., bias=None, residual=None, output_dtype=torch.bfloat16, workers=148,
                 input_buffer=None, weight_buffer=None, output_buffer=None, residual_buffer=None, round_before_residual=False,
                 geglu_output=None, gelu=False, rms_factors=None, skinny=False, rope=None, kv_cache=None, rope_key_offset=0,
                 cache_base=0):
        self.handle = ctypes.c_void_p()
        if inputs.ndim != 2 or weights.ndim != 2 or inputs.shape[1] != weights.shape[1]:
            raise ValueError("inputs [M, K] and weights [N, K] must share K")
        dtype = inputs.dtype
        if dtype not in (torch.bfloat16, torch.float8_e4m3fn) or weights.dtype != dtype:
            raise ValueError("inputs and weights must both be BF16 or both FP8 E4M3")
        if output_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("output_dtype must be torch.bfloat16 or torch.float32")
        m, k = inputs.shape
        n = weights.shape[0]
        self.alpha = ctypes.c_float(alpha).value
        if min(m, n, k) < 1 or not math.isfinite(self.alpha) or self.alpha <= 0:
            raise ValueError("dimensions must be positive and alpha a positive finite FP32 number")
        fp8 = dtype == torch.float8_e4m3fn
        bf16_path = not fp8 and output_dtype == torch.bfloat16
        self._check_options(bf16_path, m, n, bias, residual, residual_buffer, round_before_residual, geglu_output, gelu,
                            rms_factors, skinny, rope, kv_cache)
        self.logical_rows, self.logical_columns, self.logical_k = m, n, k
        self.workers, self.skinny = workers, skinny
        self.device = inputs.device if inputs.is_cuda else torch.device("cuda", torch.cuda.current_device())
        mp, np_, kp = _round_up(m, 128), _round_up(n, 128), _round_up(k, 128 if fp8 else 64)
        self.library = lib = _native.load(library)

        def bound(value, shape, kind, what):
            """A caller-owned padded buffer, or a fresh zeroed one."""
            if value is None:
                return torch.zeros(shape, dtype=kind, device=self.device)
            if (value.device != self.device or value.dtype != kind or tuple(value.shape) != tuple(shape) or not value.is_contiguous()
                    or value.data_ptr() % 128):
                raise ValueError(f"{what} must be a contiguous {kind} tensor of padded shape {tuple(shape)} on {self.device}, 128-byte aligned")
            return value

        with torch.cuda.device(self.device):
            self.a = bound(input_buffer, (mp, kp), dtype, "input_buffer")
            self.b = bound(weight_buffer, (np_, kp), dtype, "weight_buffer")
            if input_buffer is None:
                self.a[:m, :k].copy_(inputs)
            if weight_buffer is None:
                stored = weights
                if rope is not None:
                    stored = weights.clone()
                    order = head_order(weights.device)
                    for start in range(0, rope_key_offset + _HEAD, _HEAD):          # every Q head and the K head
                        stored[start:start + _HEAD] = weights[start:start + _HEAD][order]
                self.b[:n, :k].copy_(stored)
            self.inputs, self.weights = self.a[:m, :k], self.b[:n, :k]
            self.bias = self.residual = None
            if bias is not None:
                value = torch.as_tensor(bias, dtype=torch.bfloat16, device=self.device)
                if tuple(value.shape) != (n,):
                    raise ValueError(f"bias must have shape ({n},)")
                self.bias = torch.zeros(np_, dtype=torch.bfloat16, device=self.device)
                self.bias[:n].copy_(value)
            if residual_buffer is not None:
                self.residual = bound(residual_buffer, (mp, np_), torch.bfloat16, "residual_buffer")
            elif residual is not None:
                value = torch.as_tensor(residual, dtype=torch.bfloat16, device=self.device)
                if tuple(value.shape) != (m, n):
                    raise ValueError(f"residual must have shape ({m}, {n})")
                self.residual = torch.zeros((mp, np_), dtype=torch.bfloat16, device=self.device)
                self.residual[:m, :n].copy_(value)
            self.output = bound(output_buffer, (mp, np_), output_dtype, "output_buffer")
            self.logical_output = self.output[:m, :n]
            _native.check(lib.create_dense(ctypes.byref(self.handle), self.a.data_ptr(), self.b.data_ptr(), self.output.data_ptr(),
                                           _native.ptr(self.bias), _native.ptr(self.residual), mp, np_, kp, workers, int(fp8),
                                           int(output_dtype == torch.bfloat16), self.alpha), "Native dense setup")
            try:
                if round_before_residual:
                    _native.check(lib.configure_dense_round_before_residual(self.handle), "Native dense residual rounding")
                if geglu_output is not None:
                    bound(geglu_output, (mp, np_ // 2), torch.bfloat16, "geglu_output")
                    _native.check(lib.configure_dense_geglu(self.handle, geglu_output.data_ptr()), "Native dense GeGLU epilogue")
                    self.geglu_output = geglu_output
                    self.logical_output = geglu_output[:m, :n // 2]
                if gelu:
                    _native.check(lib.configure_dense_gelu(self.handle, n), "Native dense GELU epilogue")
                if rms_factors is not None:
                    bound(rms_factors, (mp,), torch.float32, "rms_factors")
                    _native.check(lib.configure_dense_rms_factor(self.handle, rms_factors.data_ptr()), "Native dense RMS factor")
                    self.rms_factors = rms_factors
                if skinny:
                    _native.check(lib.configure_dense_skinny(self.handle), "Native dense skinny setup")
                elif m < mp:
                    _native.check(lib.configure_dense_rows(self.handle, m), "Native dense rows")
                if rope is not None:
                    self._bind_rope(rope, kv_cache, m, rope_key_offset, cache_base)
            except Exception:
                self.close()
                raise

    @staticmethod
    def _check_options(bf16_path, m, n, bias, residual, residual_buffer, round_before_residual, geglu_output, gelu, rms_factors,
                       skinny, rope, kv_cache):
        fused_add = bias is not None or residual is not None
        if residual_buffer is not None and residual is None:
            raise ValueError("residual_buffer needs residual")
        if round_before_residual and (residual is None or not bf16_path):
            raise ValueError("round_before_residual needs a residual on the BF16 path")
        if geglu_output is not None and (not bf16_path or fused_add or n % 256):
            raise ValueError("GeGLU needs BF16 gate/up pairs (N a multiple of 256) without bias or residual")
        if gelu and (not bf16_path or residual is not None or geglu_output is not None):
            raise ValueError("GELU needs the BF16 path without residual or GeGLU")
        if rms_factors is not None and (not bf16_path or fused_add):
            raise ValueError("RMS row factors need the BF16 path without bias or residual")
        if skinny and (m > 64 or not bf16_path):
            raise ValueError("skinny projections have at most 64 BF16 rows")
        if rope is not None and (kv_cache is None or len(rope) != 2 or len(kv_cache) != 2 or not bf16_path or fused_add):
            raise ValueError("the QKV RoPE epilogue needs (cos, sin), (cache_k, cache_v) and a plain BF16 projection")

    def _bind_rope(self, rope, kv_cache, m, key_offset, cache_base):
        cos, sin = rope
        cache_k, cache_v = kv_cache
        tables_ok = all(tuple(t.shape) == (1, m, _HEAD) and t.dtype == torch.bfloat16 for t in (cos, sin))
        caches_ok = (cache_k.shape == cache_v.shape and cache_k.ndim == 4 and cache_k.shape[0] == 1 and tuple(cache_k.shape[2:]) == (1, _HEAD)
                     and cache_k.dtype == cache_v.dtype == torch.bfloat16 and cache_base + m <= cache_k.shape[1])
        placed = all(t.device == self.device and t.is_contiguous() for t in (cos, sin, cache_k, cache_v))
        if not (tables_ok and caches_ok and placed):
            raise ValueError("RoPE tables must be BF16 [1, M, 256] and the caches BF16 [1, rows, 1, 256] with room for the new rows")
        self.rope, self.kv_cache = rope, kv_cache
        _native.check(self.library.configure_dense_qkv_rope(self.handle, cos.data_ptr(), sin.data_ptr(), cache_k.data_ptr(),
                                                            cache_v.data_ptr(), m, key_offset, cache_base), "Native dense QKV RoPE setup")

    def forward(self):
        if not self.handle.value:
            raise RuntimeError("Dense instance is closed")
        with torch.cuda.device(self.device):
            _native.check(self.library.launch_dense(self.handle, torch.cuda.current_stream(self.device).cuda_stream), "Native dense launch")
        return self.logical_output

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.library, self.handle)

    def close(self):
        if self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.library.destroy_dense(self.handle), "Native dense teardown")
            self.handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
