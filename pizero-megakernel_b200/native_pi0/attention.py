"""Attention operator: MHA / GQA / MQA over BF16 Q, K, V with FP32 softmax.

Constructor-compatible with the reference ``ResidentAttention`` (``native_pi0/attention.py:8-139``) for
the pi0 cases: BF16 tensors ``q [B, Nq, H, d]``, ``k, v [B, Nk, Hk, d]`` (views with a common row stride
are accepted), optional pi0 suffix mask (``prefix``), optional KV cache, optional split-KV with merge.
Optional per-head biases, rotate-half RoPE tables and a boolean visibility mask as in the reference; with biases, tables
or a head size other than 72 / 256 an operand-preparation stage runs in front of the attention inside the same launch.

Two tile implementations sit behind the one operator: tcgen05 tiles (operands by TMA, scores, probabilities and
output in tensor memory) where the geometry allows them - heads that occupy 128 or 256 elements in memory and at most
256 keys per tile - and mma.sync tiles otherwise; ``path`` forces one of them.  ``head_dim`` smaller than the last
tensor dimension declares a padded layout (e.g. SigLIP's 72-wide heads stored 128 apart, zeros behind them).
"""
import ctypes

import torch

from native_pi0 import _native


class ResidentAttention:
    def __init__(self, library, q, k, v, *, workers=16, scale=None, prefix=None, splits=1, kv_cache=None,
                 cached_prefix_rows=0, output=None, q_bias=None, k_bias=None, v_bias=None, q_rope=None,
                 k_rope=None, mask=None, fp4_output=None, fused_merge=False, path=None, head_dim=None, fp4_pitch=None, bias=None):
        if bias is not None:                                 # the reference's form: one (query, key, value) triple
            if len(bias) != 3 or any(x is not None for x in (q_bias, k_bias, v_bias)):
                raise ValueError("bias is a (query, key, value) triple; give it or the separate arguments")
            q_bias, k_bias, v_bias = bias
        for t in (q, k, v):
            if t.dtype != torch.bfloat16 or t.ndim != 4 or not t.is_cuda or t.stride(-1) != 1:
                raise ValueError("q, k, v must be CUDA BF16 [batch, rows, heads, dim] with contiguous dim")
        b, nq, h, stored = q.shape
        bk, nk, hk, dk = k.shape
        d = stored if head_dim is None else int(head_dim)
        if v.shape != k.shape or bk != b or dk != stored or h % hk or d % 8 or not 8 <= d <= 256 or d > stored or (d < stored and stored not in (128, 256)):
            raise ValueError("Unsupported attention geometry (head_dim a multiple of 8 up to 256, heads a multiple of kv heads)")
        extras = any(x is not None for x in (q_bias, k_bias, v_bias, q_rope, k_rope))
        if (extras or d not in (72, 256)) and (d < stored or kv_cache is not None):
            raise ValueError("Biases, RoPE tables and other head sizes take unpadded heads and no KV cache")
        if path not in (None, "mma.sync", "tcgen05"):
            raise ValueError("path is None, 'mma.sync' or 'tcgen05'")
        if q.stride(2) != stored or k.stride(2) != stored or v.stride(2) != stored or k.stride(1) != v.stride(1):
            raise ValueError("Heads must be adjacent and K/V must share a row stride")
        if b > 1 and (q.stride(0) != nq * q.stride(1) or k.stride(0) != nk * k.stride(1) or v.stride(0) != nk * v.stride(1)):
            raise ValueError("Batches must be stacked rows")
        self.device = q.device
        self.scale = float(d ** -0.5 if scale is None else scale)
        self.q, self.k, self.v = q, k, v
        self.library = _native.load(library)
        self.handle = ctypes.c_void_p()
        self.kv_cache = kv_cache
        with torch.cuda.device(self.device):
            if output is None:
                output = torch.zeros((b, nq, h, d), dtype=torch.bfloat16, device=self.device)
            if output.dtype != torch.bfloat16 or tuple(output.shape) != (b, nq, h, d) or output.stride(2) != d:
                raise ValueError("Output must be BF16 [batch, rows, heads, dim]")
            self.output = output

            def optional(value, shape, what, dtype=torch.bfloat16):
                if value is None:
                    return None
                tensor = torch.as_tensor(value, device=self.device).to(dtype).contiguous()
                if tuple(tensor.shape) != tuple(shape):
                    raise ValueError(f"{what} must have shape {tuple(shape)}")
                return tensor

            self.bias = [optional(x, (heads, d), "bias") for x, heads in zip((q_bias, k_bias, v_bias), (h, hk, hk))]
            for tables in (q_rope, k_rope):
                if tables is not None and (len(tables) != 2 or any(x is None for x in tables)):
                    raise ValueError("RoPE needs cosine and sine tensors")
            self.q_rope = [None, None] if q_rope is None else [optional(x, (b, nq, d), "query RoPE table") for x in q_rope]
            self.k_rope = [None, None] if k_rope is None else [optional(x, (b, nk, d), "key RoPE table") for x in k_rope]
            self.mask = optional(mask, (b, nq, nk), "mask", torch.uint8)
            _native.check(self.library.create_attention(
                ctypes.byref(self.handle), q.data_ptr(), k.data_ptr(), v.data_ptr(), *[_native.ptr(x) for x in self.bias],
                _native.ptr(self.q_rope[0]), _native.ptr(self.q_rope[1]), _native.ptr(self.k_rope[0]), _native.ptr(self.k_rope[1]),
                output.data_ptr(), _native.ptr(self.mask), b, nq, nk, h, hk, d, q.stride(1), k.stride(1), output.stride(1), 0, workers,
                -1 if prefix is None else int(prefix), self.scale), "Native attention setup")
            try:
                if d < stored:
                    _native.check(self.library.configure_attention_head_pad(self.handle, stored), "Native attention head padding")
                if kv_cache is not None:
                    ck, cv = kv_cache
                    rows = cached_prefix_rows + nk
                    _native.check(self.library.configure_attention_cache(self.handle, ck.data_ptr(), cv.data_ptr(), rows,
                                                                         cached_prefix_rows), "Native attention cache")
                if fp4_output is not None:
                    data, scales, gs = fp4_output
                    pitch = d if fp4_pitch is None else int(fp4_pitch)
                    if pitch != d:
                        _native.check(self.library.configure_attention_fp4_pitch(self.handle, pitch), "Native attention FP4 head pitch")
                    _native.check(self.library.configure_attention_fp4_output(
                        self.handle, data.data_ptr(), scales.data_ptr(), data.stride(0), h * pitch // 16, float(gs)),
                        "Native attention FP4 output")
                if splits != 1:
                    _native.check(self.library.configure_attention_splits(self.handle, int(splits)), "Native attention splits")
                    if fused_merge:
                        _native.check(self.library.configure_attention_fused_merge(self.handle, 1), "Native attention fused merge")
                if path is not None:
                    _native.check(self.library.configure_attention_path(self.handle, int(path == "tcgen05")), "Native attention path")
                _native.check(self.library.attention_validate(self.handle), "Native attention configuration (prepared operands and masks need the tcgen05 tiles: at most 256 keys per tile)")
            except Exception:
                self.close()
                raise
        self.splits = splits

    @property
    def merge_handle(self):
        out = ctypes.c_void_p()
        _native.check(self.library.attention_merge_handle(self.handle, ctypes.byref(out)), "Native attention merge handle")
        return out

    def forward(self):
        if not self.handle.value:
            raise RuntimeError("Attention instance is closed")
        with torch.cuda.device(self.device):
            _native.check(self.library.launch_attention(self.handle, torch.cuda.current_stream(self.device).cuda_stream),
                          "Native attention launch")
        return self.output

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.library, self.handle)

    def _split_only(self):
        if not self.handle.value or self.splits == 1:
            raise RuntimeError("A live split attention instance is required")

    def poison_partials(self):
        """Development aid (``native_pi0/attention.py:131-137``): overwrite the split-KV scratch with NaN patterns on
        the current stream, so that a following launch which read a stale partial would show it."""
        self._split_only()
        with torch.cuda.device(self.device):
            _native.check(self.library.attention_poison_partials(self.handle, torch.cuda.current_stream(self.device).cuda_stream),
                          "Attention scratch poisoning")

    def read_split_counts(self):
        """Development aid (``native_pi0/attention.py:120-129``): synchronise and return the launch count and, per
        (128-query tile, head) group, the number of split tiles that have arrived so far; after clean launches every
        count is ``splits * epoch``."""
        self._split_only()
        groups = self.q.shape[2] * ((self.q.shape[1] + 127) // 128)
        counts, epoch = (ctypes.c_ulonglong * groups)(), ctypes.c_uint()
        with torch.cuda.device(self.device):
            _native.check(self.library.attention_split_diagnostics(self.handle, counts, groups, ctypes.byref(epoch)),
                          "Attention diagnostics")
        return {"epoch": epoch.value, "counts": list(counts)}

    def close(self):
        if self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.library.destroy_attention(self.handle), "Native attention teardown")
            self.handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
