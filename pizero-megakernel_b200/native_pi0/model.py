"""NVFP4 pi0 on one B200: the whole forward as one persistent launch over static instruction streams.

``NativePi0`` keeps the surface of the reference class (``native_pi0/model.py:34-348``):
``from_openpi`` / ``from_model`` constructors, ``forward(images, state, noise, tokens)`` returning the
reused FP32 action tensor ``[1, chunk, 32]``, ``launch_component``, ``read_timings``, ``close`` and the
context-manager protocol, with the attributes ``output, plan, stages, landmarks, component_ranges, epoch,
precision_policy``.  What differs is the engine underneath: every transformer linear is an NVFP4
block-scaled GEMM on tcgen05 (weights packed on the device at setup with the ``ceil`` scale policy and a
per-tensor scale of amax/(6*448); activations quantised on the fly with the ``nearest`` policy and tensor
scale 1), RoPE and the KV-cache write live in the QKV epilogue, GeGLU/GELU + requantisation live in the
MLP epilogues, and the 51-row action expert uses split-KV attention with a merge stage.

``precision`` selects the operand format of the transformer linears site by site: ``"nvfp4"`` (or ``"auto"``) for
all of them, ``"bf16"`` for all of them (the reference's ``bf16_reference`` policy: BF16 weights and activations on
``tcgen05.mma kind::f16``, projections rounded to BF16 before the residual add as OpenPI's eager model does), or a
dict of ``fnmatch`` patterns over site names -> ``"nvfp4" | "bf16"`` with an optional ``"default"``; the first
matching pattern wins.  Sites are ``vision.<layer>.{qkv,out,fc1,fc2}``, ``vision.projector``,
``prefix.<layer>.{qkv,o_proj,gate_up,down}`` and ``expert.<layer>.{qkv,o_proj,gate_up,down}`` (an expert site covers
all Euler steps: they share the weight).  A producer writes its output in the format its consumer reads, so a
BF16 site costs its own weight traffic and nothing else.

Setup owns all layouts, buffers, weight transforms and the instruction streams; ``forward`` only launches.
"""
from __future__ import annotations

import ctypes as C
import fnmatch
import math
from pathlib import Path

import numpy as np
import torch

from native_pi0 import _native
from native_pi0._native import NativeSpec
from native_pi0.program import LinearWork, linear_streams, program_summary, spread_streams, validate_streams
from native_pi0.quantization import swizzled_size
from native_pi0.storage import packed_tma_buffer
from native_pi0.weights import EXPERT, LANGUAGE, PROJECTOR, VISION, Pi0Config, StateDictModel

SAME, ALL = 0, 1


def padded(n, a):
    return (n + a - 1) // a * a


class Fp4Matrix:
    """Device-resident NVFP4 matrix: packed codes [rows_pad, k/2], swizzled E4M3 scales, FP32 tensor scale."""

    def __init__(self, rows_pad, k, device, global_scale=1.0):
        self.rows_pad, self.k = rows_pad, k
        self.data = packed_tma_buffer((rows_pad, k // 2), device=device)
        self.scales = torch.zeros(swizzled_size(rows_pad, k // 16), dtype=torch.uint8, device=device)
        self.global_scale = float(np.float32(global_scale))


class DenseMatrix:
    """Device-resident BF16 weight [rows_pad, k] (K contiguous, padded to 64) of a BF16 site."""

    def __init__(self, data, logical_rows):
        self.data, self.rows_pad, self.k, self.logical_rows = data, data.shape[0], data.shape[1], logical_rows
        self.tiled = 0


class Activation:
    """A GEMM input that one producer stage writes: NVFP4 (codes + block scales) and / or BF16 rows, whichever its
    consumers read.  The buffers are created on first demand and shared by every layer that uses this slot."""

    def __init__(self, engine, rows_pad, width):
        self.engine, self.rows_pad, self.width = engine, rows_pad, width
        self.fp4 = self.bf16 = None

    def require(self, precision):
        if precision == "nvfp4" and self.fp4 is None:
            self.fp4 = self.engine.fp4(self.rows_pad, self.width)
        if precision == "bf16" and self.bf16 is None:
            self.bf16 = self.engine.tensor((self.rows_pad, self.width))
        return self

    def only(self, precision):
        """This slot restricted to one form (what a producer should write for one particular consumer)."""
        view = Activation(self.engine, self.rows_pad, self.width)
        self.require(precision)
        view.fp4, view.bf16 = (self.fp4, None) if precision == "nvfp4" else (None, self.bf16)
        return view


class StageOutput:
    """What one stage writes, for validators that compare or replace a stage's result: ``name`` is the stage name
    (suffixed ``.q`` / ``.k`` / ``.v`` for the three parts of a fused QKV projection), ``kind`` one of ``bf16``,
    ``f32``, ``fp4`` (an ``Fp4Matrix``), ``sumsq`` (FP32 sums of squares of the BF16 rows per output tile, ``head`` =
    (tile width,)), ``q_rope`` (BF16 query heads, rotation partners adjacent), ``k_cache`` (the
    same layout, rows ``base..base+rows`` of the layer's key cache) and ``v_cache``; ``rows`` x ``cols`` is the
    logical extent inside the padded buffer."""

    def __init__(self, name, kind, buffer, rows, cols, base=0, head=None):
        self.name, self.kind, self.buffer, self.rows, self.cols, self.base = name, kind, buffer, rows, cols, base
        self.head = head            # kind "bf16": (head width, pitch) when heads are stored apart with zeros between them


class NativePi0:
    @classmethod
    def from_openpi(cls, checkpoint_path, *, num_views=3, prompt_len=0, chunk_size=50, flow_steps=10,
                    precision="auto", library=None, **kwargs):
        """Load an OpenPI ``model.safetensors`` (parameter names of ``PI0Pytorch``) straight into the engine."""
        from safetensors.torch import load_file
        path = Path(checkpoint_path)
        if path.is_dir():
            path = path / "model.safetensors"
        sd = load_file(str(path), device="cuda")
        config = kwargs.pop("config", None) or Pi0Config.from_state_dict(sd)
        return cls(StateDictModel(config, sd), num_views=num_views, prompt_len=prompt_len, chunk_size=chunk_size,
                   flow_steps=flow_steps, precision=precision, library=library, **kwargs)

    @classmethod
    def from_model(cls, model, **kwargs):
        return cls(model, **kwargs)

    @classmethod
    def from_state_dict(cls, state_dict, config=None, **kwargs):
        return cls(StateDictModel(config or Pi0Config(), state_dict), **kwargs)

    def __init__(self, model, *, num_views=3, prompt_len=0, chunk_size=50, flow_steps=10, precision="auto",
                 library=None, workers=None, partitioned=False, expert_splits=None, prefix_splits=None, expert_block_n=None, vision_block_n=64, fold_layernorms=True,
                 rope_inv_freq_dtype=torch.float32, keep_debug_outputs=False, verbose=False, tile_weights=True, schedule="affine",
                 fold_norms=True, attention_path=None, weight_store=None):
        config = getattr(model, "config", None)
        if config is None or getattr(config, "pi05", False):
            raise ValueError("This engine runs ordinary pi0 (not pi0.5)")
        if isinstance(precision, dict):
            self.precision_map = [(k, v) for k, v in precision.items() if k != "default"]
            self.default_precision = precision.get("default", "nvfp4")
        elif precision in ("auto", "nvfp4", "bf16"):
            self.precision_map, self.default_precision = [], "bf16" if precision == "bf16" else "nvfp4"
        else:
            raise ValueError("precision must be 'auto', 'nvfp4', 'bf16' or a dict of site patterns")
        if any(v not in ("nvfp4", "bf16") for _, v in self.precision_map) or self.default_precision not in ("nvfp4", "bf16"):
            raise ValueError("site precisions are 'nvfp4' or 'bf16'")
        if num_views not in (1, 2, 3) or prompt_len < 0 or chunk_size < 1 or chunk_size > 127 or flow_steps < 1:
            raise ValueError("Invalid fixed inference dimensions")
        if not isinstance(config, Pi0Config):
            config = Pi0Config(**{k: getattr(config, k) for k in Pi0Config.__dataclass_fields__ if hasattr(config, k)})
        self.config = config
        self.num_views, self.prompt_len, self.chunk_size, self.flow_steps = num_views, prompt_len, chunk_size, flow_steps
        self.site_precisions = {}
        self.partitioned = partitioned
        self.expert_splits = expert_splits
        self.prefix_splits = prefix_splits
        self.vision_block_n = vision_block_n
        self.fold_layernorms = bool(fold_layernorms)
        # output tile widths of the action expert's projections: an int for all four, or a dict per operation.  The default
        # gives the projections with few output columns 32-wide tiles (twice the workers, half the bytes of weight and half
        # the serial epilogue per worker); gate/up runs as 64 tiles of 128, which leaves its neighbours (32 tiles each)
        # workers of their own, so that no tile of the three stages starts on a worker that has just run its source
        if expert_block_n is None:
            expert_block_n = {"qkv": 64, "o_proj": 32, "gate_up": 128, "down": 32}
        self.expert_block_n = expert_block_n
        self.rope_inv_freq_dtype = rope_inv_freq_dtype
        self.keep_debug_outputs = keep_debug_outputs
        self.tile_weights = tile_weights
        self.fold_norms = bool(fold_norms)
        if attention_path not in (None, "mma.sync", "tcgen05"):
            raise ValueError("attention_path is None (by geometry), 'mma.sync' or 'tcgen05'")
        self.attention_path = attention_path
        if schedule not in ("spread", "affine", "linear"):
            raise ValueError("schedule must be 'spread', 'affine' or 'linear'")
        self.schedule = schedule
        self.verbose = verbose
        sd = model.state_dict()
        self.device = next(iter(sd.values())).device
        if self.device.type != "cuda":
            raise ValueError("Supply CUDA-resident parameters")
        self.library_path = Path(library).resolve() if library is not None else _native.LIBRARY
        self.lib = _native.load(self.library_path)
        with torch.cuda.device(self.device):
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.workers = min(sms, 148) if workers is None else workers
        self.sd = sd
        self.buffers, self.handles, self._cache = [], [], {}
        # packed weights, keyed by parameter and operand format: engines of different shapes (views, prompt, chunk) that
        # are given the same store share one copy of every weight (EngineCache)
        self._weights = weight_store if weight_store is not None else {}
        self.stages, self.stage_tiles, self.stage_cost, self.stage_names, self.stage_outputs = [], [], [], [], []
        self.landmarks, self.landmark_stage = {}, {}
        self.handle = C.c_void_p()
        self.epoch = 0
        try:
            with torch.cuda.device(self.device), torch.no_grad():
                self._build()
        except Exception:
            self.close()
            raise
        self.sd = None
        used = set(self.site_precisions.values())
        self.precision_policy = "nvfp4" if used == {"nvfp4"} else "bf16_reference" if used == {"bf16"} else "mixed"

    def site(self, name):
        """Operand format of the linear at ``name``: first matching pattern of the precision dict, else the default."""
        if name not in self.site_precisions:
            chosen = next((v for k, v in self.precision_map if fnmatch.fnmatchcase(name, k)), self.default_precision)
            self.site_precisions[name] = chosen
        return self.site_precisions[name]

    # ------------------------------------------------------------------------------------------ buffers
    def tensor(self, shape, dtype=torch.bfloat16):
        t = torch.zeros(shape, device=self.device, dtype=dtype)
        self.buffers.append(t)
        return t

    def fp4(self, rows_pad, k):
        m = Fp4Matrix(rows_pad, k, self.device)
        self.buffers.append(m)
        return m

    def cached(self, key, make):
        """Build a derived tensor once and share it between stages: string keys name weights (quantised matrices, folded
        gammas; also shared between engines through ``weight_store``), other keys name buffers of this engine."""
        store = self._weights if isinstance(key, str) else self._cache
        if key not in store:
            store[key] = make()
        return store[key]

    def weight(self, w, *, rows_to=128, block_n=128, precision="nvfp4", row_sums=False):
        """BF16/FP32 [N, K] -> the site's operand format on the device: NVFP4 (ceil block scales, tensor scale
        amax/(6*448)) or zero-padded BF16.

        When K is a multiple of 256 the packed NVFP4 codes are re-laid tile-major for ``block_n``-wide output tiles
        (``Fp4Matrix.tiled = block_n``): every TMA box of the weight operand is then one contiguous read."""
        n, k = w.shape
        np_, kp = padded(n, rows_to), padded(k, 64)
        src = torch.zeros((np_, kp), device=self.device, dtype=torch.bfloat16)
        src[:n, :k] = w.to(torch.bfloat16)
        if precision == "bf16":
            m = DenseMatrix(src, n)
            self.buffers.append(m)
            return m
        gs = max(float(src.float().abs().max()) / (6.0 * 448.0), 1e-30)
        m = Fp4Matrix(np_, kp, self.device, gs)
        m.logical_rows = n
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _native.check(self.lib.quantize_nvfp4(src.data_ptr(), m.data.data_ptr(), m.scales.data_ptr(), np_, kp, kp, kp // 16,
                                              m.global_scale, 1, stream), "weight quantisation")
        if row_sums:
            m.row_sums = self._fp4_row_sums(m, np_, kp)     # sum over K of every row as the MMA reads it (folded LayerNorm)
        if block_n == 32:
            from native_pi0.primitives import narrow_tile_scales
            m.scales = narrow_tile_scales(m.scales, np_, kp // 16)     # an atom of scales per 32-row tile
        m.scale_tile = block_n if block_n == 32 else 128
        m.tiled = 0
        if self.tile_weights and kp % 256 == 0 and np_ % block_n == 0:
            tiled = m.data.view(np_ // block_n, block_n, kp // 256, 128).permute(0, 2, 1, 3).contiguous()
            m.data.copy_(tiled.view(np_, kp // 2))
            m.tiled = block_n
        torch.cuda.current_stream(self.device).synchronize()
        self.buffers.append(m)
        return m

    def _fp4_row_sums(self, m, rows, k):
        """FP32 [rows]: the sum over K of every row of a freshly quantised NVFP4 matrix (codes row-major, scales in the
        standard atom layout), decoded exactly as the tensor core decodes it."""
        from native_pi0.quantization import E2M1, UE4M3, scale_offsets
        values = torch.tensor(np.concatenate((E2M1, -E2M1)), device=self.device)
        data = m.data[:rows, :k // 2].long()
        pairs = values[data & 15] + values[data >> 4]                      # [rows, k / 2]: two elements per byte
        blocks = pairs.view(rows, k // 16, 8).sum(-1)
        where = torch.from_numpy(scale_offsets(rows, k // 16).astype(np.int64)).to(self.device)
        scale = torch.tensor(UE4M3, device=self.device)[m.scales[where].long()]
        return ((blocks * scale).sum(-1) * np.float32(m.global_scale)).float().contiguous()

    # ------------------------------------------------------------------------------------------ stages
    def add(self, kind, handle, name, sources=(), outputs=()):
        tiles, bands, cost = C.c_int(), C.c_int(), C.c_int()
        _native.check(self.lib.op_geometry(handle, C.byref(tiles), C.byref(bands), C.byref(cost)), "operator geometry")
        spec = NativeSpec()
        spec.kind, spec.handle = kind, handle.value if isinstance(handle, C.c_void_p) else handle
        srcs = [(s, m) for s, m in sources if s is not None and s >= 0]
        if len(srcs) > 4:
            raise ValueError("Too many stage sources")
        for i in range(4):
            spec.sources[i], spec.modes[i] = srcs[i] if i < len(srcs) else (-1, ALL)
        self.stages.append(spec)
        self.stage_tiles.append(tiles.value)
        self.stage_cost.append(padded(max(cost.value, 64), 64))
        self.stage_names.append(name)
        self.stage_outputs.append(list(outputs))
        return len(self.stages) - 1

    def mark(self, name, tensor):
        self.landmarks[name] = tensor
        self.landmark_stage[name] = len(self.stages)       # valid once stages [0, this) have run

    def _own(self, handle):
        self.handles.append(handle)
        return handle

    def gemm(self, name, a: Activation, w, *, rows, sources, out=None, bias=None, residual=None,
             out_act: Activation = None, out_precision=None, activation=0, act_cols=None, rope=None, block_n=128,
             stream=None, row_rms=None, row_ln=None, head_pad=None):
        """One projection stage.  ``w`` decides the operand format (``Fp4Matrix``: NVFP4 on ``a.fp4``; ``DenseMatrix``:
        BF16 on ``a.bf16``).  The result goes to ``out`` (BF16, + bias + residual), to the fused QKV destinations
        (``rope``), or to ``out_act`` in the format ``out_precision`` of the consuming site with ``activation``
        0 none / 1 GELU / 2 GeGLU over interleaved gate/up columns (``act_cols``: logical width for the GELU).
        ``stream=(copy, sumsq)``: besides ``out`` the stage writes the un-normalised NVFP4 copy of its rows into the
        ``Activation`` ``copy`` and per-tile sums of squares into ``sumsq``; ``row_rms=(sumsq, parts, width, eps)``: the
        stage reads such a copy and applies the RMS row factor itself (its weight carries the norm weight).  The LayerNorm
        form: ``stream=(copy, sumsq, sums)`` (statistics rows ``sumsq.shape[1]`` slots long) and
        ``row_ln=(sumsq, sums, width, eps, center)`` with ``center`` the row sums of the weight."""
        h = C.c_void_p()
        dense = isinstance(w, DenseMatrix)
        src = a.bf16 if dense else a.fp4
        if src is None:
            raise ValueError(f"{name}: the producer of this activation does not write the {'BF16' if dense else 'NVFP4'} form")
        m, n, k = a.rows_pad, w.rows_pad, w.k
        if (src.shape[1] if dense else src.k) != k:
            raise ValueError(f"{name}: K mismatch")
        target = None if out_act is None else (out_act.bf16 if out_precision == "bf16" else out_act.fp4)
        placeholder = src if dense else src.data            # every path below binds the real destination
        if dense:
            _native.check(self.lib.create_dense(C.byref(h), src.data_ptr(), w.data.data_ptr(), placeholder.data_ptr(), None, None,
                                                m, n, k, self.workers, 0, 1, 1.0), name)
        else:
            _native.check(self.lib.create_resident_fp4(C.byref(h), src.data.data_ptr(), w.data.data_ptr(), src.scales.data_ptr(),
                                                       w.scales.data_ptr(), placeholder.data_ptr(), m, n, k, self.workers,
                                                       float(np.float32(src.global_scale) * np.float32(w.global_scale))), name)
        self._own(h)
        cols = getattr(w, "logical_rows", n)
        if rope is not None:
            q = rope.get("q")
            _native.check(self.lib.configure_resident_fp4_qkv_rope(
                h, _native.ptr(q), 0 if q is None else q.stride(0), rope["cos"].data_ptr(), rope["sin"].data_ptr(),
                rope["cache_k"].data_ptr(), rope["cache_v"].data_ptr(), rope["q_cols"], self.config.head_dim, rope["cache_base"]), name)
            hd = self.config.head_dim
            outs = [StageOutput(name + ".k", "k_cache", rope["cache_k"], rows, hd, rope["cache_base"]),
                    StageOutput(name + ".v", "v_cache", rope["cache_v"], rows, hd, rope["cache_base"])]
            if q is not None:
                outs.append(StageOutput(name + ".q", "q_rope", q, rows, rope["q_cols"]))
        elif out_act is not None and out_precision == "nvfp4":
            _native.check(self.lib.configure_resident_fp4_quantized(h, _native.ptr(bias), _native.ptr(residual), target.data.data_ptr(),
                                                                    target.scales.data_ptr(), target.global_scale, activation), name)
            outs = [StageOutput(name, "fp4", target, rows, cols // 2 if activation == 2 else cols)]
        elif out_act is not None:
            # BF16 activation for a BF16 consumer: GELU of the BF16-rounded projection, or the compact GeGLU
            if activation == 2:
                _native.check(self.lib.configure_resident_fp4_bf16(h, None, None, placeholder.data_ptr()), name)
                _native.check(self.lib.configure_dense_geglu(h, target.data_ptr()), name)
            else:
                _native.check(self.lib.configure_resident_fp4_bf16(h, _native.ptr(bias), _native.ptr(residual), target.data_ptr()), name)
                if activation == 1:
                    _native.check(self.lib.configure_dense_gelu(h, act_cols if act_cols is not None else cols), name)
            outs = [StageOutput(name, "bf16", target, rows, cols // 2 if activation == 2 else cols)]
        elif stream is not None:
            copy, sumsq = stream[:2]
            _native.check(self.lib.configure_resident_fp4_stream(h, _native.ptr(bias), _native.ptr(residual), out.data_ptr(),
                                                                 copy.fp4.data.data_ptr(), copy.fp4.scales.data_ptr(),
                                                                 copy.fp4.global_scale, sumsq.data_ptr()), name)
            outs = [StageOutput(name, "bf16", out, rows, cols), StageOutput(name, "fp4", copy.fp4, rows, cols),
                    StageOutput(name, "sumsq", sumsq, rows, n // block_n, head=(block_n,))]
            if len(stream) > 2:
                outs.append(StageOutput(name, "sum", stream[2], rows, n // block_n, head=(block_n,)))
        else:
            _native.check(self.lib.configure_resident_fp4_bf16(h, _native.ptr(bias), _native.ptr(residual), out.data_ptr()), name)
            if dense and residual is not None:
                # the BF16 model rounds the projection before the residual add (OpenPI eager: x + o in BF16)
                _native.check(self.lib.configure_dense_round_before_residual(h), name)
            if head_pad is not None:
                _native.check(self.lib.configure_dense_head_pad(h, head_pad[0], head_pad[1], out.stride(0)), name)
            outs = [StageOutput(name, "bf16", out, rows, cols, head=head_pad)]
        if row_rms is not None:
            sumsq, parts, width, eps = row_rms
            _native.check(self.lib.configure_resident_fp4_row_rms(h, sumsq.data_ptr(), parts, width, float(eps)), name)
        _native.check(self.lib.configure_resident_fp4_rows(h, rows), name)
        if block_n != 128:
            _native.check(self.lib.configure_resident_fp4_tile(h, block_n), name)
        if (block_n == 32) != (getattr(w, "scale_tile", 128) == 32):
            raise ValueError(f"{name}: 32-wide tiles read weight scales laid out per tile, and only they do")
        if getattr(w, "tiled", 0):
            if w.tiled != block_n:
                raise ValueError(f"{name}: weight tiled for {w.tiled}-wide tiles, used with {block_n}")
            _native.check(self.lib.configure_resident_fp4_weight_layout(h, 1), name)
        if stream is not None and len(stream) > 2:
            _native.check(self.lib.configure_resident_fp4_stream_sums(h, stream[2].data_ptr(), stream[1].shape[1]), name)
        if row_ln is not None:
            sumsq, sums, width, eps, center = row_ln
            _native.check(self.lib.configure_resident_fp4_row_layernorm(h, sumsq.data_ptr(), sums.data_ptr(), sumsq.shape[1], width,
                                                                        float(eps), center.data_ptr()), name)
        return self.add(0, h, name, sources, outs)

    def norm(self, name, x, out: Activation, *, rows, sources, kind, gamma=None, beta=None, eps=1e-6):
        """LayerNorm / RMSNorm / plain quantiser stage writing every form of ``out`` that exists (NVFP4 and / or BF16)."""
        h = C.c_void_p()
        width = x.shape[1]
        if out.fp4 is not None:
            _native.check(self.lib.create_norm(C.byref(h), x.data_ptr(), None, _native.ptr(gamma), _native.ptr(beta), None, None,
                                               out.fp4.data.data_ptr(), out.fp4.scales.data_ptr(), rows, width, self.workers, 0, 4,
                                               int(kind == "layer"), 1, 1, 0, float(eps), out.fp4.global_scale), name)
            outs = [StageOutput(name, "fp4", out.fp4, rows, width)]
        else:
            _native.check(self.lib.create_norm(C.byref(h), x.data_ptr(), None, _native.ptr(gamma), _native.ptr(beta), None, None,
                                               out.bf16.data_ptr(), None, rows, width, self.workers, 0, 16,
                                               int(kind == "layer"), 1, 1, 0, float(eps), 1.0), name)
            outs = [StageOutput(name, "bf16", out.bf16, rows, width)]
        self._own(h)
        if kind == "none":
            _native.check(self.lib.configure_norm_quantize_only(h, 0), name)
        if out.fp4 is not None and out.bf16 is not None:
            _native.check(self.lib.configure_norm_bf16_copy(h, out.bf16.data_ptr()), name)
            outs.append(StageOutput(name, "bf16", out.bf16, rows, width))
        return self.add(2, h, name, sources, outs)

    def linear32(self, name, x, w, bias, out, *, rows, sources, ldx=None, x_bf16=False, out_bf16=False, silu=False,
                 rms=False, euler=False, prev=None, slot=0, prev_slot=0, x_row_offset=0, dt=0.0, eps=1e-6):
        h = C.c_void_p()
        n, k = w.shape
        flags = int(x_bf16) | int(out_bf16) << 1 | int(silu) << 2 | int(rms) << 3 | int(euler) << 4
        _native.check(self.lib.create_linear32(C.byref(h), _native.ptr(x), w.data_ptr(), _native.ptr(bias), _native.ptr(prev),
                                               out.data_ptr(), rows, n, k, ldx if ldx is not None else k, out.stride(0), flags,
                                               slot, prev_slot, x_row_offset, float(dt), float(eps), self.workers), name)
        self._own(h)
        return self.add(3, h, name, sources, [StageOutput(name, "bf16" if out_bf16 else "f32", out, rows, n)])

    # ------------------------------------------------------------------------------------------ tables
    def rope(self, rows, offset):
        hd = self.config.head_dim
        inv = 1.0 / (self.config.rope_base ** (torch.arange(0, hd, 2, dtype=torch.float32, device=self.device) / hd))
        inv = inv.to(self.rope_inv_freq_dtype).float()
        pos = torch.arange(offset, offset + rows, device=self.device, dtype=torch.float32)
        freqs = pos[:, None] * inv[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        rows_pad = padded(rows, 128)
        cos = torch.zeros((rows_pad, hd), device=self.device, dtype=torch.bfloat16)
        sin = torch.zeros_like(cos)
        cos[:rows] = emb.cos().to(torch.bfloat16)
        sin[:rows] = emb.sin().to(torch.bfloat16)
        self.buffers.extend((cos, sin))
        return cos, sin

    def _interleave_heads(self, w):
        """Reorder the rows of a Q or K projection so rotate-half partners (i, i + hd/2) become adjacent."""
        hd = self.config.head_dim
        idx = torch.stack((torch.arange(hd // 2), torch.arange(hd // 2) + hd // 2), dim=1).reshape(-1).to(w.device)
        heads = w.shape[0] // hd
        return w.reshape(heads, hd, -1)[:, idx, :].reshape(w.shape)

    # ------------------------------------------------------------------------------------------ blocks
    def _vision(self):
        c, sd, lib = self.config, self.sd, self.lib
        V, W = self.num_views, c.vision_width
        M = V * 256
        hd = W // c.vision_heads
        patch_w = sd[VISION + "embeddings.patch_embedding.weight"].float().permute(2, 3, 1, 0).reshape(588, W).contiguous()
        patch_b = sd[VISION + "embeddings.patch_embedding.bias"].float().contiguous()
        pos = sd[VISION + "embeddings.position_embedding.weight"].float().contiguous()
        self.buffers.extend((patch_w, patch_b, pos))
        xa, xb = self.tensor((M, W)), self.tensor((M, W))
        h = C.c_void_p()
        _native.check(lib.create_patch_embed(C.byref(h), None, patch_w.data_ptr(), patch_b.data_ptr(), pos.data_ptr(), xa.data_ptr(),
                                             V, W, self.workers), "patch embedding")
        self._own(h)
        s_x = self.add(3, h, "vision.patch", (), [StageOutput("vision.patch", "bf16", xa, M, W)])
        self.mark("patch", xa)
        mlp_pad = padded(c.vision_mlp, 128)
        a_ln, a_att, a_ln2, a_h = Activation(self, M, W), Activation(self, M, W), Activation(self, M, W), Activation(self, M, mlp_pad)
        # Q | K | V with every 72-wide head on a 128-element pitch (zeros between): full 128-byte chunks for the TMA boxes of
        # the tensor-core attention tiles; with the mma.sync tiles the heads are adjacent
        padded_heads = self.attention_path != "mma.sync"
        pitch = 128 if padded_heads else hd
        WP = c.vision_heads * pitch
        qkv = [self.tensor((M, 3 * WP)), self.tensor((M, 3 * WP))]
        a_att.bf16 = self.tensor((M, W))                    # the attention stage always writes BF16 rows
        att = a_att.bf16
        # NVFP4 rows for the output projection straight from the tensor-core attention tiles: every head on a pitch of 80
        # columns (the next multiple of the 16-element scale block), the projection's weight with zero columns to match
        # the projections back to the 1152-wide stream have 9 column tiles of 128 per row band - 54 tiles for 148 workers: 64-wide
        # tiles double the workers that share their weight stream
        narrow = lambda precision: self.vision_block_n if precision == "nvfp4" else 128
        fp4_pitch = padded(hd, 16)
        a_att_fp4 = Activation(self, M, c.vision_heads * fp4_pitch)

        def spread_heads(w):
            wide = torch.zeros((w.shape[0], c.vision_heads, fp4_pitch), device=w.device, dtype=w.dtype)
            wide[:, :, :hd] = w.view(w.shape[0], c.vision_heads, hd)
            return wide.view(w.shape[0], -1)
        # Folded LayerNorms (``fold_norms`` and ``fold_layernorms``, NVFP4 sites): the projection in front of a norm (out, fc2)
        # also leaves the NVFP4 copy of its un-normalised rows and per-tile sums and sums of squares; the projection behind
        # it (fc1, the next layer's q|k|v) carries gamma in its weight columns and ``bias + W beta`` as bias, and centres and
        # scales its accumulator rows.  The first layer's norm reads the patch embedding and stays a stage.
        fold_ln = self.fold_norms and self.fold_layernorms
        slots = padded(W // self.vision_block_n, 4)          # statistics slots per row: one per column tile, padded to a multiple of 4
        stats = lambda key: self.cached((key, M, slots), lambda: self.tensor((M, slots), torch.float32))

        def folded(weight, bias, gamma, beta, rows_pad=None):
            """(gamma in the columns, bias + W beta in BF16 padded to rows_pad) of a projection behind a folded LayerNorm."""
            w = weight.to(torch.bfloat16).float()
            shifted = bias.float() + w @ beta
            out = torch.zeros(rows_pad or shifted.numel(), device=self.device, dtype=torch.bfloat16)
            out[:shifted.numel()] = shifted.to(torch.bfloat16)
            return (w * gamma[None, :]).to(torch.bfloat16), out

        fold1 = False                                        # this layer's first norm is folded (decided by the layer before)
        for i in range(c.vision_layers):
            p = f"{VISION}encoder.layers.{i}."
            p_qkv, p_out, p_fc1, p_fc2 = [self.site(f"vision.{i}.{n}") for n in ("qkv", "out", "fc1", "fc2")]
            g1, b1 = sd[p + "layer_norm1.weight"].float().contiguous(), sd[p + "layer_norm1.bias"].float().contiguous()
            g2, b2 = sd[p + "layer_norm2.weight"].float().contiguous(), sd[p + "layer_norm2.bias"].float().contiguous()
            fold2 = fold_ln and p_out == "nvfp4" and p_fc1 == "nvfp4"
            fold1_next = fold_ln and p_fc2 == "nvfp4" and i + 1 < c.vision_layers and self.site(f"vision.{i + 1}.qkv") == "nvfp4"
            w_qkv_raw = lambda: torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"])
            b_qkv_raw = torch.cat([sd[p + f"self_attn.{n}_proj.bias"] for n in "qkv"])
            if fold1:
                wqkv = self.cached(p + "qkv.nvfp4.ln", lambda: self.weight(folded(w_qkv_raw(), b_qkv_raw, g1, b1)[0], row_sums=True))
                bqkv = folded(w_qkv_raw(), b_qkv_raw, g1, b1)[1]
            else:
                wqkv = self.cached(p + "qkv." + p_qkv, lambda: self.weight(w_qkv_raw(), precision=p_qkv))
                bqkv = b_qkv_raw.to(torch.bfloat16).contiguous()
            quant_in_tile = padded_heads and p_out == "nvfp4"
            if quant_in_tile:
                wo = self.cached(p + "out.nvfp4.spread", lambda: self.weight(spread_heads(sd[p + "self_attn.out_proj.weight"]), block_n=narrow("nvfp4")))
            else:
                wo = self.cached(p + "out." + p_out, lambda: self.weight(sd[p + "self_attn.out_proj.weight"], block_n=narrow(p_out), precision=p_out))
            bo = sd[p + "self_attn.out_proj.bias"].to(torch.bfloat16).contiguous()
            if fold2:
                w1 = self.cached(p + "fc1.nvfp4.ln", lambda: self.weight(folded(sd[p + "mlp.fc1.weight"], sd[p + "mlp.fc1.bias"], g2, b2)[0], row_sums=True))
                bias1 = folded(sd[p + "mlp.fc1.weight"], sd[p + "mlp.fc1.bias"], g2, b2, mlp_pad)[1]
            else:
                w1 = self.cached(p + "fc1." + p_fc1, lambda: self.weight(sd[p + "mlp.fc1.weight"], precision=p_fc1))
                bias1 = torch.zeros(mlp_pad, device=self.device, dtype=torch.bfloat16)
                bias1[:c.vision_mlp] = sd[p + "mlp.fc1.bias"].to(torch.bfloat16)
            w2 = self.cached(p + "fc2." + p_fc2, lambda: self.weight(sd[p + "mlp.fc2.weight"], block_n=narrow(p_fc2), precision=p_fc2))
            bias2 = sd[p + "mlp.fc2.bias"].to(torch.bfloat16).contiguous()
            self.buffers.extend((g1, b1, g2, b2, bqkv, bo, bias1, bias2))
            buf = qkv[i & 1]
            if fold1:
                s_ln, ln1 = s_x, (stats("vision.sumsq1"), stats("vision.sum1"), W, c.ln_eps, wqkv.row_sums)
            else:
                s_ln, ln1 = self.norm(f"vision.{i}.ln1", xa, a_ln.only(p_qkv), rows=M, sources=[(s_x, SAME)], kind="layer", gamma=g1,
                                      beta=b1, eps=c.ln_eps), None
            s_qkv = self.gemm(f"vision.{i}.qkv", a_ln, wqkv, rows=M, sources=[(s_ln, SAME)], out=buf, bias=bqkv,
                              head_pad=(hd, pitch) if padded_heads else None, row_ln=ln1)
            h = C.c_void_p()
            q, k, v = buf[:, :WP], buf[:, WP:2 * WP], buf[:, 2 * WP:]
            _native.check(lib.create_attention(C.byref(h), q.data_ptr(), k.data_ptr(), v.data_ptr(), None, None, None, None, None,
                                               None, None, att.data_ptr(), None, V, 256, 256, c.vision_heads, c.vision_heads, hd,
                                               3 * WP, 3 * WP, W, 0, self.workers, -1, float(hd ** -0.5)), "vision attention")
            self._own(h)
            if padded_heads:
                _native.check(lib.configure_attention_head_pad(h, pitch), "vision attention")
            outs = [StageOutput(f"vision.{i}.attention", "bf16", att, M, W)]
            if quant_in_tile:
                fp4 = a_att_fp4.require("nvfp4").fp4
                _native.check(lib.configure_attention_fp4_pitch(h, fp4_pitch), "vision attention")
                _native.check(lib.configure_attention_fp4_output(h, fp4.data.data_ptr(), fp4.scales.data_ptr(), fp4.data.stride(0),
                                                                 fp4.k // 16, fp4.global_scale), "vision attention")
                outs.append(StageOutput(f"vision.{i}.attention", "fp4", fp4, M, c.vision_heads * fp4_pitch, head=(hd, fp4_pitch)))
            self._attention_path(h, "vision attention")
            s_att = self.add(1, h, f"vision.{i}.attention", [(s_qkv, ALL)], outs)
            if p_out == "nvfp4" and not quant_in_tile:
                # the mma.sync tiles do not quantise 72-wide heads: a quantiser stage of its own
                s_att = self.norm(f"vision.{i}.attention_quant", att, a_att.only("nvfp4"), rows=M, sources=[(s_att, SAME)], kind="none")
            s_o = self.gemm(f"vision.{i}.out", a_att_fp4 if quant_in_tile else a_att, wo, rows=M, sources=[(s_att, SAME)], out=xb,
                            bias=bo, residual=xa, block_n=narrow(p_out),
                            stream=(a_ln2.require("nvfp4"), stats("vision.sumsq2"), stats("vision.sum2")) if fold2 else None)
            if fold2:
                s_ln2, ln2 = s_o, (stats("vision.sumsq2"), stats("vision.sum2"), W, c.ln_eps, w1.row_sums)
            else:
                s_ln2, ln2 = self.norm(f"vision.{i}.ln2", xb, a_ln2.only(p_fc1), rows=M, sources=[(s_o, SAME)], kind="layer", gamma=g2,
                                       beta=b2, eps=c.ln_eps), None
            s_fc1 = self.gemm(f"vision.{i}.fc1", a_ln2, w1, rows=M, sources=[(s_ln2, SAME)], out_act=a_h.require(p_fc2), out_precision=p_fc2,
                              bias=bias1, activation=1, act_cols=c.vision_mlp, row_ln=ln2)
            s_x = self.gemm(f"vision.{i}.fc2", a_h, w2, rows=M, sources=[(s_fc1, SAME)], out=xa, bias=bias2, residual=xb,
                            block_n=narrow(p_fc2),
                            stream=(a_ln.require("nvfp4"), stats("vision.sumsq1"), stats("vision.sum1")) if fold1_next else None)
            fold1 = fold1_next
            if i == 0:
                self.mark("vision.0.qkv", buf), self.mark("vision.0.attention", att)
            self.mark(f"vision.{i}", xa)
            if self.verbose and (i + 1) % 9 == 0:
                print("NativePi0: vision layers", i + 1, flush=True)
        gp, bp = sd[VISION + "post_layernorm.weight"].float().contiguous(), sd[VISION + "post_layernorm.bias"].float().contiguous()
        self.buffers.extend((gp, bp))
        p_proj = self.site("vision.projector")
        a_post = a_ln.only(p_proj)
        s_pl = self.norm("vision.post_layernorm", xa, a_post, rows=M, sources=[(s_x, SAME)], kind="layer", gamma=gp, beta=bp, eps=c.ln_eps)
        return s_pl, a_post

    def _expert_splits(self, keys):
        """KV splits of the expert attention: as many as leave every tile a worker of its own that did NOT run a tile
        of the QKV projection in front of it (such a worker starts 2-3 microseconds late), at most 16 and at least
        32 keys per split."""
        if self.expert_splits is not None:
            return int(self.expert_splits)
        c = self.config
        width = self.expert_block_n["qkv"] if isinstance(self.expert_block_n, dict) else self.expert_block_n
        qkv_tiles = -(-(c.heads + 2) * c.head_dim // width)
        return max(1, min(16, (self.workers - qkv_tiles) // c.heads, keys // 32))

    def _prefix_splits(self, rows):
        """KV splits of the prefix attention.  The tensor-core tiles hold at most 256 keys, so the split count is
        ceil(rows / 256); with the mma.sync tiles: as many as keep every tile of the stage on a worker of its own, at
        most four.  Returns (splits, fused): the merge runs inside the attention stage (the tiles of a head meet on a
        ticket) only when every tile has a worker of its own, otherwise as a stage behind it."""
        groups = -(-rows // 128) * self.config.heads
        if self.prefix_splits is not None:
            splits = int(self.prefix_splits)
        elif self.attention_path == "mma.sync":
            splits = max(1, min(4, self.workers // groups))
        else:
            splits = -(-rows // 256)
        return splits, splits > 1 and groups * splits <= self.workers

    def _attention_path(self, handle, name):
        if self.attention_path is not None:
            _native.check(self.lib.configure_attention_path(handle, int(self.attention_path == "tcgen05")), name)

    def _gemma_layer(self, name, site, prefix, i, x_in, x_mid, bufs, *, rows, s_x, extra_sources, cos, sin, cache, cache_base,
                     attention_rows, mask_prefix, splits, kv_only, block_n, prefix_cache_stage=None, streamed_in=None,
                     next_site=None):
        """One Gemma decoder layer.  ``name`` labels the stages (``expert.<step>.<layer>``), ``site`` the weights
        (``expert.<layer>``: one operand format for all Euler steps).

        Folded norms (``fold_norms``, NVFP4 sites): an RMSNorm between two NVFP4 projections is not a stage.  The
        producing projection (o_proj, down) also writes the NVFP4 copy of its un-normalised BF16 rows and per-tile
        sums of their squares; the consuming projection (gate/up, the next layer's QKV), whose weight columns carry
        ``1 + w`` of the norm, multiplies every accumulator row by ``rsqrt(mean square + eps)``.  ``streamed_in`` is
        the ``(sumsq, parts)`` left by the previous layer's down projection (None: this layer runs its input norm);
        ``next_site`` names the layer that follows, whose QKV projection decides whether this layer's down projection
        streams.  Returns (last stage, KV stage, streamed_out)."""
        c, sd, lib = self.config, self.sd, self.lib
        p = f"{prefix}layers.{i}."
        width = x_in.shape[1]
        H, hd = c.heads, c.head_dim
        a1, a2, a3, a4, qbuf = bufs
        p_qkv, p_o, p_gu, p_dn = [self.site(f"{site}.{n}") for n in ("qkv", "o_proj", "gate_up", "down")]
        widths = block_n if isinstance(block_n, dict) else dict.fromkeys(("qkv", "o_proj", "gate_up", "down"), block_n)
        p_of = dict(zip(("qkv", "o_proj", "gate_up", "down"), (p_qkv, p_o, p_gu, p_dn)))
        tile = lambda op: widths[op] if p_of[op] == "nvfp4" else 128            # BF16 sites use full-width tiles
        sums = lambda key, parts: self.cached((key, x_in.shape[0], parts), lambda: self.tensor((x_in.shape[0], parts), torch.float32))
        gamma1 = lambda: (1.0 + sd[p + "input_layernorm.weight"].float()).contiguous()
        if streamed_in is None:
            g1 = self.cached(p + "g1", gamma1)
            s_n1 = self.norm(f"{name}.norm1", x_in, a1.only(p_qkv), rows=rows, sources=[(s_x, SAME)] + extra_sources, kind="rms", gamma=g1, eps=c.rms_eps)
            fold1 = None
        else:
            s_n1, fold1 = s_x, (streamed_in[0], streamed_in[1], width, c.rms_eps)
        def make_qkv():
            wk = self._interleave_heads(sd[p + "self_attn.k_proj.weight"])
            wv = sd[p + "self_attn.v_proj.weight"]
            w = torch.cat((wk, wv)) if kv_only else torch.cat((self._interleave_heads(sd[p + "self_attn.q_proj.weight"]), wk, wv))
            if fold1 is not None:
                w = w.float() * gamma1()[None, :]
            return self.weight(w, block_n=tile("qkv"), precision=p_qkv)

        wqkv = self.cached(f"{p}qkv.{p_qkv}.{int(fold1 is not None)}.{int(kv_only)}.{tile("qkv")}", make_qkv)
        q_cols, q = (0, None) if kv_only else (H * hd, qbuf)
        s_qkv = self.gemm(f"{name}.qkv", a1, wqkv, rows=rows, sources=[(s_n1, SAME)], block_n=tile("qkv"), row_rms=fold1,
                          rope=dict(q=q, cos=cos, sin=sin, cache_k=cache[0], cache_v=cache[1], q_cols=q_cols, cache_base=cache_base))
        if kv_only:
            return s_qkv, s_qkv, None
        attn_out = a2.bf16
        h = C.c_void_p()
        _native.check(lib.create_attention(C.byref(h), qbuf.data_ptr(), cache[0].data_ptr(), cache[1].data_ptr(), None, None, None,
                                           None, None, None, None, attn_out.data_ptr(), None, 1, rows, attention_rows, H, 1, hd,
                                           H * hd, hd, H * hd, 0, self.workers, mask_prefix, float(hd ** -0.5)), f"{name}.attention")
        self._own(h)
        outs = [StageOutput(f"{name}.attention", "bf16", attn_out, rows, H * hd)]
        if p_o == "nvfp4":
            fp4 = a2.require("nvfp4").fp4
            _native.check(lib.configure_attention_fp4_output(h, fp4.data.data_ptr(), fp4.scales.data_ptr(), fp4.data.stride(0),
                                                             fp4.k // 16, fp4.global_scale), f"{name}.attention")
            outs.append(StageOutput(f"{name}.attention", "fp4", fp4, rows, H * hd))
        att_sources = [(s_qkv, ALL)] + ([(prefix_cache_stage, ALL)] if prefix_cache_stage is not None else [])
        splits, fused = splits if isinstance(splits, tuple) else (splits, splits > 1)
        if splits > 1:
            _native.check(lib.configure_attention_splits(h, splits), f"{name}.attention")
            if fused:
                # the merge inside the attention stage: the tiles of a head meet on a ticket and each merges its share of rows
                _native.check(lib.configure_attention_fused_merge(h, 1), f"{name}.attention")
        self._attention_path(h, f"{name}.attention")
        if splits > 1 and not fused:
            # more tiles than workers: partial rows first, the merge as a stage of its own behind them
            s_part = self.add(1, h, f"{name}.attention_tiles", att_sources)
            merge = C.c_void_p()
            _native.check(lib.attention_merge_handle(h, C.byref(merge)), f"{name}.attention")
            s_att = self.add(4, merge, f"{name}.attention", [(s_part, ALL)], outs)
        else:
            s_att = self.add(1, h, f"{name}.attention", att_sources, outs)
        wo = self.cached(f"{p}o.{p_o}.{tile("o_proj")}", lambda: self.weight(sd[p + "self_attn.o_proj.weight"], block_n=tile("o_proj"), precision=p_o))
        # ---- attention output projection; the post-attention norm is folded when both neighbours are NVFP4 sites
        fold2 = self.fold_norms and p_o == "nvfp4" and p_gu == "nvfp4"
        gamma2 = lambda: (1.0 + sd[p + "post_attention_layernorm.weight"].float()).contiguous()
        if fold2:
            parts2 = width // tile("o_proj")
            ss2 = sums("sumsq2", parts2)
            s_o = self.gemm(f"{name}.o_proj", a2, wo, rows=rows, sources=[(s_att, SAME)], out=x_mid, residual=x_in, block_n=tile("o_proj"),
                            stream=(a3.require("nvfp4"), ss2))
            s_n2, rms2 = s_o, (ss2, parts2, width, c.rms_eps)
        else:
            s_o = self.gemm(f"{name}.o_proj", a2, wo, rows=rows, sources=[(s_att, SAME)], out=x_mid, residual=x_in, block_n=tile("o_proj"))
            g2 = self.cached(p + "g2", gamma2)
            s_n2 = self.norm(f"{name}.norm2", x_mid, a3.only(p_gu), rows=rows, sources=[(s_o, SAME)], kind="rms", gamma=g2, eps=c.rms_eps)
            rms2 = None
        def make_gate_up():
            gate, up = sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]
            w = torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], gate.shape[1])
            if fold2:
                w = w.float() * gamma2()[None, :]
            return self.weight(w, block_n=tile("gate_up"), precision=p_gu)

        wgu = self.cached(f"{p}gate_up.{p_gu}.{int(fold2)}.{tile("gate_up")}", make_gate_up)
        s_gu = self.gemm(f"{name}.gate_up", a3, wgu, rows=rows, sources=[(s_n2, SAME)], out_act=a4.require(p_dn), out_precision=p_dn,
                         activation=2, block_n=tile("gate_up"), row_rms=rms2)
        wd = self.cached(f"{p}down.{p_dn}.{tile("down")}", lambda: self.weight(sd[p + "mlp.down_proj.weight"], block_n=tile("down"), precision=p_dn))
        # ---- down projection; streams for the next layer's QKV when that reads NVFP4 too
        streamed_out = None
        if self.fold_norms and next_site is not None and p_dn == "nvfp4" and self.site(f"{next_site}.qkv") == "nvfp4":
            parts1 = width // tile("down")
            ss1 = sums("sumsq1", parts1)
            s_dn = self.gemm(f"{name}.down", a4, wd, rows=rows, sources=[(s_gu, SAME)], out=x_in, residual=x_mid, block_n=tile("down"),
                             stream=(a1.require("nvfp4"), ss1))
            streamed_out = (ss1, parts1)
        else:
            s_dn = self.gemm(f"{name}.down", a4, wd, rows=rows, sources=[(s_gu, SAME)], out=x_in, residual=x_mid, block_n=tile("down"))
        return s_dn, s_qkv, streamed_out

    def _build(self):
        c, sd, lib = self.config, self.sd, self.lib
        V = self.num_views
        P = V * 256 + self.prompt_len
        P_pad = padded(P, 128)
        S = self.chunk_size + 1
        S_pad = 128
        H, hd = c.heads, c.head_dim
        # ---------------- vision tower + projector -> prefix rows [0, V*256)
        s_pl, a_post = self._vision()
        x_a, x_b = self.tensor((P_pad, c.width)), self.tensor((P_pad, c.width))
        wproj = self.cached(PROJECTOR + self.site("vision.projector"), lambda: self.weight(sd[PROJECTOR + "weight"], precision=self.site("vision.projector")))
        bproj = sd[PROJECTOR + "bias"].to(torch.bfloat16).contiguous()
        self.buffers.append(bproj)
        s_x = self.gemm("vision.projector", a_post, wproj, rows=V * 256, sources=[(s_pl, SAME)], out=x_a, bias=bproj)
        self.mark("image_tokens", x_a)
        vision_end = len(self.stages)
        # ---------------- Gemma-2B prefix: builds the KV cache
        extra = []
        if self.prompt_len:
            table = sd[LANGUAGE + "embed_tokens.weight"]
            if table.dtype != torch.bfloat16:
                table = table.to(torch.bfloat16)
            table = table.contiguous()
            self.buffers.append(table)
            h = C.c_void_p()
            _native.check(lib.create_token_embed(C.byref(h), None, table.data_ptr(), x_a.data_ptr(), self.prompt_len, c.width,
                                                 V * 256, table.shape[0], float(math.sqrt(c.width)), self.workers), "token embedding")
            self._own(h)
            extra = [(self.add(3, h, "prefix.embed"), ALL)]
        self.mark("prefix.input", x_a)
        cos_p, sin_p = self.rope(P, 0)
        self.caches = [(self.tensor((P + S_pad, hd)), self.tensor((P + S_pad, hd))) for _ in range(c.prefix_layers)]
        bufs = (Activation(self, P_pad, c.width), Activation(self, P_pad, H * hd), Activation(self, P_pad, c.width),
                Activation(self, P_pad, c.mlp), self.tensor((P_pad, H * hd)))
        bufs[1].bf16 = self.tensor((P_pad, H * hd))          # attention output rows (BF16), always written
        cache_stage, streamed = [], None
        for i in range(c.prefix_layers):
            s_x, s_kv, streamed = self._gemma_layer(
                f"prefix.{i}", f"prefix.{i}", LANGUAGE, i, x_a, x_b, bufs, rows=P, s_x=s_x, extra_sources=extra if i == 0 else [],
                cos=cos_p, sin=sin_p, cache=self.caches[i], cache_base=0, attention_rows=P, mask_prefix=-1,
                splits=self._prefix_splits(P), kv_only=(i == c.prefix_layers - 1), block_n=128, streamed_in=streamed,
                next_site=f"prefix.{i + 1}" if i + 1 < c.prefix_layers else None)
            cache_stage.append(s_kv)
            if i == 0:
                self.mark("prefix.0.q", bufs[4]), self.mark("prefix.0.attention", bufs[1].bf16)
            self.mark(f"prefix.{i}", x_a)
            if self.verbose and (i + 1) % 6 == 0:
                print("NativePi0: prefix layers", i + 1, flush=True)
        prefix_end = len(self.stages)
        # ---------------- action expert, flow_steps Euler updates
        W = c.expert_width
        f32 = lambda t: t.float().contiguous()
        w_state, b_state = f32(sd["state_proj.weight"]), f32(sd["state_proj.bias"])
        w_in, b_in = f32(sd["action_in_proj.weight"]), f32(sd["action_in_proj.bias"])
        w_t1, b_t1 = f32(sd["action_time_mlp_in.weight"]), f32(sd["action_time_mlp_in.bias"])
        w_t2, b_t2 = f32(sd["action_time_mlp_out.weight"]), f32(sd["action_time_mlp_out.bias"])
        # action half of the first time-MLP layer folded into the action projection:
        # W_a (W_in x + b_in) = (W_a W_in) x + W_a b_in; the time half is a per-step bias.
        w_fused = (w_t1[:, :W] @ w_in).contiguous()
        b_fused = w_t1[:, :W] @ b_in
        final_w = (f32(sd["action_out_proj.weight"]) * (1.0 + f32(sd[EXPERT + "norm.weight"]))[None, :]).contiguous()
        final_b = f32(sd["action_out_proj.bias"])
        self.buffers.extend((w_state, b_state, w_fused, w_t2, b_t2, final_w, final_b))
        state_emb = self.tensor((1, W), torch.float32)
        s_state = self.linear32("expert.state", None, w_state, b_state, state_emb, rows=1, sources=[], slot=2)
        h1 = self.tensor((self.chunk_size, W), torch.float32)
        actions = self.tensor((self.chunk_size, c.action_dim), torch.float32)
        xe_a, xe_b = self.tensor((S_pad, W)), self.tensor((S_pad, W))
        cos_s, sin_s = self.rope(S, P)
        ebufs = (Activation(self, S_pad, W), Activation(self, S_pad, H * hd), Activation(self, S_pad, W),
                 Activation(self, S_pad, c.expert_mlp), self.tensor((S_pad, H * hd)))
        ebufs[1].bf16 = self.tensor((S_pad, H * hd))
        time, dt = np.float32(1.0), np.float32(-1.0 / self.flow_steps)
        s_prev = None
        for step in range(self.flow_steps):
            fraction = torch.linspace(0.0, 1.0, W // 2, device=self.device, dtype=torch.float64)
            period = 0.004 * (4.0 / 0.004) ** fraction
            angle = float(time) / period * (2.0 * math.pi)
            t_emb = torch.cat((angle.sin(), angle.cos())).float()
            step_bias = (b_fused + w_t1[:, W:] @ t_emb + b_t1).contiguous()
            self.buffers.append(step_bias)
            first = step == 0
            s_t1 = self.linear32(f"expert.{step}.time_in", None if first else actions, w_fused, step_bias, h1, rows=self.chunk_size,
                                 sources=[(s_prev, ALL)], slot=3 if first else 0, silu=True)
            # time_out writes the action tokens as BF16 rows 1.. of the expert input; its first tiles add row 0 (the state token)
            s_x = self.linear32(f"expert.{step}.time_out", h1, w_t2, b_t2, xe_a[1:], rows=self.chunk_size,
                                sources=[(s_t1, ALL), (s_state, ALL)], out_bf16=True)
            _native.check(lib.configure_linear32_extra_row(self.handles[-1], state_emb.data_ptr(), xe_a.data_ptr()), "state row")
            self.mark(f"expert.{step}.input", xe_a)
            streamed = None
            for i in range(c.expert_layers):
                s_x, _, streamed = self._expert_layer(step, i, xe_a, xe_b, ebufs, S, P, s_x, cos_s, sin_s, cache_stage[i], streamed)
                self.mark(f"expert.{step}.{i}", xe_a)
            s_prev = self.linear32(f"expert.{step}.euler", xe_a, final_w, final_b, actions, rows=self.chunk_size, sources=[(s_x, ALL)],
                                   ldx=W, x_bf16=True, rms=True, euler=True, prev=None if first else actions,
                                   prev_slot=3 if first else 0, x_row_offset=1, dt=float(dt), eps=c.rms_eps)
            self.mark(f"actions.{step}", actions)
            time = np.float32(time + dt)
            if self.verbose:
                print("NativePi0: expert denoising step", step + 1, "wired", flush=True)
        self.output = actions.view(1, self.chunk_size, c.action_dim)
        self.component_ranges = {"vision": (0, vision_end), "prefix": (vision_end, prefix_end), "expert": (prefix_end, len(self.stages))}
        # ---------------- static instruction streams + program
        work = [LinearWork(t, k) for t, k in zip(self.stage_tiles, self.stage_cost)]
        if self.schedule in ("spread", "affine"):
            # "affine": workers also keep to the kinds of instruction they have run before (the stage name's last component)
            kinds = [n.rsplit(".", 1)[-1] for n in self.stage_names] if self.schedule == "affine" else None
            self.code = spread_streams(work, self.workers, [[s for s in spec.sources] for spec in self.stages], kinds)
        else:
            self.code = linear_streams(work, self.workers)
        validate_streams(self.code, self.stage_tiles)
        self.plan = program_summary(self.code)
        self.plan["stages"] = len(self.stages)
        specs = (NativeSpec * len(self.stages))(*self.stages)
        _native.check(lib.create_native_model(C.byref(self.handle), len(specs), C.cast(specs, C.c_void_p), self.code.ctypes.data,
                                              self.workers, self.code.shape[1]), "Native pi0 setup")
        lean = C.c_int()
        _native.check(lib.native_model_kernel_variant(self.handle, C.byref(lean)), "Native pi0 setup")
        self.plan["kernel"] = "lean" if lean.value else "full"      # which variant of the persistent kernel the program launches
        if self.verbose:
            print("NativePi0 static program:", self.plan, flush=True)

    def _expert_layer(self, step, i, x_in, x_mid, bufs, S, P, s_x, cos, sin, prefix_cache_stage, streamed):
        """Every Euler step wires its own stages; the NVFP4 weights are shared through the keyed weight cache."""
        last = i + 1 == self.config.expert_layers
        return self._gemma_layer(f"expert.{step}.{i}", f"expert.{i}", EXPERT, i, x_in, x_mid, bufs, rows=S, s_x=s_x, extra_sources=[], cos=cos, sin=sin,
                                 cache=self.caches[i], cache_base=P, attention_rows=P + S, mask_prefix=P, splits=self._expert_splits(P + S),
                                 kv_only=False, block_n=self.expert_block_n, prefix_cache_stage=prefix_cache_stage, streamed_in=streamed,
                                 next_site=None if last else f"expert.{i + 1}")

    # ------------------------------------------------------------------------------------------ running
    def _check_inputs(self, images, state, noise, tokens):
        if not self.handle.value:
            raise RuntimeError("Native pi0 engine is closed")
        wanted = ((images, (self.num_views, 224, 224, 3), torch.float32), (state, (1, self.config.action_dim), torch.float32),
                  (noise, (1, self.chunk_size, self.config.action_dim), torch.float32), (tokens, (1, self.prompt_len), torch.int64))
        for t, shape, dtype in wanted:
            if t.device != self.device or t.dtype != dtype or tuple(t.shape) != shape or not t.is_contiguous():
                raise ValueError(("Resident pi0 input layout", shape, dtype))

    def forward(self, images, state, noise, tokens):
        """One action chunk.  Inputs are CUDA-resident and contiguous; the returned tensor is reused by the next call."""
        self._check_inputs(images, state, noise, tokens)
        if self.partitioned:
            for n, name in enumerate(("vision", "prefix", "expert")):
                self.launch_component(name, images, state, noise, tokens, new_epoch=(n == 0))
        else:
            self.launch_component(None, images, state, noise, tokens)
        self.epoch += 1
        return self.output

    def sample_actions(self, images, state, noise, tokens=None):
        """Host-facing call: inputs are CPU tensors (pinned memory avoids a staging copy); they are copied to
        resident device buffers, one forward pass runs, and the action chunk comes back as a CPU FP32 tensor
        ``[1, chunk, action_dim]``.  Equivalent of OpenPI's ``sample_actions`` with caller-supplied noise."""
        if tokens is None:
            tokens = torch.zeros((1, self.prompt_len), dtype=torch.int64)
        if not hasattr(self, "_resident_inputs"):
            with torch.cuda.device(self.device):
                self._resident_inputs = (
                    torch.zeros((self.num_views, 224, 224, 3), dtype=torch.float32, device=self.device),
                    torch.zeros((1, self.config.action_dim), dtype=torch.float32, device=self.device),
                    torch.zeros((1, self.chunk_size, self.config.action_dim), dtype=torch.float32, device=self.device),
                    torch.zeros((1, self.prompt_len), dtype=torch.int64, device=self.device))
                self._host_output = torch.zeros((1, self.chunk_size, self.config.action_dim), dtype=torch.float32).pin_memory()
        for dst, src in zip(self._resident_inputs, (images, state, noise, tokens)):
            if tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype:
                raise ValueError(("pi0 input layout", tuple(dst.shape), dst.dtype))
            dst.copy_(src, non_blocking=True)
        out = self.forward(*self._resident_inputs)
        self._host_output.copy_(out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._host_output

    def launch_component(self, name, images, state, noise, tokens, new_epoch=True):
        begin, end = (0, len(self.stages)) if name is None else self.component_ranges[name]
        self.launch_range(begin, end, images, state, noise, tokens, new_epoch)

    def launch_range(self, begin, end, images, state, noise, tokens, new_epoch):
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            code = self.lib.launch_native_model_range(self.handle, stream, images.data_ptr(), state.data_ptr(), noise.data_ptr(),
                                                      tokens.data_ptr(), begin, end, int(new_epoch))
        if code:
            raise RuntimeError(f"Native pi0 launch error {code}")

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.lib, self.handle)

    def enable_timings(self, enable=True):
        _native.check(self.lib.enable_native_model_timings(self.handle, int(enable)), "timing setup")

    def read_timings(self, name=None):
        """Global-timer stamps (ns) int64 [workers, stream_length, 8] of the last launch with timings enabled: start,
        producers ready, end, copies issued, first operands landed, MMAs issued, first accumulator ready, last stores
        done (the last five only for GEMM and attention instructions)."""
        out = np.zeros((self.workers, self.code.shape[1], 8), dtype=np.int64)
        with torch.cuda.device(self.device):
            _native.check(self.lib.read_native_model_timings(self.handle, out.ctypes.data, out.size), "timing read")
        return out

    def stage_profile(self):
        """Per-stage wall span of the last timed launch: list of (name, ready_ns, end_ns, instructions) where
        ready is the earliest moment a worker had the stage's producers complete and end the last worker's finish,
        relative to the earliest stamp (device global timer).  Call ``enable_timings()`` before the launch."""
        from native_pi0.timing import stage_spans
        return stage_spans(self.read_timings(), self.code, self.stage_names)

    def calibrate(self, calibration, sample, images, state, noise, tokens):
        """Record the |max| of every projection's BF16 output for one observation into an ``ActivationCalibration``:
        the forward runs stage by stage (one launch each) and every BF16 / FP32 stage output is observed under its
        site name, expert stages with their Euler step.  Meant for an engine built with ``precision="bf16"``, whose
        activations are unquantised; ``native_pi0.calibration.site_precisions`` turns the finished record into the
        ``precision`` argument of the serving engine."""
        self._check_inputs(images, state, noise, tokens)
        for s in range(len(self.stages)):
            self.launch_range(s, s + 1, images, state, noise, tokens, new_epoch=(s == 0))
            for out in self.stage_outputs[s]:
                if out.kind not in ("bf16", "f32") or out.head is not None:
                    continue
                parts = out.name.split(".")
                step = None
                if parts[0] == "expert" and len(parts) == 4:          # expert.<step>.<layer>.<operation>
                    step, parts = int(parts[1]), [parts[0]] + parts[2:]
                if len(parts) != 3:
                    continue
                value = float(out.buffer[:out.rows, :out.cols].float().abs().max())
                calibration.observe(".".join(parts), [value], sample=sample, step=step)
        self.epoch += 1
        return calibration

    def operation_report(self):
        """Per phase and operation type: layers, median active workers, median busy time and the chain time of the
        last timed launch (``native_pi0.timing.operation_report``)."""
        from native_pi0.timing import operation_report
        return operation_report(self.read_timings(), self.code, self.stage_names)

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.lib.destroy_native_model(self.handle), "Native pi0 teardown")
            self.handle = C.c_void_p()
        for h in getattr(self, "handles", []):
            if h.value:
                with torch.cuda.device(self.device):
                    self.lib.destroy_op(h)
                h.value = None
        self.handles = []

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


class EngineCache:
    """Engines for several input shapes over one set of packed weights.

    A program is compiled for fixed (views, prompt length, chunk size); a deployment that sees a few shapes keeps one
    engine per shape.  The engines share a ``weight_store``, so every weight is packed and resident once (1.46 GB in
    NVFP4) and an additional shape costs only its activations, KV caches and instruction streams.  At most
    ``capacity`` engines stay alive; the least recently used one is closed when another shape arrives.  The state dict
    is kept for building further shapes.
    """

    def __init__(self, model, *, capacity=4, **engine_options):
        if capacity < 1:
            raise ValueError("capacity >= 1")
        self.model, self.capacity, self.options = model, capacity, dict(engine_options)
        self.weights, self.engines = {}, {}

    def get(self, num_views=3, prompt_len=0, chunk_size=50):
        key = (int(num_views), int(prompt_len), int(chunk_size))
        engine = self.engines.pop(key, None)
        if engine is None:
            while len(self.engines) >= self.capacity:
                oldest = next(iter(self.engines))
                self.engines.pop(oldest).close()
            engine = NativePi0(self.model, num_views=key[0], prompt_len=key[1], chunk_size=key[2], weight_store=self.weights,
                               **self.options)
        self.engines[key] = engine                          # most recently used last
        return engine

    def close(self):
        for engine in self.engines.values():
            engine.close()
        self.engines.clear()
        self.weights.clear()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
