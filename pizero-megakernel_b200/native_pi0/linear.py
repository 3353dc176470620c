"""Chains of NVFP4 projections in one persistent launch with row-band counters.

Counterpart of the reference ``NativeLinearProgram`` (``native_pi0/linear.py:11-73``), which chains BF16
projections; here every stage is a ``ResidentNVFP4`` whose output is packed NVFP4 (feeding the next stage)
or BF16/FP32 (last stage).  ``sources[i] = -1`` reads the stage's own resident activation, otherwise the
packed output of an earlier stage is bound as its A operand.  A tile waits only for its own 128-row band of
the producer.  ``read_counters()`` returns the per-band tile counts against ``tiles * epoch``.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import torch

from native_pi0 import _native
from native_pi0.program import LinearWork, linear_streams, program_summary


class NativeLinearProgram:
    def __init__(self, library, stages, *, sources=None, workers=148):
        self.handle = C.c_void_p()
        self.stages = tuple(stages)
        self.library = _native.load(library)
        self.epoch = 0
        if not self.stages:
            raise ValueError("At least one projection is required")
        self.device = self.stages[0].device
        if len({s.handle.value for s in self.stages}) != len(self.stages):
            raise ValueError("Stages must have distinct handles")
        for s in self.stages:
            if not s.handle.value or s.device != self.device:
                raise ValueError("Projection handles must be live on this device")
        sources = [-1] + list(range(len(self.stages) - 1)) if sources is None else list(sources)
        if len(sources) != len(self.stages) or any(not isinstance(p, int) or p < -1 or p >= i for i, p in enumerate(sources)):
            raise ValueError("Sources must be -1 or an earlier stage")
        for i, parent in enumerate(sources):
            if parent >= 0:
                producer, consumer = self.stages[parent], self.stages[i]
                if producer.output.dtype != torch.uint8 or tuple(producer.output.shape) != tuple(consumer.a.shape):
                    raise ValueError("Producer must emit packed NVFP4 of the consumer's activation shape")
                if producer.output.data_ptr() != consumer.a.data_ptr():
                    raise ValueError("Bind the consumer's activation buffers to the producer's output at construction")
        self.sources = sources
        geometry = []
        for s in self.stages:
            tiles, bands, cost = C.c_int(), C.c_int(), C.c_int()
            _native.check(self.library.op_geometry(s.handle, C.byref(tiles), C.byref(bands), C.byref(cost)), "geometry")
            geometry.append((tiles.value, bands.value, cost.value))
        self.code = linear_streams([LinearWork(t, k) for t, _, k in geometry], workers)
        self.plan = program_summary(self.code)
        self.counter_tiles = np.concatenate([np.full(b, t // b, dtype=np.uint64) for t, b, _ in geometry])
        handles = np.asarray([s.handle.value for s in self.stages], dtype=np.uintp)
        parents = np.asarray(sources, dtype=np.int32)
        with torch.cuda.device(self.device):
            _native.check(self.library.create_native_linear(C.byref(self.handle), len(self.stages), handles.ctypes.data,
                                                            parents.ctypes.data, self.code.ctypes.data, workers,
                                                            self.code.shape[1]), "Native linear setup")
        self.output = self.stages[-1].output

    def forward(self):
        if not self.handle.value or any(not s.handle.value for s in self.stages):
            raise RuntimeError("Native program or child is closed")
        with torch.cuda.device(self.device):
            _native.check(self.library.launch_native_linear(self.handle, torch.cuda.current_stream(self.device).cuda_stream),
                          "Native linear launch")
        self.epoch += 1
        return self.output

    def read_counters(self):
        counters = np.empty(len(self.counter_tiles), dtype=np.uint64)
        epoch = np.zeros(1, dtype=np.uint64)
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            _native.check(self.library.read_native_linear(self.handle, counters.ctypes.data, len(counters), epoch.ctypes.data),
                          "Native counter read")
        return {"counts": counters, "expected": self.counter_tiles * epoch[0], "epoch": int(epoch[0])}

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.library, self.handle)

    def close(self):
        if self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.library.destroy_native_linear(self.handle), "Native linear teardown")
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


class NativeStageProgram:
    """Any operator handles as one persistent launch (extension; the reference chains only dense projections).

    ``stages`` is a list of ``(operator, sources)``: ``operator`` is a wrapper object (``ResidentNVFP4``,
    ``ResidentNorm``, ``ResidentAttention``) and ``sources`` a list of ``(producer_index, mode)`` with mode 0 = wait
    for the producer's tiles of the same 128-row band, 1 = wait for all of them.  The caller binds the buffers
    (a consumer reads what its producer writes); the program only adds the ordering.
    """
    _KIND = {"ResidentNVFP4": 0, "ResidentDense": 0, "ResidentAttention": 1, "ResidentNorm": 2}

    def __init__(self, library, stages, *, workers=148, schedule="linear"):
        from native_pi0.program import spread_streams, validate_streams
        self.library = _native.load(library)
        self.handle = C.c_void_p()
        self.operators = [op for op, _ in stages]
        if not self.operators:
            raise ValueError("At least one stage is required")
        self.device = self.operators[0].device
        specs, tiles, work = [], [], []
        for index, (op, sources) in enumerate(stages):
            kind = self._KIND.get(type(op).__name__)
            if kind is None or not op.handle.value:
                raise ValueError("Stages must be live operator wrappers")
            sources = list(sources)
            if len(sources) > 4 or any(not (0 <= s < index) or m not in (0, 1) for s, m in sources):
                raise ValueError("Sources must be (earlier stage, mode 0|1), at most four")
            spec = _native.NativeSpec()
            spec.kind, spec.handle = kind, op.handle.value
            for slot in range(4):
                spec.sources[slot], spec.modes[slot] = sources[slot] if slot < len(sources) else (-1, 1)
            specs.append(spec)
            t, b, k = C.c_int(), C.c_int(), C.c_int()
            _native.check(self.library.op_geometry(op.handle, C.byref(t), C.byref(b), C.byref(k)), "geometry")
            tiles.append(t.value)
            work.append(LinearWork(t.value, max(64, (k.value + 63) // 64 * 64)))
        if schedule == "spread":
            self.code = spread_streams(work, workers, [[s for s in spec.sources] for spec in specs])
        else:
            self.code = linear_streams(work, workers)
        validate_streams(self.code, tiles)
        self.plan = program_summary(self.code)
        array = (_native.NativeSpec * len(specs))(*specs)
        with torch.cuda.device(self.device):
            _native.check(self.library.create_native_model(C.byref(self.handle), len(specs), C.cast(array, C.c_void_p),
                                                           self.code.ctypes.data, workers, self.code.shape[1]), "Native stage program setup")

    def forward(self):
        if not self.handle.value:
            raise RuntimeError("Native stage program is closed")
        with torch.cuda.device(self.device):
            _native.check(self.library.launch_native_model(self.handle, torch.cuda.current_stream(self.device).cuda_stream,
                                                           None, None, None, None), "Native stage program launch")
        return self.operators[-1].output

    def status(self):
        with torch.cuda.device(self.device):
            return _native.status(self.library, self.handle)

    def close(self):
        if self.handle.value:
            with torch.cuda.device(self.device):
                _native.check(self.library.destroy_native_model(self.handle), "Native stage program teardown")
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
