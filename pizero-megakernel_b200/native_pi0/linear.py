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
