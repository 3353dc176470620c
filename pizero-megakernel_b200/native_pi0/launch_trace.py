"""Count kernel launches with CUPTI driver callbacks.

    with LaunchTrace() as trace:
        engine.forward(...)
        torch.cuda.synchronize()
    assert trace.count == 1 and "pi0_vm_kernel" in trace.symbol

The usage of the reference helper (``native_pi0/launch_trace.py:5-34``) over the three exports of
``launch_trace.cpp:25-47``; here they live in ``libpi0_trace.so`` and are typed by ``_native.load_trace``.
``count`` and ``symbol`` (name of the first kernel seen) are set when the block is left.
"""
import ctypes

from native_pi0 import _native

_SYMBOL_BYTES = 2048


class LaunchTrace:
    count = None
    symbol = ""

    def __init__(self, library=None):
        self._lib = _native.load_trace(library)
        self._session = None

    def _raise_on(self, code, what):
        if code:
            text = self._lib.launch_trace_error(code)
            raise RuntimeError(f"CUPTI launch trace error {code} while {what}: {text.decode() if text else 'unknown'}")

    def __enter__(self):
        if self._session is not None:
            raise RuntimeError("LaunchTrace is already recording")
        session = ctypes.c_void_p()
        self._raise_on(self._lib.begin_launch_trace(ctypes.byref(session)), "subscribing")
        self._session = session
        return self

    def __exit__(self, exc_type, exc, tb):
        session, self._session = self._session, None
        launches = ctypes.c_int(0)
        name = ctypes.create_string_buffer(_SYMBOL_BYTES)
        code = self._lib.end_launch_trace(session, ctypes.byref(launches), name, _SYMBOL_BYTES)
        if exc_type is None:
            self._raise_on(code, "unsubscribing")
        self.count, self.symbol = launches.value, name.value.decode(errors="replace")
        return False
