"""Count kernel launches with CUPTI driver callbacks (``with LaunchTrace() as t: ...; t.count``).

Same usage as the reference ``native_pi0/launch_trace.py:5-34``; lives in its own small library
(``libpi0_trace.so``) so the engine itself does not depend on CUPTI.
"""
import ctypes

from native_pi0 import _native


class LaunchTrace:
    def __init__(self, library=None):
        path = library if library is not None else _native.TRACE_LIBRARY
        self.library = ctypes.CDLL(str(path))
        self.begin = self.library.begin_launch_trace
        self.begin.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        self.begin.restype = ctypes.c_int
        self.end = self.library.end_launch_trace
        self.end.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_void_p, ctypes.c_int]
        self.end.restype = ctypes.c_int
        self.error = self.library.launch_trace_error
        self.error.argtypes = [ctypes.c_int]
        self.error.restype = ctypes.c_char_p
        self.handle = ctypes.c_void_p()
        self.count = None
        self.symbol = ""

    def check(self, code):
        if code:
            raise RuntimeError(f"CUPTI launch trace error {code}: {self.error(code)}")

    def __enter__(self):
        self.check(self.begin(ctypes.byref(self.handle)))
        return self

    def __exit__(self, *_):
        count = ctypes.c_int()
        symbol = ctypes.create_string_buffer(2048)
        code = self.end(self.handle, ctypes.byref(count), symbol, len(symbol))
        self.handle = ctypes.c_void_p()
        self.check(code)
        self.count = count.value
        self.symbol = symbol.value.decode()
