"""B200-native pi0 engine: NVFP4 tcgen05 GEMMs, fused producers and one persistent instruction-stream kernel.

Drop-in for the reference package of the same name (``native_pi0/__init__.py:2-4`` exports ``NativePi0``).
The CUDA extension ``libpi0_native.so`` must have been built (``native_pi0._native.build()``); nothing here
falls back to the CPU.
"""
__all__ = ["NativePi0"]


def __getattr__(name):
    if name == "NativePi0":           # imported lazily so the offline tools work without torch/CUDA
        from native_pi0.model import NativePi0
        return NativePi0
    raise AttributeError(name)
