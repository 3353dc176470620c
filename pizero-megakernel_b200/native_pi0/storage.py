"""Device storage for packed operands that are read through TMA tensor maps.

Counterpart of the reference ``native_pi0/storage.py:7-17``.  TMA boxes are
rounded up to whole 128-byte swizzle spans, so the allocation keeps 127 spare,
zero-initialised bytes behind the logical extent; a view of the logical shape is
returned.  The allocation start is at least 256-byte aligned (PyTorch caching
allocator), which satisfies the 16-byte TMA base-address rule.
"""
import math

import torch

TAIL_BYTES = 127


def packed_tma_buffer(shape, *, device):
    count = math.prod(shape)
    backing = torch.zeros(count + TAIL_BYTES, dtype=torch.uint8, device=device)
    return backing[:count].view(shape)
