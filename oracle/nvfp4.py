"""NumPy restatement of the reference NVFP4 quantizer (test infrastructure).

Follows the algorithm of the reference ``native_pi0/quantization.py``:
``E2M1`` / ``UE4M3`` tables ``:14-19``, nearest-with-even-code-ties ``:22-27``,
``pack_nvfp4`` ``:48-93``, ``PackedNVFP4.dequantize`` ``:37-45``,
``scale_offsets`` ``:104-115``.  It is deliberately the slow, obvious form
(exhaustive nearest-entry search over the code tables) so that it shares no
arithmetic shortcuts with the shipped packer or the CUDA kernels.

Pinned against: the reference's own known-answer tests
(``native_pi0/test_quantization.py:9-64``) and golden vectors produced by
importing the reference module in the build container
(``tests/golden/make_golden.py`` -> ``tests/golden/nvfp4_*.npz``).
"""
import numpy as np

E2M1_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)


def ue4m3_value(code):
    """``quantization.py:15-19``: code<8 subnormal ``m*2^-9``, else ``(1+m/8)*2^(e-7)``."""
    code = int(code)
    m, e = code & 7, code >> 3
    return np.float32(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))


UE4M3_VALUES = np.array([ue4m3_value(c) for c in range(127)], dtype=np.float32)


def nearest_code(values, table):
    """Index of the closest table entry; exact midpoints pick the even index
    (``quantization.py:22-27``).  Values beyond the last entry saturate."""
    v = np.asarray(values, dtype=np.float32).reshape(-1, 1).astype(np.float64)
    t = table.astype(np.float64).reshape(1, -1)
    dist = np.abs(v - t)
    best = dist.min(axis=1, keepdims=True)
    idx = np.arange(table.size).reshape(1, -1)
    cand = np.where(dist == best, idx, 10 ** 6)
    # at most two candidates (neighbours); prefer the even one
    even = np.where(cand % 2 == 0, cand, 10 ** 6).min(axis=1)
    anyc = cand.min(axis=1)
    pick = np.where(even < 10 ** 6, even, anyc)
    return pick.reshape(np.shape(values))


def ceil_code(values, table):
    """Smallest index whose entry is >= value, clipped to the table
    (``quantization.py:79-80``: ``searchsorted(...).clip(0,126)``)."""
    v = np.asarray(values, dtype=np.float32)
    out = np.zeros(v.shape, dtype=np.int64)
    flat = v.reshape(-1)
    res = out.reshape(-1)
    for i, x in enumerate(flat):
        j = 0
        while j < table.size - 1 and table[j] < x:
            j += 1
        res[i] = j
    return out


def pack(matrix, global_scale=1.0, scale_policy="nearest", row_alignment=1, column_alignment=16):
    """``quantization.py:48-93`` step by step.  Returns (data u8[R,K/2], scales u8[R,K/16])."""
    x = np.asarray(matrix, dtype=np.float32)
    gs = np.float32(global_scale)
    rows, cols = x.shape
    pr = (rows + row_alignment - 1) // row_alignment * row_alignment
    pk = (cols + column_alignment - 1) // column_alignment * column_alignment
    padded = np.zeros((pr, pk), dtype=np.float32)
    padded[:rows, :cols] = x * np.float32(np.float32(1) / gs)            # :72
    blocks = padded.reshape(pr, pk // 16, 16)
    desired = np.abs(blocks).max(axis=-1) * np.float32(1 / 6)            # :76
    if scale_policy == "ceil":
        codes = ceil_code(desired, UE4M3_VALUES)                          # :78
    else:
        codes = nearest_code(desired, UE4M3_VALUES)                       # :80
    scale = UE4M3_VALUES[codes]
    recip = np.zeros_like(scale)
    nz = scale > 0
    recip[nz] = np.float32(1) / scale[nz]                                 # :84  (FP32 reciprocal)
    normalized = blocks * recip[..., None]                                # :85
    normalized[~nz] = 0                                                   # :86
    q = nearest_code(np.abs(normalized), E2M1_VALUES).astype(np.uint8)    # :87
    q = q | (np.signbit(normalized).astype(np.uint8) << 3)                # :88
    q = q.reshape(pr, pk)
    data = q[:, 0::2] | (q[:, 1::2] << 4)                                 # :92 low nibble = even column
    return data.astype(np.uint8), codes.astype(np.uint8)


def dequantize(data, scales, global_scale, logical_shape):
    """``quantization.py:37-45``."""
    r, half = data.shape
    codes = np.zeros((r, half * 2), dtype=np.uint8)
    codes[:, 0::2] = data & 15
    codes[:, 1::2] = data >> 4
    vals = E2M1_VALUES[codes & 7] * np.where(codes & 8, np.float32(-1), np.float32(1))
    vals = vals * np.repeat(UE4M3_VALUES[scales], 16, axis=1)
    vals = (vals * np.float32(global_scale)).astype(np.float32)
    return vals[:logical_shape[0], :logical_shape[1]]


def scale_offset(row, block, blocks):
    """``quantization.py:104-115`` for a single (row, block)."""
    return ((row // 128) * ((blocks + 3) // 4) + block // 4) * 512 + (row % 32) * 16 \
        + (row % 128 // 32) * 4 + block % 4


def swizzle(linear):
    """``quantization.py:118-127`` with explicit loops."""
    rows, blocks = linear.shape
    out = np.zeros(((rows + 127) // 128) * ((blocks + 3) // 4) * 512, dtype=np.uint8)
    for r in range(rows):
        for b in range(blocks):
            out[scale_offset(r, b, blocks)] = linear[r, b]
    return out


def unswizzle(swizzled, rows, blocks):
    out = np.zeros((rows, blocks), dtype=np.uint8)
    for r in range(rows):
        for b in range(blocks):
            out[r, b] = swizzled[scale_offset(r, b, blocks)]
    return out


def gemm(a_data, a_scales, a_gs, b_data, b_scales, b_gs, m, n, k):
    """Dequantized-NVFP4 GEMM, the oracle the reference validator uses
    (``scripts/validate_nvfp4.py:49``): ``deq(A) @ deq(B).T`` in FP32/FP64."""
    a = dequantize(a_data, a_scales, a_gs, (m, k)).astype(np.float64)
    b = dequantize(b_data, b_scales, b_gs, (n, k)).astype(np.float64)
    return (a @ b.T).astype(np.float32)
