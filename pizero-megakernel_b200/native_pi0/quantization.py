"""Offline NVFP4 packing for the B200 pi0 engine (setup-time, NumPy only).

Drop-in for the reference module ``native_pi0/quantization.py`` (``pack_nvfp4``
at ``native_pi0/quantization.py:48-93``, ``PackedNVFP4`` ``:30-45``,
``interleave_gate_up`` ``:96-101``, ``scale_offsets`` / ``swizzle_scales`` /
``unswizzle_scales`` ``:104-135``).  The arithmetic is written independently:
codes are computed from exponent/mantissa arithmetic and threshold compares
instead of table searches, but every byte it emits is identical.

Format
------
* value codes: E2M1, magnitudes ``{0, .5, 1, 1.5, 2, 3, 4, 6}``, sign in bit 3;
  two codes per byte, the even column in the low nibble.
* block scales: one unsigned E4M3 code (0..126, 126 == 448) for every 16
  consecutive K elements of a row.
* tensor scale: one FP32 number; ``value = e2m1 * ue4m3 * global_scale``.

The device kernels of this package (``csrc/``) reproduce exactly this
arithmetic: ``amax * fp32(1/6)`` -> E4M3 (round-to-nearest-even or ceiling),
element times the FP32 reciprocal of the decoded scale -> E2M1 RNE.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

# Public decode tables (same names and contents as the reference exports).
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def _decode_ue4m3(codes):
    """Unsigned E4M3 byte -> FP32 (bias 7, subnormal step 2**-9)."""
    codes = np.asarray(codes).astype(np.int64)
    mant = (codes & 7).astype(np.float64)
    expo = codes >> 3
    normal = np.ldexp(1.0 + mant / 8.0, expo - 7)
    sub = np.ldexp(mant, -9)
    return np.where(expo == 0, sub, normal).astype(np.float32)


UE4M3 = _decode_ue4m3(np.arange(127))


def _encode_ue4m3(desired, ceil):
    """Non-negative FP32 -> code 0..126; RNE on even codes, or smallest code >= x."""
    d = np.asarray(desired, dtype=np.float64)
    # Position on the code axis: every binade [2**e, 2**(e+1)) holds 8 codes.
    safe = np.maximum(d, 2.0 ** -6)
    mant, expo = np.frexp(safe)              # safe = mant * 2**expo, mant in [.5,1)
    e = expo - 1                              # safe = (2*mant) * 2**e
    frac = (2.0 * mant - 1.0) * 8.0           # 0 <= frac < 8, exact
    normal_axis = (e + 7) * 8 + frac
    sub_axis = d * 2.0 ** 9                   # exact, codes 0..8
    axis = np.where(d < 2.0 ** -6, sub_axis, normal_axis)
    code = np.ceil(axis) if ceil else np.rint(axis)   # rint == ties to even code
    return np.clip(code, 0, 126).astype(np.int64)


def _encode_e2m1(magnitude):
    """|x| -> code 0..7 with midpoint ties going to the even code, saturating at 6."""
    m = magnitude
    return ((m > 0.25).astype(np.uint8) + (m >= 0.75) + (m > 1.25) + (m >= 1.75)
            + (m > 2.5) + (m >= 3.5) + (m > 5.0)).astype(np.uint8)


def _nearest_even(values, table):
    """Nearest table index with even-index ties (kept for API parity, ``quantization.py:22-27``)."""
    values = np.asarray(values, dtype=np.float32)
    table = np.asarray(table, dtype=np.float32)
    if table.shape == E2M1.shape and np.array_equal(table, E2M1):
        return _encode_e2m1(values).astype(np.int64)
    if table.shape == UE4M3.shape and np.array_equal(table, UE4M3):
        return _encode_ue4m3(values, ceil=False)
    gap = np.abs(values[..., None].astype(np.float64) - table.astype(np.float64))
    best = gap.min(axis=-1, keepdims=True)
    hit = gap == best
    index = np.arange(table.size)
    even_first = np.where(hit & (index % 2 == 0), index, table.size)
    any_first = np.where(hit, index, table.size)
    pick_even = even_first.min(axis=-1)
    return np.where(pick_even < table.size, pick_even, any_first.min(axis=-1))


@dataclass(frozen=True)
class PackedNVFP4:
    """Packed matrix: ``data`` u8[R, K/2], ``scales`` u8[R, K/16] (linear), FP32 tensor scale."""
    data: np.ndarray
    scales: np.ndarray
    global_scale: np.float32
    logical_shape: tuple

    def dequantize(self):
        lo = self.data & 0x0F
        hi = self.data >> 4
        nib = np.stack((lo, hi), axis=-1).reshape(self.data.shape[0], -1)
        mag = E2M1[nib & 7]
        out = np.where(nib & 8, -mag, mag).astype(np.float32)
        out *= np.repeat(UE4M3[self.scales], 16, axis=1)
        out *= self.global_scale
        r, c = self.logical_shape
        return out[:r, :c]


def pack_nvfp4(matrix, *, global_scale=1.0, scale_policy="nearest", row_alignment=1,
               column_alignment=16):
    """Quantize an ``[rows, K]`` matrix to NVFP4.

    ``scale_policy='nearest'`` is the activation rule (block scale = RNE of
    ``amax/6``); ``'ceil'`` is the weight rule (smallest representable scale not
    below ``amax/6``).  Rows/columns are zero padded to the given alignments;
    padded codes and scales are zero.  A block whose scale code is 0 encodes as
    all-zero codes.  Elements are scaled by the FP32 *reciprocal* of the decoded
    block scale (not divided), which decides E2M1 midpoint ties the same way the
    device converter does.
    """
    x = np.asarray(matrix, dtype=np.float32)
    gs = np.float32(global_scale)
    if x.ndim != 2 or 0 in x.shape or not np.all(np.isfinite(x)):
        raise ValueError("Expected a nonempty finite matrix")
    if not (np.isfinite(gs) and gs > 0):
        raise ValueError("global_scale must be finite and positive")
    if scale_policy not in ("nearest", "ceil"):
        raise ValueError("scale_policy must be nearest or ceil")
    ok_rows = isinstance(row_alignment, int) and row_alignment >= 1
    ok_cols = (isinstance(column_alignment, int) and column_alignment >= 16
               and column_alignment % 16 == 0)
    if not (ok_rows and ok_cols):
        raise ValueError("Invalid row alignment or column alignment (multiple of 16 required)")
    rows, cols = x.shape
    pr = -(-rows // row_alignment) * row_alignment
    pk = -(-cols // column_alignment) * column_alignment
    work = np.zeros((pr, pk), dtype=np.float32)
    inv_gs = np.float32(1) / gs
    with np.errstate(over="ignore"):
        work[:rows, :cols] = x * inv_gs
    if not np.all(np.isfinite(work)):
        raise ValueError("global_scale overflows normalized values")
    blocks = work.reshape(pr, pk // 16, 16)
    sixth = np.float32(1.0 / 6.0)
    desired = np.abs(blocks).max(axis=2) * sixth                  # FP32 product
    codes = _encode_ue4m3(desired, ceil=(scale_policy == "ceil"))
    decoded = UE4M3[codes]
    live = decoded > 0
    recip = np.zeros_like(decoded)
    np.divide(np.float32(1), decoded, out=recip, where=live)      # FP32 reciprocal
    scaled = blocks * recip[:, :, None]                           # FP32 product
    scaled[~live] = 0.0
    nib = _encode_e2m1(np.abs(scaled)) | (np.signbit(scaled).astype(np.uint8) << 3)
    nib = nib.reshape(pr, pk)
    data = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return PackedNVFP4(np.ascontiguousarray(data), codes.astype(np.uint8), gs, (rows, cols))


def interleave_gate_up(gate, up):
    """Row-interleave two ``[N, K]`` matrices: g0, u0, g1, u1, ... (GeGLU pairs become adjacent N columns)."""
    gate = np.asarray(gate)
    up = np.asarray(up)
    if gate.ndim != 2 or gate.shape != up.shape:
        raise ValueError("gate and up must be equal-shaped matrices")
    out = np.empty((2 * gate.shape[0], gate.shape[1]), dtype=np.result_type(gate, up))
    out[0::2] = gate
    out[1::2] = up
    return out


def scale_offsets(rows, blocks):
    """Byte offset of scale (row, block) in the SM100 block-scale layout.

    128 rows x 4 blocks form one 512-byte atom: 32 lines of 16 bytes; line
    ``row % 32`` holds, at byte ``4 * (row % 128 // 32) + block % 4``, the scale
    of that row.  Atoms are ordered row-tile major, then by K group of 64.
    """
    if not (isinstance(rows, int) and isinstance(blocks, int)) or rows < 1 or blocks < 1:
        raise ValueError("rows and blocks must be positive integers")
    r = np.arange(rows, dtype=np.int64).reshape(-1, 1)
    b = np.arange(blocks, dtype=np.int64).reshape(1, -1)
    atoms_per_row_tile = -(-blocks // 4)
    atom = (r >> 7) * atoms_per_row_tile + (b >> 2)
    return atom * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)


def swizzled_size(rows, blocks):
    return (-(-rows // 128)) * (-(-blocks // 4)) * 512


def swizzle_scales(linear):
    """u8[R, B] linear scales -> 1-D SM100 layout, zero in every padded slot."""
    linear = np.asarray(linear)
    if linear.ndim != 2 or linear.dtype != np.uint8 or 0 in linear.shape:
        raise ValueError("Expected a nonempty uint8 scale matrix")
    rows, blocks = linear.shape
    out = np.zeros(swizzled_size(rows, blocks), dtype=np.uint8)
    out[scale_offsets(rows, blocks)] = linear
    return out


def unswizzle_scales(swizzled, rows, blocks):
    where = scale_offsets(rows, blocks)
    swizzled = np.asarray(swizzled)
    if swizzled.ndim != 1 or swizzled.dtype != np.uint8 or swizzled.size != swizzled_size(rows, blocks):
        raise ValueError("Incorrect swizzled scale buffer size or dtype")
    return swizzled[where].copy()
