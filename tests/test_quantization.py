"""NVFP4 packer: shipped packer and CPU oracle against the reference's golden
vectors and known-answer tests (reference ``native_pi0/test_quantization.py``)."""
import json

import numpy as np
import pytest

from native_pi0.quantization import (E2M1, UE4M3, PackedNVFP4, _nearest_even, interleave_gate_up,
                                     pack_nvfp4, scale_offsets, swizzle_scales, unswizzle_scales)
from oracle import nvfp4 as oracle


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(golden_dir / "nvfp4_pack.npz"), json.loads((golden_dir / "nvfp4_pack.json").read_text())


def test_tables_match_oracle():
    np.testing.assert_array_equal(E2M1, oracle.E2M1_VALUES)
    np.testing.assert_array_equal(UE4M3, oracle.UE4M3_VALUES)
    assert UE4M3[-1] == 448 and UE4M3[1] == 2.0 ** -9 and UE4M3.size == 127


def test_packer_matches_reference_golden(gold):
    data, meta = gold
    for name, kw in meta.items():
        p = pack_nvfp4(data[name + "_in"], **kw)
        np.testing.assert_array_equal(p.data, data[name + "_data"], err_msg=name)
        np.testing.assert_array_equal(p.scales, data[name + "_scales"], err_msg=name)
        if name + "_deq" in data:
            np.testing.assert_array_equal(p.dequantize(), data[name + "_deq"], err_msg=name)


def test_oracle_matches_reference_golden(gold):
    data, meta = gold
    for name, kw in meta.items():
        x = data[name + "_in"]
        d, s = oracle.pack(x, **kw)
        np.testing.assert_array_equal(d, data[name + "_data"], err_msg=name)
        np.testing.assert_array_equal(s, data[name + "_scales"], err_msg=name)
        if name + "_deq" in data:
            np.testing.assert_array_equal(oracle.dequantize(d, s, kw.get("global_scale", 1.0), x.shape),
                                          data[name + "_deq"], err_msg=name)


# --- known answers held by the reference's own unit tests ------------------------------------
def test_reciprocal_midpoint_semantics():            # test_quantization.py:9-16
    v = np.zeros((1, 16), np.float32)
    v[0, :2] = [5.625, 1.171875]
    for packed in (pack_nvfp4(v), PackedNVFP4(*oracle.pack(v), np.float32(1), (1, 16))):
        assert packed.scales[0, 0] == 55
        assert packed.data[0, 0] == 0x37


def test_formats_and_ties():                         # :18-23
    np.testing.assert_array_equal(_nearest_even(E2M1, E2M1), np.arange(8))
    mid = (E2M1[:-1] + E2M1[1:]) / 2
    np.testing.assert_array_equal(_nearest_even(mid, E2M1), [0, 2, 2, 4, 4, 6, 6])
    np.testing.assert_array_equal(oracle.nearest_code(mid, oracle.E2M1_VALUES), [0, 2, 2, 4, 4, 6, 6])
    np.testing.assert_array_equal(_nearest_even(UE4M3, UE4M3), np.arange(127))


def test_exact_codes_and_nibble_order():             # :25-30
    x = np.concatenate((E2M1, -E2M1))[None, :]
    p = pack_nvfp4(x)
    np.testing.assert_array_equal(p.scales, [[56]])
    np.testing.assert_array_equal(p.data, [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]])
    np.testing.assert_array_equal(p.dequantize(), x)
    d, s = oracle.pack(x)
    np.testing.assert_array_equal(d, p.data)
    np.testing.assert_array_equal(s, p.scales)


def test_zero_tiny_and_padding():                    # :32-43
    x = np.full((3, 17), 1e-12, np.float32)
    x[1] *= -1
    p = pack_nvfp4(x, row_alignment=128, column_alignment=128)
    assert not p.scales.any() and not p.data.any()
    assert p.data.shape == (128, 64) and p.scales.shape == (128, 8)
    assert p.dequantize().shape == x.shape
    c = pack_nvfp4(x, scale_policy="ceil")
    assert (c.scales[:, :1] == 1).all()
    assert np.isfinite(c.dequantize()).all()


def test_global_scale_and_representative_shapes():   # :45-52
    rng = np.random.default_rng(7)
    for rows, cols in ((51, 1024), (256, 1152), (768, 2048), (3, 4304)):
        x = rng.normal(size=(rows, cols)).astype(np.float32)
        p = pack_nvfp4(x, global_scale=.125)
        err = np.linalg.norm(p.dequantize() - x) / np.linalg.norm(x)
        assert err < .13
        assert np.isfinite(p.dequantize()).all()


def test_gate_up_and_invalid_inputs(golden_dir):     # :54-64
    g = np.arange(12).reshape(3, 4)
    r = interleave_gate_up(g, g + 100)
    np.testing.assert_array_equal(r[::2], g)
    np.testing.assert_array_equal(r[1::2], g + 100)
    np.testing.assert_array_equal(r, np.load(golden_dir / "nvfp4_swizzle.npz")["interleave"])
    for x in (np.array([[np.nan]]), np.array([[np.inf]]), np.empty((0, 4)), np.ones(4)):
        with pytest.raises(ValueError):
            pack_nvfp4(x)
    for s in (0, -1, float("nan")):
        with pytest.raises(ValueError):
            pack_nvfp4([[1]], global_scale=s)
    with pytest.raises(ValueError):
        pack_nvfp4([[1]], scale_policy="floor")
    with pytest.raises(ValueError):
        pack_nvfp4([[1]], column_alignment=24)
    with pytest.raises(ValueError):
        interleave_gate_up(g, g[:2])


def test_swizzle_layout(golden_dir):
    z = np.load(golden_dir / "nvfp4_swizzle.npz")
    np.testing.assert_array_equal(scale_offsets(130, 9), z["offsets_130_9"])
    for key in z.files:
        if not key.startswith("lin_"):
            continue
        _, rows, blocks = key.split("_")
        rows, blocks = int(rows), int(blocks)
        lin = z[key]
        swz = swizzle_scales(lin)
        np.testing.assert_array_equal(swz, z[f"swz_{rows}_{blocks}"])
        np.testing.assert_array_equal(unswizzle_scales(swz, rows, blocks), lin)
        if rows * blocks <= 40000:
            np.testing.assert_array_equal(oracle.swizzle(lin), swz)
            np.testing.assert_array_equal(oracle.unswizzle(swz, rows, blocks), lin)
    with pytest.raises(ValueError):
        swizzle_scales(np.zeros((2, 2), np.int32))
    with pytest.raises(ValueError):
        unswizzle_scales(np.zeros(100, np.uint8), 2, 2)
    with pytest.raises(ValueError):
        scale_offsets(0, 1)


def test_random_agreement_packer_vs_oracle():
    rng = np.random.default_rng(11)
    for policy in ("nearest", "ceil"):
        x = (rng.normal(size=(9, 80)) * np.exp(rng.normal(size=(9, 80)) * 3)).astype(np.float32)
        p = pack_nvfp4(x, scale_policy=policy, global_scale=0.37, row_alignment=4, column_alignment=32)
        d, s = oracle.pack(x, 0.37, policy, 4, 32)
        np.testing.assert_array_equal(p.data, d)
        np.testing.assert_array_equal(p.scales, s)
