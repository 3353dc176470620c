"""GPU parity of every operator against the CPU oracles, through the C ABI (ctypes).

Tolerances: NVFP4 packing and scales bit-exact; GEMM / attention outputs <= 1e-2 relative RMS against the
dequantised-NVFP4 / FP32 oracle (BF16 outputs add one BF16 rounding).
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0 import _native
from native_pi0.attention import ResidentAttention
from native_pi0.normalization import ResidentNorm
from native_pi0.primitives import ResidentNVFP4
from native_pi0.quantization import PackedNVFP4, interleave_gate_up, pack_nvfp4, swizzle_scales, unswizzle_scales
from oracle import nvfp4 as oracle
from oracle import ops as oracle_ops


def bf16(x):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).bfloat16()


def relrms(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def config1_inputs(n=4096):
    rng = np.random.default_rng(0)
    x = rng.normal(size=(51, 1024)).astype(np.float32)
    x[rng.random(x.shape) < 0.001] *= 20
    w = rng.normal(scale=0.02, size=(n, 1024)).astype(np.float32)
    return bf16(x).float().numpy(), bf16(w).float().numpy()


def device_quantize(x, policy, global_scale=1.0, row_alignment=128):
    lib = _native.load()
    xt = bf16(x).cuda()
    rows, width = xt.shape
    rp = (rows + row_alignment - 1) // row_alignment * row_alignment
    out = torch.zeros(rp, width // 2, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(((rp + 127) // 128) * ((width // 16 + 3) // 4) * 512, dtype=torch.uint8, device="cuda")
    _native.check(lib.quantize_nvfp4(xt.data_ptr(), out.data_ptr(), sc.data_ptr(), rows, width, width, width // 16,
                                     float(global_scale), int(policy == "ceil"), None), "quantize")
    torch.cuda.synchronize()
    return out.cpu().numpy(), unswizzle_scales(sc.cpu().numpy(), rp, width // 16)


def test_quantizer_bit_exact_config1_and_golden(golden_dir):
    x, w = config1_inputs(512)
    for arr, policy, gs in ((x, "nearest", 1.0), (w, "ceil", 1.0), (w, "ceil", float(np.abs(w).max() / (6 * 448)))):
        data, scales = device_quantize(arr, policy, gs)
        ref = pack_nvfp4(arr, scale_policy=policy, global_scale=gs, row_alignment=128)
        np.testing.assert_array_equal(data, ref.data)
        np.testing.assert_array_equal(scales, ref.scales)
        od, osc = oracle.pack(arr[:8], gs, policy)
        np.testing.assert_array_equal(data[:8], od)
        np.testing.assert_array_equal(scales[:8], osc)
    gold = np.load(golden_dir / "nvfp4_pack.npz")          # vectors produced by the reference packer itself
    for name, policy in (("cfg1_x", "nearest"), ("cfg1_w", "ceil"), ("ties", "nearest"), ("ties_ceil", "ceil"),
                         ("wide_range", "nearest"), ("wide_range_ceil", "ceil")):
        arr = gold[name + "_in"]
        if not np.array_equal(bf16(arr).float().numpy(), arr):
            continue                                        # the device quantiser consumes BF16 inputs
        data, scales = device_quantize(arr, policy)
        rows = arr.shape[0]
        np.testing.assert_array_equal(data[:rows], gold[name + "_data"][:rows], err_msg=name)
        np.testing.assert_array_equal(scales[:rows], gold[name + "_scales"][:rows], err_msg=name)


def test_quantizer_edge_cases():
    # zeros, tiny blocks (zero scale -> zero codes), saturation, exact midpoints
    x = np.zeros((3, 64), np.float32)
    x[1, :16] = 1e-12
    x[1, 16:32] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x[2, :] = 3000.0
    for policy in ("nearest", "ceil"):
        data, scales = device_quantize(x, policy)
        ref = pack_nvfp4(bf16(x).float().numpy(), scale_policy=policy, row_alignment=128)
        np.testing.assert_array_equal(data, ref.data)
        np.testing.assert_array_equal(scales, ref.scales)
    assert not data[3:].any() and not scales[3:].any()


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 1152), (256, 384, 4352), (768, 2560, 2048), (128, 1024, 4096)])
def test_gemm_fp32_matches_dequantised_oracle(m, n, k):
    rng = np.random.default_rng(23 + m + n + k)
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(scale=0.02, size=(n, k)).astype(np.float32)
    pa, pb = pack_nvfp4(a, global_scale=0.5), pack_nvfp4(b, scale_policy="ceil", global_scale=0.001)
    ref = oracle.gemm(pa.data, pa.scales, 0.5, pb.data, pb.scales, 0.001, m, n, k)
    with ResidentNVFP4(None, pa, pb, workers=min(148, (m // 128) * (n // 128))) as op:
        got = op.forward().cpu().numpy()
        assert op.status()["code"] == 0
        again = op.forward().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=3e-5, atol=1e-5 * max(1.0, np.abs(ref).max()))
    np.testing.assert_array_equal(got, again)               # replay is bit-exact


def test_gemm_config1_bf16_output():
    x, w = config1_inputs()
    pa, pb = pack_nvfp4(x, row_alignment=128), pack_nvfp4(w, scale_policy="ceil")
    ref = oracle.gemm(pa.data, pa.scales, 1.0, pb.data, pb.scales, 1.0, 128, 4096, 1024)
    with ResidentNVFP4(None, pa, pb, workers=32, output_dtype=torch.bfloat16, rows=51) as op:
        y = op.forward().float().cpu().numpy()
    assert relrms(y[:51], ref[:51]) <= 1e-2                 # stated tolerance; one BF16 rounding gives ~2e-3
    assert relrms(y[:51], ref[:51]) <= 3e-3
    assert not y[51:].any()                                 # rows beyond the logical count are never stored
    assert relrms(ref[:51], x @ w.T) < 0.2                  # sanity: NVFP4 itself is ~14 % from the BF16 product


def test_gemm_bias_residual_and_tiles():
    rng = np.random.default_rng(47)
    m, n, k = 256, 512, 1024
    a, b = rng.normal(size=(m, k)).astype(np.float32), rng.normal(scale=0.05, size=(n, k)).astype(np.float32)
    bias, res = bf16(rng.normal(size=n)), bf16(rng.normal(size=(m, n)))
    pa, pb = pack_nvfp4(a), pack_nvfp4(b, scale_policy="ceil")
    ref = oracle.gemm(pa.data, pa.scales, 1.0, pb.data, pb.scales, 1.0, m, n, k) + bias.float().numpy()[None] + res.float().numpy()
    expect = bf16(ref).float().numpy()
    results = []
    for block_n, tiled in ((128, False), (64, False), (128, True), (64, True), (32, False), (32, True)):
        with ResidentNVFP4(None, pa, pb, workers=7, output_dtype=torch.bfloat16, bias=bias, residual=res, block_n=block_n,
                           tiled_weight=tiled) as op:
            y = op.forward().float().cpu().numpy()
            assert op.status()["code"] == 0
        mism = float((y != expect).mean())
        assert mism < 1e-3, (block_n, tiled, mism)          # BF16 result equal except FP32 summation-order ties
        assert relrms(y, expect) < 1e-3
        results.append(y)
    for y in results[1:]:                                   # tile width and weight layout do not change a single bit
        np.testing.assert_array_equal(y, results[0])
    with pytest.raises(RuntimeError):
        ResidentNVFP4(None, pa, pb, block_n=16)             # tiles are 128, 64 or 32 columns wide


def _decode(op, rows, width):
    data = op.output.cpu().numpy()
    scales = unswizzle_scales(op.output_scales.cpu().numpy(), data.shape[0], width // 16)
    return PackedNVFP4(data, scales, np.float32(op.output_global_scale), (rows, width))


def test_gemm_fp4_epilogues():
    rng = np.random.default_rng(61)
    m, n, k = 256, 512, 1152
    a, b = rng.normal(size=(m, k)).astype(np.float32), rng.normal(scale=0.03, size=(n, k)).astype(np.float32)
    bias = bf16(rng.normal(scale=0.5, size=n))
    pa, pb = pack_nvfp4(a), pack_nvfp4(b, scale_policy="ceil")
    acc = oracle.gemm(pa.data, pa.scales, 1.0, pb.data, pb.scales, 1.0, m, n, k)
    # GELU(acc + bias) -> NVFP4
    want = oracle_ops.gelu_tanh(torch.from_numpy(acc + bias.float().numpy()[None])).numpy()
    ref = pack_nvfp4(want, global_scale=0.5)
    with ResidentNVFP4(None, pa, pb, workers=8, output_dtype=torch.uint8, bias=bias, output_gelu=True, output_global_scale=0.5) as op:
        op.forward()
        got = _decode(op, m, n)
    assert float((got.scales != ref.scales).mean()) < 2e-3
    assert float((got.data != ref.data).mean()) < 5e-3      # differences only where FP32 rounding moves a tie
    assert relrms(got.dequantize(), ref.dequantize()) < 1e-2
    # compact GeGLU over interleaved gate/up columns -> NVFP4 of width n/2
    gate, up = b[: n // 2], b[n // 2:]
    pgu = pack_nvfp4(interleave_gate_up(gate, up), scale_policy="ceil")
    acc = oracle.gemm(pa.data, pa.scales, 1.0, pgu.data, pgu.scales, 1.0, m, n, k)
    want = oracle_ops.gelu_tanh(torch.from_numpy(acc[:, 0::2])).numpy() * acc[:, 1::2]
    ref = pack_nvfp4(want)
    with ResidentNVFP4(None, pa, pgu, workers=8, output_dtype=torch.uint8, output_geglu=True) as op:
        op.forward()
        got = _decode(op, m, n // 2)
    assert float((got.scales != ref.scales).mean()) < 2e-3
    assert float((got.data != ref.data).mean()) < 5e-3
    assert relrms(got.dequantize(), ref.dequantize()) < 1e-2
    with pytest.raises(ValueError):
        ResidentNVFP4(None, pa, pgu, output_dtype=torch.uint8, output_geglu=True, bias=bias)


def _device_packed(x, policy, global_scale=1.0):
    """NVFP4 operand packed on the device (bit-exact with pack_nvfp4, see test_quantizer_*): large weights in seconds."""
    data, scales = device_quantize(x, policy, global_scale)
    return PackedNVFP4(data, scales, np.float32(global_scale), x.shape)


def _oracle_product(pa, pb):
    """deq(A) . deq(B)^T: the oracle's dequantisation, the product in FP64 on the GPU (exact operands, so only the
    summation differs from the CPU oracle's; used where the CPU product would take minutes)."""
    a = torch.from_numpy(oracle.dequantize(pa.data, pa.scales, pa.global_scale, pa.data.shape[0:1] + (pa.data.shape[1] * 2,))).cuda().double()
    b = torch.from_numpy(oracle.dequantize(pb.data, pb.scales, pb.global_scale, pb.data.shape[0:1] + (pb.data.shape[1] * 2,))).cuda().double()
    return (a @ b.T).float().cpu().numpy()


def test_gemma_mlp_block_at_full_shape():
    """The Gemma-2B MLP block at its real size: X[768, 2048] -> RMSNorm -> NVFP4 -> gate/up 2048 -> 2 x 16384 with the
    GeGLU epilogue -> NVFP4 -> down 16384 -> 2048 + residual (BF16).  Every stage is checked against the oracle fed
    with the stage's actual input (N = 32768 output columns, K = 16384 = 256 K-groups through the operand ring), then
    the three stages run as one program and must reproduce the separate launches bit for bit."""
    from native_pi0.linear import NativeStageProgram
    rng = np.random.default_rng(2)
    m, width, mlp = 768, 2048, 16384
    x = bf16(rng.normal(size=(m, width)))
    gamma = torch.from_numpy((1 + rng.normal(scale=0.02, size=width)).astype(np.float32))
    gate = bf16(rng.normal(scale=0.02, size=(mlp, width))).float().numpy()
    up = bf16(rng.normal(scale=0.02, size=(mlp, width))).float().numpy()
    down = bf16(rng.normal(scale=0.02, size=(width, mlp))).float().numpy()
    gs_gu = float(max(np.abs(gate).max(), np.abs(up).max()) / (6 * 448))
    gs_dn = float(np.abs(down).max() / (6 * 448))
    p_gu = _device_packed(interleave_gate_up(gate, up), "ceil", gs_gu)
    p_dn = _device_packed(down, "ceil", gs_dn)
    placeholder_a = PackedNVFP4(np.zeros((m, width // 2), np.uint8), np.zeros((m, width // 16), np.uint8), np.float32(1), (m, width))
    placeholder_h = PackedNVFP4(np.zeros((m, mlp // 2), np.uint8), np.zeros((m, mlp // 16), np.uint8), np.float32(1), (m, mlp))
    with ResidentNorm(None, x, kind="rms", gamma=gamma, workers=148, row_alignment=128, keep_bf16=True) as norm, \
            ResidentNVFP4(None, placeholder_a, p_gu, workers=148, output_dtype=torch.uint8, output_geglu=True,
                          activation_buffers=(norm.output, norm.output_scales), tiled_weight=True) as gu, \
            ResidentNVFP4(None, placeholder_h, p_dn, workers=148, output_dtype=torch.bfloat16, residual=x,
                          activation_buffers=(gu.output, gu.output_scales), tiled_weight=True) as dn:
        norm.forward(); gu.forward(); y = dn.forward().float().cpu().numpy()
        for op in (norm, gu, dn):
            assert op.status()["code"] == 0
        # stage 1: normalised rows against the norm oracle, codes against the packer
        normalized = norm.normalized[:m].float().cpu()
        want = oracle_ops.norm(x, "rms", gamma, None)
        assert relrms(normalized.numpy(), want.numpy()) < 5e-3
        a_data = norm.output.cpu().numpy()
        a_scales = unswizzle_scales(norm.output_scales.cpu().numpy(), m, width // 16)
        ref = pack_nvfp4(normalized.numpy(), row_alignment=128)
        np.testing.assert_array_equal(a_data, ref.data)
        np.testing.assert_array_equal(a_scales, ref.scales)
        ideal = pack_nvfp4(want.numpy(), row_alignment=128)
        assert float((a_data != ideal.data).mean()) < 1e-2              # BF16 rounding ties of the normalised value
        # stage 2: GeGLU(gate, up) of the device's own stage-1 codes
        pa = PackedNVFP4(a_data, a_scales, np.float32(1), (m, width))
        acc = _oracle_product(pa, p_gu)
        hidden = oracle_ops.gelu_tanh(torch.from_numpy(acc[:, 0::2])).numpy() * acc[:, 1::2]
        ref_h = pack_nvfp4(hidden)
        got_h = _decode(gu, m, mlp)
        assert float((got_h.scales != ref_h.scales).mean()) < 2e-3
        assert float((got_h.data != ref_h.data).mean()) < 5e-3
        assert relrms(got_h.dequantize(), ref_h.dequantize()) < 1e-2
        # stage 3: down projection of the device's own stage-2 codes, + residual, one BF16 rounding
        out = _oracle_product(got_h, p_dn) + x.float().numpy()
        assert relrms(y, out) < 1e-2
        assert relrms(y, bf16(out).float().numpy()) < 3e-3
        # the same three stages as ONE launch with row-band dependencies
        for schedule in ("linear", "spread"):
            with NativeStageProgram(None, [(norm, []), (gu, [(0, 0)]), (dn, [(1, 0)])], workers=148, schedule=schedule) as program:
                dn.output.fill_(float("nan"))
                z = program.forward().float().cpu().numpy()
                assert program.status()["code"] == 0
                np.testing.assert_array_equal(z, y)


def test_residual_stream_epilogue_and_row_rms_consumer():
    """A folded RMSNorm between two NVFP4 projections: the producer writes its BF16 rows, their un-normalised NVFP4 copy
    and per-tile sums of squares; the consumer multiplies its accumulator rows by rsqrt(mean square + eps)."""
    lib = _native.load()
    rng = np.random.default_rng(97)
    m, k, n, n2 = 256, 512, 1024, 384
    a, w = rng.normal(size=(m, k)).astype(np.float32), rng.normal(scale=0.05, size=(n, k)).astype(np.float32)
    w2 = rng.normal(scale=0.05, size=(n2, n)).astype(np.float32)
    res = bf16(rng.normal(size=(m, n)))
    pa, pw, pw2 = pack_nvfp4(a), pack_nvfp4(w, scale_policy="ceil"), pack_nvfp4(w2, scale_policy="ceil")
    placeholder = pack_nvfp4(np.zeros((m, n), np.float32))
    for block_n in (128, 64, 32):
        parts = n // block_n
        with ResidentNVFP4(None, pa, pw, workers=16, output_dtype=torch.bfloat16, residual=res, block_n=block_n) as plain, \
                ResidentNVFP4(None, pa, pw, workers=16, output_dtype=torch.bfloat16, residual=res, block_n=block_n) as producer:
            want = plain.forward().clone()
            copy = torch.zeros(m, n // 2, dtype=torch.uint8, device="cuda")
            copy_scales = torch.zeros((m // 128) * (n // 64) * 512, dtype=torch.uint8, device="cuda")
            sumsq = torch.full((m, parts), float("nan"), dtype=torch.float32, device="cuda")
            _native.check(lib.configure_resident_fp4_stream(producer.handle, None, producer.residual.data_ptr(), producer.output.data_ptr(),
                                                            copy.data_ptr(), copy_scales.data_ptr(), 0.5, sumsq.data_ptr()), "stream")
            out = producer.forward()
            torch.cuda.synchronize()
            assert producer.status()["code"] == 0
            assert torch.equal(out, want)                                   # the BF16 rows are those of the plain epilogue
            ref = pack_nvfp4(out.float().cpu().numpy(), global_scale=0.5)   # the copy is the packer's image of those rows
            np.testing.assert_array_equal(copy.cpu().numpy(), ref.data)
            np.testing.assert_array_equal(unswizzle_scales(copy_scales.cpu().numpy(), m, n // 16), ref.scales)
            tiles = out.float().reshape(m, parts, block_n).square().sum(-1)
            assert relrms(sumsq.cpu().numpy(), tiles.cpu().numpy()) < 1e-6
            with ResidentNVFP4(None, placeholder, pw2, workers=8, activation_buffers=(copy, copy_scales)) as raw, \
                    ResidentNVFP4(None, placeholder, pw2, workers=8, activation_buffers=(copy, copy_scales)) as consumer:
                base = raw.forward().clone() * 0.5                        # (the wrapper's alpha assumes tensor scale 1 for the bound copy)
                _native.check(lib.configure_resident_fp4_row_rms(consumer.handle, sumsq.data_ptr(), parts, n, 1e-6), "row rms")
                got = consumer.forward() * 0.5
                factor = torch.rsqrt(out.float().square().mean(-1, keepdim=True) + 1e-6)
                assert relrms((got).cpu().numpy(), (base * factor).cpu().numpy()) < 1e-5
                assert lib.configure_resident_fp4_row_rms(consumer.handle, sumsq.data_ptr(), 6, n, 1e-6) == 1


def test_folded_layernorm_between_two_projections():
    """LayerNorm folded into the projection that follows: the producer leaves per-tile sums and sums of squares (row
    stride padded to a multiple of 4 slots), the consumer - weight columns times gamma, bias + W beta - turns its
    accumulator rows into rstd * (acc - mean * sum_k W'[n, k]).  Checked against LayerNorm + projection in FP32 on the
    operands the MMA reads (the dequantised copy and weight), for the BF16 and the NVFP4-output epilogue."""
    lib = _native.load()
    rng = np.random.default_rng(131)
    m, k, n, n2 = 256, 512, 1152, 384                        # 1152 / 64 = 18 tiles: the statistics rows are padded to 20 slots
    a, w = rng.normal(size=(m, k)).astype(np.float32), rng.normal(scale=0.05, size=(n, k)).astype(np.float32)
    res = bf16(rng.normal(loc=0.7, size=(m, n)))            # a row mean well away from zero
    gamma, beta = rng.normal(loc=1.0, scale=0.2, size=n).astype(np.float32), rng.normal(scale=0.3, size=n).astype(np.float32)
    w2 = rng.normal(scale=0.05, size=(n2, n)).astype(np.float32)
    b2 = rng.normal(scale=0.2, size=n2).astype(np.float32)
    folded = bf16(w2 * gamma[None, :]).float().numpy()
    pa, pw, pw2 = pack_nvfp4(a), pack_nvfp4(w, scale_policy="ceil"), pack_nvfp4(folded, scale_policy="ceil")
    w2_deq = oracle.dequantize(pw2.data, pw2.scales, pw2.global_scale, (n2, n))
    center = torch.from_numpy(w2_deq.sum(1).astype(np.float32)).cuda()
    bias2 = bf16(b2 + w2 @ beta)
    placeholder = pack_nvfp4(np.zeros((m, n), np.float32))
    block_n, ld = 64, 20
    with ResidentNVFP4(None, pa, pw, workers=16, output_dtype=torch.bfloat16, residual=res, block_n=block_n) as producer:
        copy = torch.zeros(m, n // 2, dtype=torch.uint8, device="cuda")
        copy_scales = torch.zeros((m // 128) * (n // 64) * 512, dtype=torch.uint8, device="cuda")
        sumsq, sums = torch.zeros((m, ld), device="cuda"), torch.zeros((m, ld), device="cuda")
        _native.check(lib.configure_resident_fp4_stream(producer.handle, None, producer.residual.data_ptr(), producer.output.data_ptr(),
                                                        copy.data_ptr(), copy_scales.data_ptr(), 1.0, sumsq.data_ptr()), "stream")
        _native.check(lib.configure_resident_fp4_stream_sums(producer.handle, sums.data_ptr(), ld), "stream sums")
        assert lib.configure_resident_fp4_stream_sums(producer.handle, sums.data_ptr(), 16) == 1       # fewer slots than tiles
        out = producer.forward().float()
        torch.cuda.synchronize()
        assert producer.status()["code"] == 0
        tiles = out.reshape(m, n // block_n, block_n)
        assert relrms(sums[:, :18].cpu().numpy(), tiles.sum(-1).cpu().numpy()) < 1e-5
        assert relrms(sumsq[:, :18].cpu().numpy(), tiles.square().sum(-1).cpu().numpy()) < 1e-6
        assert not sums[:, 18:].any() and not sumsq[:, 18:].any()
        x_deq = oracle.dequantize(copy.cpu().numpy(), unswizzle_scales(copy_scales.cpu().numpy(), m, n // 16), 1.0, (m, n))
        mean = out.mean(-1, keepdim=True).cpu().numpy()
        rstd = 1.0 / np.sqrt(out.var(-1, unbiased=False, keepdim=True).cpu().numpy() + 1e-6)
        want = rstd * (x_deq @ w2_deq.T - mean * w2_deq.sum(1)[None, :]) + bias2.float().numpy()[None, :]
        # the same thing the long way round: LayerNorm of the rows the MMA reads, then the projection
        direct = ((x_deq - mean) * rstd) @ w2_deq.T + bias2.float().numpy()[None, :]
        assert relrms(want, direct) < 1e-5
        for fp4_out in (False, True):
            kw = dict(output_dtype=torch.uint8, output_gelu=True, output_global_scale=0.5) if fp4_out else dict(output_dtype=torch.bfloat16)
            with ResidentNVFP4(None, placeholder, pw2, workers=8, bias=bias2, activation_buffers=(copy, copy_scales), **kw) as consumer:
                _native.check(lib.configure_resident_fp4_row_layernorm(consumer.handle, sumsq.data_ptr(), sums.data_ptr(), ld, n, 1e-6,
                                                                       center.data_ptr()), "row layernorm")
                got = consumer.forward()
                torch.cuda.synchronize()
                assert consumer.status()["code"] == 0
                if fp4_out:
                    got = oracle.dequantize(got.cpu().numpy(), unswizzle_scales(consumer.output_scales.cpu().numpy(), m, n2 // 16), 0.5, (m, n2))
                    ref = oracle_ops.gelu_tanh(torch.from_numpy(want)).numpy()
                    assert relrms(got, ref) < 0.12                               # one NVFP4 rounding of the activations
                else:
                    assert relrms(got.float().cpu().numpy(), want) < 4e-3        # BF16 rounding of the result


def test_gemm_qkv_rope_epilogue():
    lib = _native.load()
    rng = np.random.default_rng(71)
    rows, k, heads, hd = 200, 1024, 2, 256
    n = (heads + 2) * hd
    a, w = rng.normal(size=(256, k)).astype(np.float32), rng.normal(scale=0.03, size=(n, k)).astype(np.float32)
    half = hd // 2
    idx = np.stack((np.arange(half), np.arange(half) + half), 1).reshape(-1)
    wperm = w.copy()
    for h in range(heads + 1):                              # Q heads and the K head are stored pair-interleaved
        wperm[h * hd:(h + 1) * hd] = w[h * hd:(h + 1) * hd][idx]
    pa, pb = pack_nvfp4(a), pack_nvfp4(wperm, scale_policy="ceil")
    acc = oracle.gemm(pa.data, pa.scales, 1.0, pack_nvfp4(w, scale_policy="ceil").data, pack_nvfp4(w, scale_policy="ceil").scales, 1.0, 256, n, k)
    pos = torch.arange(37, 37 + rows).float()
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2).float() / hd))
    emb = torch.cat((pos[:, None] * inv[None], pos[:, None] * inv[None]), -1)
    cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()
    cosd, sind = torch.zeros(256, hd, dtype=torch.bfloat16), torch.zeros(256, hd, dtype=torch.bfloat16)
    cosd[:rows], sind[:rows] = cos, sin
    cosd, sind = cosd.cuda(), sind.cuda()
    qout = torch.zeros(256, heads * hd, dtype=torch.bfloat16, device="cuda")
    ck = torch.full((300, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    cv = torch.full((300, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    with ResidentNVFP4(None, pa, pb, workers=10, output_dtype=torch.bfloat16, rows=rows) as op:
        _native.check(lib.configure_resident_fp4_qkv_rope(op.handle, qout.data_ptr(), heads * hd, cosd.data_ptr(), sind.data_ptr(),
                                                          ck.data_ptr(), cv.data_ptr(), heads * hd, hd, 50), "rope")
        op.forward()
        torch.cuda.synchronize()
        assert op.status()["code"] == 0
    y = torch.from_numpy(acc[:rows]).bfloat16()
    for h in range(heads):
        want = oracle_ops.rope_interleaved(y[:, h * hd:(h + 1) * hd], cos, sin).float().numpy()
        got = qout[:rows, h * hd:(h + 1) * hd].float().cpu().numpy()
        assert relrms(got, want) < 4e-3 and float((got != want).mean()) < 0.02
    want_k = oracle_ops.rope_interleaved(y[:, heads * hd:(heads + 1) * hd], cos, sin).float().numpy()
    got_k = ck[50:50 + rows].float().cpu().numpy()
    assert relrms(got_k, want_k) < 4e-3
    got_v = cv[50:50 + rows].float().cpu().numpy()
    assert relrms(got_v, y[:, (heads + 1) * hd:].float().numpy()) < 4e-3
    assert (ck[:50] == 7).all() and (ck[50 + rows:] == 7).all() and not qout[rows:].any()


@pytest.mark.parametrize("rows,width,kind", [(51, 1024, "rms"), (768, 2048, "rms"), (256, 1152, "layer"), (7, 64, "layer")])
def test_norm_to_nvfp4(rows, width, kind):
    torch.manual_seed(83)
    x = torch.randn(rows, width).bfloat16()
    gamma = 1 + torch.randn(width) * 0.05
    beta = torch.randn(width) * 0.05 if kind == "layer" else None
    with ResidentNorm(None, x, kind=kind, gamma=gamma, beta=beta, workers=24, global_scale=0.5, row_alignment=128, keep_bf16=True) as op:
        op.forward()
        torch.cuda.synchronize()
        assert op.status()["code"] == 0
        normalized = op.normalized[:rows].float().cpu()
        data = op.output.cpu().numpy()
        scales = unswizzle_scales(op.output_scales.cpu().numpy(), data.shape[0], width // 16)
        first = data.copy()
        op.forward()
        np.testing.assert_array_equal(op.output.cpu().numpy(), first)
    want = oracle_ops.norm(x, kind, gamma, beta)
    assert relrms(normalized.numpy(), want.numpy()) < 5e-3
    assert float((normalized != want).float().mean()) < 0.02        # BF16 values equal except rounding ties
    ref = pack_nvfp4(normalized.numpy(), global_scale=0.5, row_alignment=128)   # CPU packer == device quantiser
    np.testing.assert_array_equal(data, ref.data)
    np.testing.assert_array_equal(scales, ref.scales)
    assert not data[rows:].any() and not scales[rows:].any()


def test_norm_residual_inverse_scale_fp8_and_factor_outputs():
    """The reference operator's remaining outputs (``scripts/validate_norm.py:95-130``): fused residual add with the sum
    kept for the next connection, AWQ-style inverse scale, FP8 E4M3 rows and the FP32 row factor."""
    torch.manual_seed(89)
    rows, width = 200, 1024
    x, r = torch.randn(rows, width).bfloat16(), (torch.randn(rows, width) * 0.1).bfloat16()
    gamma, awq = 1 + torch.randn(width) * 0.05, 0.5 + torch.rand(width)
    total = (x.float() + r.float()).bfloat16()
    want = oracle_ops.norm(total, "rms", gamma, None, round_normalized=False) * awq
    want = want.bfloat16().float()
    with ResidentNorm(None, x, kind="rms", precision="bf16", gamma=gamma, inverse_scale=awq, residual=r, workers=64) as op:
        got = op.forward()[:rows].float().cpu()
        assert op.status()["code"] == 0
        assert torch.equal(op.residual_output.cpu(), total)                 # the sum, rounded once, bit for bit
    assert relrms(got.numpy(), want.numpy()) < 5e-3 and float((got != want).float().mean()) < 0.02
    with ResidentNorm(None, x, kind="rms", precision="fp4", gamma=gamma, residual=r, workers=64, row_alignment=128, keep_bf16=True) as op:
        op.forward()
        torch.cuda.synchronize()
        ref = pack_nvfp4(op.normalized[:rows].float().cpu().numpy(), row_alignment=128)
        np.testing.assert_array_equal(op.output.cpu().numpy(), ref.data)
        assert relrms(op.normalized[:rows].float().cpu().numpy(), oracle_ops.norm(total, "rms", gamma, None).numpy()) < 5e-3
    y = oracle_ops.norm(x, "layer", gamma, awq * 0.1)                       # (beta reused from the random vector)
    with ResidentNorm(None, x, kind="layer", precision="fp8", gamma=gamma, beta=awq * 0.1, workers=64, global_scale=0.25) as op:
        fp8 = op.forward()[:rows].float().cpu() * 0.25
    assert relrms(fp8.numpy(), y.numpy()) < 0.04                            # E4M3: three mantissa bits
    assert float(((y / 0.25).to(torch.float8_e4m3fn).float() * 0.25 != fp8).float().mean()) < 0.02
    with ResidentNorm(None, x, kind="rms", precision="factor", workers=64) as op:
        factor = op.forward()[:rows].cpu()
    torch.testing.assert_close(factor, torch.rsqrt(x.float().square().mean(-1) + 1e-6), rtol=2e-6, atol=0)
    with pytest.raises(ValueError):
        ResidentNorm(None, x, kind="rms", precision="factor", gamma=gamma)


def test_norm_argument_errors():
    x = torch.randn(4, 64).bfloat16()
    with pytest.raises(ValueError):
        ResidentNorm(None, x.float())
    with pytest.raises(ValueError):
        ResidentNorm(None, x, kind="rms", beta=torch.zeros(64))
    with pytest.raises(ValueError):
        ResidentNorm(None, x, precision="int8")
    with pytest.raises(ValueError):
        ResidentNorm(None, torch.randn(4, 40).bfloat16())


ATTENTION_CASES = [
    # batches, nq, nk, heads, kv_heads, hd, prefix, splits
    (3, 256, 256, 16, 16, 72, None, 1),      # SigLIP
    (1, 768, 768, 8, 1, 256, None, 1),       # Gemma prefix, MQA
    (1, 200, 200, 4, 2, 256, None, 1),       # GQA, ragged rows
    (1, 51, 819, 8, 1, 256, 768, 1),         # action suffix over the cached prefix, state-row mask
    (1, 51, 819, 8, 1, 256, 768, 8),         # split-KV 8 + merge
    (1, 64, 848, 8, 1, 256, 784, 4),
    (1, 1, 5, 1, 1, 256, 2, 1),
    (1, 300, 500, 4, 1, 256, None, 3),       # split-KV over several 128-query tiles (ragged last tile)
    (1, 20, 300, 2, 1, 256, None, 1),        # <= 64 queries: the two warp groups share each chunk of keys
    (2, 40, 100, 4, 4, 72, None, 1),
    (1, 51, 819, 8, 1, 256, 768, 16),
]


@pytest.mark.parametrize("b,nq,nk,h,hk,hd,prefix,splits", ATTENTION_CASES)
def test_attention(b, nq, nk, h, hk, hd, prefix, splits):
    torch.manual_seed(419 + nq + nk)
    q = torch.randn(b, nq, h, hd).bfloat16().cuda()
    k = torch.randn(b, nk, hk, hd).bfloat16().cuda()
    v = torch.randn(b, nk, hk, hd).bfloat16().cuda()
    want = oracle_ops.attention(q, k, v, hd ** -0.5, prefix).numpy()
    with ResidentAttention(None, q, k, v, workers=64, prefix=prefix, splits=splits) as op:
        op.output.fill_(float("nan"))
        if splits > 1:
            op.poison_partials()          # a partial read before it is written in this launch would surface as NaN
        got = op.forward().float().cpu().numpy()
        assert op.status()["code"] == 0
        if splits > 1:
            op.poison_partials()
        again = op.forward().float().cpu().numpy()
        if splits > 1:
            state = op.read_split_counts()
            assert state["epoch"] == 2 and all(c == 2 * splits for c in state["counts"]), state
    assert np.isfinite(got).all()
    assert relrms(got, want) <= 1e-2
    np.testing.assert_array_equal(got, again)
    if splits > 1:
        # merge inside the attention stage (tiles of a head meet on a ticket): same bits as the separate merge stage, launch after launch
        with ResidentAttention(None, q, k, v, workers=128, prefix=prefix, splits=splits, fused_merge=True) as op:
            for launch in range(3):
                op.output.fill_(float("nan"))
                op.poison_partials()
                fused = op.forward().float().cpu().numpy()
                assert op.status()["code"] == 0
                np.testing.assert_array_equal(fused, got)
                state = op.read_split_counts()
                assert state["epoch"] == launch + 1 and all(c == (launch + 1) * splits for c in state["counts"]), state
    if prefix is not None and nq > 1:
        # the state query must not depend on keys beyond the prefix boundary
        k2, v2 = k.clone(), v.clone()
        k2[:, prefix + 1:] = 9.0
        v2[:, prefix + 1:] = -9.0
        with ResidentAttention(None, q, k2, v2, workers=64, prefix=prefix, splits=splits) as op:
            other = op.forward().float().cpu().numpy()
        np.testing.assert_array_equal(other[:, 0], got[:, 0])


TC_ATTENTION_CASES = [
    # batches, nq, nk, heads, kv_heads, head_dim, stored, prefix, splits
    (1, 768, 768, 8, 1, 256, 256, None, 3),      # Gemma prefix: 256 keys per tile
    (1, 784, 784, 8, 1, 256, 256, None, 4),      # with a 16-token prompt: 196 keys per tile, ragged last query tile
    (1, 200, 200, 4, 2, 256, 256, None, 1),      # GQA, one tile of keys, ragged rows
    (1, 51, 819, 8, 1, 256, 256, 768, 8),        # action suffix over the cache, state-row mask, 103 keys per tile
    (1, 51, 819, 8, 1, 256, 256, 768, 13),
    (1, 300, 500, 4, 1, 256, 256, None, 3),
    (1, 1, 5, 1, 1, 256, 256, 2, 1),
    (3, 256, 256, 16, 16, 72, 128, None, 1),     # SigLIP heads stored 128 apart
    (2, 40, 100, 4, 4, 72, 128, None, 1),
]


@pytest.mark.parametrize("b,nq,nk,h,hk,hd,stored,prefix,splits", TC_ATTENTION_CASES)
def test_attention_tensor_core_tiles(b, nq, nk, h, hk, hd, stored, prefix, splits):
    """The tcgen05 tiles (TMA operands, S / P / O in tensor memory) against the FP32 oracle and against the mma.sync
    tiles of the same operator."""
    torch.manual_seed(1000 + nq + nk + splits)
    def heads(rows, count):
        t = torch.zeros(b, rows, count, stored)
        t[..., :hd] = torch.randn(b, rows, count, hd)
        return t.bfloat16().cuda()
    q, k, v = heads(nq, h), heads(nk, hk), heads(nk, hk)
    want = oracle_ops.attention(q[..., :hd], k[..., :hd], v[..., :hd], hd ** -0.5, prefix).numpy()
    kw = dict(workers=148, prefix=prefix, splits=splits, head_dim=hd)
    with ResidentAttention(None, q, k, v, path="tcgen05", **kw) as op:
        for launch in range(2):
            op.output.fill_(float("nan"))
            if splits > 1:
                op.poison_partials()
            got = op.forward().float().cpu().numpy()
            assert op.status()["code"] == 0
            assert np.isfinite(got).all()
            assert relrms(got, want) <= 1e-2
            if launch:
                np.testing.assert_array_equal(got, first)
            first = got
    with ResidentAttention(None, q, k, v, path="mma.sync", **kw) as op:
        legacy = op.forward().float().cpu().numpy()
    assert relrms(got, legacy) <= 5e-3                      # two evaluations in BF16 probabilities: rounding apart
    tiles = b * ((nq + 127) // 128) * h * splits
    if splits > 1 and tiles <= 148:                         # (the tiles of a head meet inside the stage: one worker each)
        with ResidentAttention(None, q, k, v, path="tcgen05", fused_merge=True, **kw) as op:
            fused = op.forward().float().cpu().numpy()
            assert op.status()["code"] == 0
        np.testing.assert_array_equal(fused, got)           # the merge inside the stage: same bits as the merge stage
    if prefix is not None and nq > 1:
        k2, v2 = k.clone(), v.clone()
        k2[:, prefix + 1:] = 9.0
        v2[:, prefix + 1:] = -9.0
        with ResidentAttention(None, q, k2, v2, path="tcgen05", **kw) as op:
            other = op.forward().float().cpu().numpy()
        np.testing.assert_array_equal(other[:, 0], got[:, 0])


@pytest.mark.parametrize("b,nq,nk,h,hk,hd,splits,bias,rope,mask,prefix", [
    (2, 100, 180, 4, 2, 64, 1, True, True, False, None),     # the Cosmos head sizes, GQA, biases and rotary tables
    (1, 200, 200, 4, 4, 128, 1, True, True, True, None),
    (1, 300, 600, 4, 1, 128, 3, False, True, True, None),    # more than 256 keys: KV splits, merge stage
    (2, 40, 100, 16, 16, 72, 1, True, False, True, None),    # 72-wide heads through the prepared (padded) layout
    (1, 51, 819, 8, 1, 256, 8, False, False, True, 768),     # boolean mask on top of the suffix mask, no preparation stage
    (1, 64, 64, 2, 2, 256, 1, True, True, False, None),
])
def test_attention_bias_rope_mask_and_head_sizes(b, nq, nk, h, hk, hd, splits, bias, rope, mask, prefix):
    """The operator's optional arguments (``native_pi0/attention.py:19-20`` of the reference) against the FP32 oracle that
    restates the reference validator: per-head biases, rotate-half tables, a boolean visibility mask (rows without a
    visible key give zeros), head sizes 64 / 128."""
    g = torch.Generator().manual_seed(2000 + nq + hd + splits)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    q, k, v = rand(b, nq, h, hd).bfloat16().cuda(), rand(b, nk, hk, hd).bfloat16().cuda(), rand(b, nk, hk, hd).bfloat16().cuda()
    biases = [(rand(n, hd) * 0.5).bfloat16() for n in (h, hk, hk)] if bias else None
    def tables(rows):
        angle = torch.rand(b, rows, hd, generator=g) * 6.28
        return angle.cos().bfloat16(), angle.sin().bfloat16()
    q_rope, k_rope = (tables(nq), tables(nk)) if rope else (None, None)
    visible = None
    if mask:
        visible = torch.rand(b, nq, nk, generator=g) < 0.7
        visible[:, 3] = False                                # a query that sees nothing
        if prefix is not None:
            visible[:, 0] = True
    want = oracle_ops.attention(q, k, v, hd ** -0.5, prefix, bias=biases, q_rope=q_rope, k_rope=k_rope, mask=visible).numpy()
    with ResidentAttention(None, q, k, v, workers=148, prefix=prefix, splits=splits, bias=biases, q_rope=q_rope, k_rope=k_rope,
                           mask=visible) as op:
        for launch in range(2):
            op.output.fill_(float("nan"))
            got = op.forward().float().cpu().numpy()
            assert op.status()["code"] == 0
            assert np.isfinite(got).all()
            assert relrms(got, want) <= 1e-2
            if mask:
                assert not got[:, 3].any()
            if launch:
                np.testing.assert_array_equal(got, first)
            first = got


def test_attention_optional_argument_errors():
    q = torch.randn(1, 64, 2, 128).bfloat16().cuda()
    k = torch.randn(1, 600, 2, 128).bfloat16().cuda()
    with pytest.raises(RuntimeError):
        ResidentAttention(None, q, k, k)                     # 600 keys in one tcgen05 tile: prepared operands need KV splits
    with pytest.raises(ValueError):
        ResidentAttention(None, q, k, k, splits=3, bias=(torch.zeros(2, 64), None, None))      # bias shape
    with pytest.raises(ValueError):
        ResidentAttention(None, q, k, k, splits=3, q_rope=(torch.zeros(1, 64, 128), None))     # cosine without sine
    with pytest.raises(ValueError):
        ResidentAttention(None, q, k, k, splits=3, mask=torch.ones(1, 64, 599, dtype=torch.bool))
    with ResidentAttention(None, q, k, k, splits=3, path="tcgen05") as op:
        op.forward()
        assert op.status()["code"] == 0
    with pytest.raises(RuntimeError):
        ResidentAttention(None, q, k, k, splits=3, path="mma.sync")                             # prepared operands: tcgen05 tiles only


def test_attention_path_selection():
    q = torch.randn(1, 64, 2, 256).bfloat16().cuda()
    k = torch.randn(1, 600, 1, 256).bfloat16().cuda()
    with pytest.raises(RuntimeError):
        ResidentAttention(None, q, k, k, path="tcgen05")    # 600 keys in one tile: needs KV splits
    with ResidentAttention(None, q, k, k, path="tcgen05", splits=3) as op:
        op.forward()
        assert op.status()["code"] == 0
    small = torch.randn(1, 8, 2, 72).bfloat16().cuda()
    with pytest.raises(RuntimeError):
        ResidentAttention(None, small, small, small, path="tcgen05")     # 72-wide heads need the padded layout


def test_attention_fused_fp4_output():
    torch.manual_seed(5)
    nq, nk, h, hd = 100, 300, 8, 256
    q, k, v = [torch.randn(1, n, hh, hd).bfloat16().cuda() for n, hh in ((nq, h), (nk, 1), (nk, 1))]
    data = torch.zeros(128, h * hd // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros((h * hd // 64) * 512, dtype=torch.uint8, device="cuda")
    for splits in (1, 3):
        data.zero_(), scales.zero_()
        with ResidentAttention(None, q, k, v, workers=32, fp4_output=(data, scales, 0.25), splits=splits) as op:
            out = op.forward().float().cpu().numpy().reshape(nq, h * hd)
            assert op.status()["code"] == 0
        ref = pack_nvfp4(out, global_scale=0.25, row_alignment=128)
        np.testing.assert_array_equal(data.cpu().numpy(), ref.data)         # quantiser consumed the BF16 rows it stored
        np.testing.assert_array_equal(unswizzle_scales(scales.cpu().numpy(), 128, h * hd // 16), ref.scales)


@pytest.mark.parametrize("b,nq,nk,h,hd,stored,pitch", [(1, 100, 200, 8, 256, 256, 256), (3, 256, 256, 16, 72, 128, 80), (1, 40, 100, 4, 72, 128, 80)])
def test_attention_tensor_core_fp4_output(b, nq, nk, h, hd, stored, pitch):
    """NVFP4 rows straight from the unsplit tcgen05 tile: the quantiser of the BF16 rows the same launch stores, with every
    head on `pitch` columns (72-wide SigLIP heads on 80: zeros behind each head, no block straddles two heads)."""
    torch.manual_seed(17 + nq)
    def heads(rows):
        t = torch.zeros(b, rows, h, stored)
        t[..., :hd] = torch.randn(b, rows, h, hd)
        return t.bfloat16().cuda()
    q, k, v = heads(nq), heads(nk), heads(nk)
    rows = b * nq
    rows_pad = (rows + 127) // 128 * 128
    data = torch.zeros(rows_pad, h * pitch // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros((rows_pad // 128) * (h * pitch // 64) * 512, dtype=torch.uint8, device="cuda")
    with ResidentAttention(None, q, k, v, workers=148, head_dim=hd, fp4_output=(data, scales, 0.5), fp4_pitch=pitch, path="tcgen05") as op:
        for _ in range(2):
            out = op.forward().float().cpu().numpy().reshape(rows, h, hd)
            assert op.status()["code"] == 0
    want = oracle_ops.attention(q[..., :hd], k[..., :hd], v[..., :hd], hd ** -0.5, None).numpy().reshape(rows, h, hd)
    assert relrms(out, want) <= 1e-2
    spread = np.zeros((rows, h, pitch), dtype=np.float32)
    spread[..., :hd] = out
    ref = pack_nvfp4(spread.reshape(rows, h * pitch), global_scale=0.5, row_alignment=128)
    np.testing.assert_array_equal(data.cpu().numpy()[:rows], ref.data[:rows])
    np.testing.assert_array_equal(unswizzle_scales(scales.cpu().numpy(), rows_pad, h * pitch // 16)[:rows], ref.scales[:rows])
    if pitch != hd:
        with pytest.raises(RuntimeError):                   # only the unsplit tcgen05 tile writes a pitch other than head_dim
            ResidentAttention(None, q, k, v, head_dim=hd, fp4_output=(data, scales, 0.5), fp4_pitch=pitch, path="mma.sync")
        with pytest.raises(RuntimeError):
            ResidentAttention(None, q, k, v, head_dim=hd, fp4_output=(data, scales, 0.5), fp4_pitch=72)


def test_small_operators():
    lib = _native.load()
    torch.manual_seed(11)
    dev = "cuda"
    # patch embedding vs conv2d
    views, width = 2, 1152
    images = (torch.rand(views, 224, 224, 3, device=dev) * 2 - 1).contiguous()
    conv_w = torch.randn(width, 3, 14, 14, device=dev) * 0.02
    conv_b, pos = torch.randn(width, device=dev) * 0.02, torch.randn(256, width, device=dev) * 0.02
    w = conv_w.permute(2, 3, 1, 0).reshape(588, width).contiguous()
    out = torch.zeros(views * 256, width, dtype=torch.bfloat16, device=dev)
    h = C.c_void_p()
    _native.check(lib.create_patch_embed(C.byref(h), images.data_ptr(), w.data_ptr(), conv_b.data_ptr(), pos.data_ptr(), out.data_ptr(), views, width, 100), "patch")
    _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    want = torch.nn.functional.conv2d(images.permute(0, 3, 1, 2), conv_w, conv_b, stride=14).flatten(2).transpose(1, 2) + pos[None]
    assert relrms(out.float().cpu().numpy(), want.reshape(-1, width).bfloat16().float().cpu().numpy()) < 2e-3
    lib.destroy_op(h)
    # FP32 linear: bias + SiLU
    rows, n, k = 50, 1024, 32
    x, wl, b = torch.randn(rows, k, device=dev), torch.randn(n, k, device=dev) * 0.1, torch.randn(n, device=dev)
    o = torch.zeros(rows, n, device=dev)
    h = C.c_void_p()
    _native.check(lib.create_linear32(C.byref(h), x.data_ptr(), wl.data_ptr(), b.data_ptr(), None, o.data_ptr(), rows, n, k, k, n, 4, 0, 0, 0, 0.0, 1e-6, 64), "lin")
    _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    torch.testing.assert_close(o, torch.nn.functional.silu(x @ wl.T + b), rtol=1e-5, atol=1e-5)
    lib.destroy_op(h)
    # FP32 1024 -> 1024 with BF16 output one row below an extra row (the state token joining the action tokens)
    rows, n, k = 50, 1024, 1024
    x, wl, b = torch.randn(rows, k, device=dev), torch.randn(n, k, device=dev) * 0.03, torch.randn(n, device=dev)
    row0 = torch.randn(n, device=dev)
    ob = torch.zeros(128, n, dtype=torch.bfloat16, device=dev)
    h = C.c_void_p()
    _native.check(lib.create_linear32(C.byref(h), x.data_ptr(), wl.data_ptr(), b.data_ptr(), None, ob[1:].data_ptr(), rows, n, k, k, n, 2, 0, 0, 0,
                                      0.0, 1e-6, 64), "lin")
    _native.check(lib.configure_linear32_extra_row(h, row0.data_ptr(), ob.data_ptr()), "extra row")
    for _ in range(2):
        _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    torch.testing.assert_close(ob[1:51].float(), (x.double() @ wl.double().T + b).float().bfloat16().float(), rtol=1e-2, atol=1e-2)
    assert float((ob[1:51].float() - (x.double() @ wl.double().T + b).float()).abs().max()) < 2e-2
    assert torch.equal(ob[0], row0.bfloat16()) and not ob[51:].any()
    lib.destroy_op(h)
    # BF16 input with row offset, RMS factor and Euler update
    rows, n, k = 50, 32, 1024
    xb = torch.randn(128, k, device=dev).bfloat16()
    wl, b, prev = torch.randn(n, k, device=dev) * 0.05, torch.randn(n, device=dev), torch.randn(rows, n, device=dev)
    o = prev.clone()
    h = C.c_void_p()
    _native.check(lib.create_linear32(C.byref(h), xb.data_ptr(), wl.data_ptr(), b.data_ptr(), o.data_ptr(), o.data_ptr(), rows, n, k, k, n,
                                      1 | 8 | 16, 0, 0, 1, -0.1, 1e-6, 4), "lin")
    _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    xf = xb[1:51].float()
    val = (xf @ wl.T) * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6) + b
    torch.testing.assert_close(o, prev + (-0.1) * val, rtol=2e-5, atol=2e-5)
    lib.destroy_op(h)
    # suffix assembly and token embedding
    state_emb, act = torch.randn(1, 1024, device=dev), torch.randn(50, 1024, device=dev)
    xs = torch.zeros(128, 1024, dtype=torch.bfloat16, device=dev)
    h = C.c_void_p()
    _native.check(lib.create_suffix_assemble(C.byref(h), state_emb.data_ptr(), act.data_ptr(), xs.data_ptr(), 50, 1024, 8), "suffix")
    _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    assert torch.equal(xs[:51], torch.cat((state_emb, act)).bfloat16()) and not xs[51:].any()
    lib.destroy_op(h)
    table = (torch.randn(1000, 2048, device=dev) * 0.02).bfloat16()
    tokens = torch.randint(0, 1000, (1, 16), device=dev)
    xt = torch.zeros(896, 2048, dtype=torch.bfloat16, device=dev)
    h = C.c_void_p()
    _native.check(lib.create_token_embed(C.byref(h), tokens.data_ptr(), table.data_ptr(), xt.data_ptr(), 16, 2048, 768, 1000, float(2048 ** 0.5), 8), "embed")
    _native.check(lib.launch_op(h, None), "launch")
    torch.cuda.synchronize()
    assert torch.equal(xt[768:784], (table[tokens[0]].float() * torch.tensor(2048 ** 0.5).float()).bfloat16())
    assert not xt[:768].any() and not xt[784:].any()
    lib.destroy_op(h)


def test_argument_errors_return_codes():
    lib = _native.load()
    h = C.c_void_p(123)
    assert lib.create_resident_fp4(C.byref(h), None, None, None, None, None, 128, 128, 64, 1, 1.0) == 1
    assert h.value is None
    buf = torch.zeros(128 * 64, dtype=torch.uint8, device="cuda")
    assert lib.create_resident_fp4(C.byref(h), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 100, 128, 64, 1, 1.0) == 1
    assert lib.create_resident_fp4(C.byref(h), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 128, 128, 64, 100000, 1.0) == 9
    assert lib.destroy_resident_fp4(None) == 0 and lib.destroy_native_model(None) == 0 and lib.destroy_norm(None) == 0
    assert lib.launch_resident_fp4(None, None) == 1
