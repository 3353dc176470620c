"""Dense BF16 / FP8 projections (``ResidentDense``) through the C ABI against PyTorch FP32 arithmetic on the same
operands.  The product is exact in FP32 up to summation order, so FP32 outputs are held to 2e-5 relative RMS
(stated bar 1e-2); the BF16 epilogues are then checked the way the reference does (``scripts/validate_epilogues.py
:43-53``): bit for bit against the formula applied to the operator's own FP32 result.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0.dense import ResidentDense, head_order
from native_pi0.linear import NativeStageProgram
from oracle import ops as oracle_ops


def relrms(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def operands(m, n, k, seed, scale=0.05):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(m, k, generator=g).bfloat16().cuda(), (torch.randn(n, k, generator=g) * scale).bfloat16().cuda()


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 128), (256, 384, 1152), (768, 2560, 2048), (100, 200, 300), (128, 2048, 16384)])
def test_bf16_product_matches_fp32(m, n, k):
    a, b = operands(m, n, k, 11 + m + n + k)
    want = a.float() @ b.float().T
    with ResidentDense(None, a, b, output_dtype=torch.float32, alpha=0.5) as op:
        got = op.forward().clone()
        assert op.status()["code"] == 0
        again = op.forward()
        assert torch.equal(got, again)
        padded = op.output
    assert relrms(got, 0.5 * want) <= 2e-5
    assert not padded[m:].any()                              # rows beyond the logical count are never stored


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 640, 1024), (90, 300, 2048)])
def test_fp8_product_matches_fp32(m, n, k):
    g = torch.Generator().manual_seed(5 + k)
    a = torch.randn(m, k, generator=g).cuda().to(torch.float8_e4m3fn)
    b = (torch.randn(n, k, generator=g) * 0.5).cuda().to(torch.float8_e4m3fn)
    want = (a.float() @ b.float().T) * 0.03125
    with ResidentDense(None, a, b, output_dtype=torch.float32, alpha=0.03125) as op:
        got = op.forward().clone()
        assert op.status()["code"] == 0
    assert relrms(got, want) <= 2e-5
    with ResidentDense(None, a, b, output_dtype=torch.bfloat16, alpha=0.03125) as op:
        assert torch.equal(op.forward(), got.bfloat16())


def test_bf16_epilogues_are_bit_exact_against_the_fp32_result():
    m, n, k = 200, 384, 512
    a, b = operands(m, n, k, 3)
    g = torch.Generator().manual_seed(4)
    bias = torch.randn(n, generator=g).bfloat16().cuda()
    residual = torch.randn(m, n, generator=g).bfloat16().cuda()
    with ResidentDense(None, a, b, output_dtype=torch.float32) as op:
        fp32 = op.forward().clone()
    for use_bias in (False, True):
        for use_res in (False, True):
            want = fp32.clone()
            if use_res:
                want += residual.float()
            if use_bias:
                want += bias.float()
            with ResidentDense(None, a, b, bias=bias if use_bias else None, residual=residual if use_res else None) as op:
                for _ in range(2):
                    assert torch.equal(op.forward(), want.bfloat16()), (use_bias, use_res)
            # FP32 output takes bias and residual too
            with ResidentDense(None, a, b, output_dtype=torch.float32, bias=bias if use_bias else None,
                               residual=residual if use_res else None) as op:
                assert torch.equal(op.forward(), want)
    # OpenPI-eager residual: the projection (+bias) is rounded to BF16 before the residual add
    with ResidentDense(None, a, b, bias=bias, residual=residual, round_before_residual=True) as op:
        want = ((fp32 + bias.float()).bfloat16().float() + residual.float()).bfloat16()
        assert torch.equal(op.forward(), want)
    # row factors (1/rms of un-normalised rows)
    factors = torch.zeros(256, dtype=torch.float32, device="cuda")
    factors[:m] = torch.rand(m, generator=g).cuda() + 0.5
    with ResidentDense(None, a, b, rms_factors=factors) as op:
        got = op.forward()
    want = (fp32 * factors[:m, None]).bfloat16()
    assert float((got != want).float().mean()) < 1e-3 and relrms(got, want) < 1e-3      # alpha * factor is one FP32 product here
    with pytest.raises(ValueError):
        ResidentDense(None, a, b, rms_factors=factors, bias=bias)
    with pytest.raises(ValueError):
        ResidentDense(None, a, b, round_before_residual=True)
    with pytest.raises(ValueError):
        ResidentDense(None, a, b.float())


def test_gelu_and_geglu_epilogues():
    m, n, k = 256, 512, 1152
    a, b = operands(m, n, k, 9, scale=0.03)
    g = torch.Generator().manual_seed(10)
    bias = (torch.randn(n, generator=g) * 0.5).bfloat16().cuda()
    with ResidentDense(None, a, b, output_dtype=torch.float32, bias=bias) as op:
        fp32 = op.forward().clone()
    # GELU(tanh) of the BF16-rounded projection; a logical width below the padded one leaves zeros behind it
    with ResidentDense(None, a, b[:500], bias=bias[:500], gelu=True) as op:
        got = op.forward()
        padded = op.output
    want = oracle_ops.gelu_tanh(fp32[:, :500].bfloat16().float()).bfloat16()
    assert float((got != want).float().mean()) < 2e-3 and relrms(got, want) < 2e-3      # tanh differs in the last bit now and then
    assert not padded[:, 500:].any()
    # compact GeGLU: interleaved gate/up rows of the weight -> [M, N/2]
    gate, up = b[: n // 2], b[n // 2:]
    interleaved = torch.stack((gate, up), dim=1).reshape(n, k)
    with ResidentDense(None, a, interleaved, output_dtype=torch.float32) as op:
        acc = op.forward().clone()
    compact = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda")
    with ResidentDense(None, a, interleaved, geglu_output=compact) as op:
        got = op.forward()
        assert got.data_ptr() == compact.data_ptr()
    gate_v, up_v = acc[:, 0::2].bfloat16().float(), acc[:, 1::2].bfloat16().float()
    want = (oracle_ops.gelu_tanh(gate_v).bfloat16().float() * up_v).bfloat16()
    assert float((got != want).float().mean()) < 2e-3 and relrms(got, want) < 2e-3


def test_skinny_and_qkv_rope_epilogue():
    rows, k, heads = 51, 1024, 8
    n = (heads + 2) * 256
    a, w = operands(rows, n, k, 21, scale=0.03)
    pos = torch.arange(768, 768 + rows).float()
    inv = 1.0 / (10000 ** (torch.arange(0, 256, 2).float() / 256))
    emb = torch.cat((pos[:, None] * inv[None], pos[:, None] * inv[None]), -1)
    cos, sin = emb.cos().bfloat16().cuda()[None].contiguous(), emb.sin().bfloat16().cuda()[None].contiguous()
    cache_k = torch.full((1, 900, 1, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    cache_v = torch.full((1, 900, 1, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    with ResidentDense(None, a, w, output_dtype=torch.float32) as op:
        y = op.forward().clone().bfloat16()                  # the projection output as the BF16 model sees it
    with ResidentDense(None, a, w, skinny=True) as op:
        assert torch.equal(op.forward(), y)
        assert not op.output[64:].any()
    with ResidentDense(None, a, w, skinny=True, rope=(cos, sin), kv_cache=(cache_k, cache_v), rope_key_offset=heads * 256, cache_base=768) as op:
        out = op.forward().clone()
        assert op.status()["code"] == 0
    order = head_order("cuda")
    for h in range(heads):
        want = oracle_ops.rope_interleaved(y[:, h * 256:(h + 1) * 256].cpu(), cos[0].cpu(), sin[0].cpu()).cuda()
        got = out[:, h * 256:(h + 1) * 256]
        assert relrms(got, want) < 4e-3 and float((got != want).float().mean()) < 0.02
    want_k = oracle_ops.rope_interleaved(y[:, heads * 256:(heads + 1) * 256].cpu(), cos[0].cpu(), sin[0].cpu()).cuda()
    assert relrms(cache_k[0, 768:768 + rows, 0], want_k) < 4e-3
    assert torch.equal(cache_v[0, 768:768 + rows, 0], y[:, (heads + 1) * 256:])
    assert (cache_k[0, :768] == 7).all() and (cache_k[0, 768 + rows:] == 7).all()
    assert order.shape == (256,) and sorted(order.tolist()) == list(range(256))


def test_two_dense_stages_in_one_launch():
    """A BF16 chain in one persistent launch (the reference's NativeLinearProgram case): stage 1 reads stage 0's
    output band by band; same bits as the separate launches."""
    m, k, n0, n1 = 384, 512, 1024, 256
    a, w0 = operands(m, n0, k, 31)
    _, w1 = operands(1, n1, n0, 32)
    mid = torch.zeros(m, n0, dtype=torch.bfloat16, device="cuda")
    with ResidentDense(None, a, w0, output_buffer=mid, gelu=True) as s0, \
            ResidentDense(None, mid, w1, input_buffer=mid, output_dtype=torch.float32) as s1:
        s0.forward()
        want = s1.forward().clone()
        ref = oracle_ops.gelu_tanh((a.float() @ w0.float().T).bfloat16().float()).bfloat16().float() @ w1.float().T
        assert relrms(want, ref) < 2e-3
        with NativeStageProgram(None, [(s0, []), (s1, [(0, 0)])], workers=20) as program:
            mid.fill_(float("nan"))
            s1.output.fill_(float("nan"))
            got = program.forward()
            assert program.status()["code"] == 0
            assert torch.equal(got[:m, :n1], want)
