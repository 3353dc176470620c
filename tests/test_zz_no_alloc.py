"""The allocation-free split-KV attention entry point against the ordinary attention operator.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other
test.  Some callers - a control loop that must not block on the driver's allocator, a process whose device memory
is owned by another pool - cannot obtain scratch memory when they need attention; ``attention_split_noalloc`` keeps
its split-KV partials in a fixed device array inside the library instead.  The check: two calls in a row through
the C ABI (different inputs, so stale partials of the first call would show in the second) reproduce the output of
``create_attention`` + ``configure_attention_splits`` bit for bit - with at most 64 queries (the two warp groups
share every key chunk), with 65..128 queries (each warp owns its rows) and with one part per head (no partials at
all) - stay within 1e-2 NRMSE of the FP32 attention oracle, and sizes beyond the array are rejected.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0 import _native
from native_pi0.attention import ResidentAttention
from oracle import ops as oracle_ops


def run_reference(q, k, v, prefix, splits):
    # the allocation-free entry point runs the mma.sync tiles: compare with the operator on the same tiles
    with ResidentAttention(None, q, k, v, workers=64, prefix=prefix, splits=splits, path="mma.sync") as op:
        out = op.forward().clone()
        assert op.status()["code"] == 0
    return out


def hd_scale(hd):
    return float(hd ** -0.5)


def run_noalloc(lib, q, k, v, prefix, splits):
    _, nq, heads, hd = q.shape
    _, nk, kv_heads, _ = k.shape
    out = torch.full((1, nq, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    code = lib.attention_split_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), nq, nk, heads, kv_heads, hd,
                                       heads * hd, kv_heads * hd, heads * hd, -1 if prefix is None else prefix, splits,
                                       float(hd ** -0.5), torch.cuda.current_stream().cuda_stream)
    assert code == 0, code
    torch.cuda.synchronize()
    return out


def test_noalloc_attention_matches_operator_twice():
    lib = _native.load()
    torch.manual_seed(2024)
    # second call: fewer parts, leaves stale partials behind; third: more than 64 queries; fourth: one part per head
    cases = [(51, 819, 8, 768, 8), (64, 300, 4, None, 5), (100, 420, 8, None, 3), (51, 819, 8, 768, 1)]
    for nq, nk, heads, prefix, splits in cases:
        q = torch.randn(1, nq, heads, 256, device="cuda").bfloat16()
        k = torch.randn(1, nk, 1, 256, device="cuda").bfloat16()
        v = torch.randn(1, nk, 1, 256, device="cuda").bfloat16()
        want = run_reference(q, k, v, prefix, splits)
        got = run_noalloc(lib, q, k, v, prefix, splits)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)                          # same kernels' arithmetic, same order: bit-exact
        ref = oracle_ops.attention(q, k, v, hd_scale(256), prefix)
        err = float((got.float().cpu() - ref).norm() / ref.norm())
        assert err <= 1e-2, (nq, nk, splits, err)
    # the same inputs again after other data went through the shared array
    again = run_noalloc(lib, q, k, v, prefix, splits)
    assert torch.equal(again, want)


def test_noalloc_attention_rejects_sizes_beyond_the_array():
    lib = _native.load()
    q = torch.zeros(1, 16, 8, 256, device="cuda").bfloat16()
    k = torch.zeros(1, 32, 1, 256, device="cuda").bfloat16()
    out = torch.zeros_like(q)
    args = lambda nq, heads, hd, splits: (q.data_ptr(), k.data_ptr(), k.data_ptr(), out.data_ptr(), nq, 32, heads, 1, hd,
                                          heads * hd, hd, heads * hd, -1, splits, 0.0625, None)
    assert lib.attention_split_noalloc(*args(16, 8, 256, 9)) == 1       # heads * splits > 64
    assert lib.attention_split_noalloc(*args(129, 8, 256, 2)) == 1      # more than 128 queries
    assert lib.attention_split_noalloc(*args(16, 8, 128, 2)) == 1       # head_dim other than 256
    assert lib.attention_split_noalloc(*args(16, 8, 256, 0)) == 1       # no parts at all
    assert lib.attention_split_noalloc(q.data_ptr() + 2, k.data_ptr(), k.data_ptr(), out.data_ptr(), 16, 32, 8, 1, 256, 2048, 256, 2048, -1, 2,
                                       0.0625, None) == 1               # rows move in 16-byte pieces: unaligned pointers are refused
    assert lib.attention_split_noalloc(None, k.data_ptr(), k.data_ptr(), out.data_ptr(), 16, 32, 8, 1, 256, 2048, 256, 2048, -1, 2, 0.0625, None) == 1
