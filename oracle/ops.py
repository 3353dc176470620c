"""Per-operator CPU/PyTorch oracles (TEST INFRASTRUCTURE).

* ``attention`` restates the reference validator's independent FP32 attention
  (``scripts/validate_attention.py:24-42``): optional per-head biases added to Q/K/V, optional rotate-half tables
  applied to Q and K (only the first half of each table is read), GQA by repeating KV heads, scale, the pi0 suffix
  mask (query 0 sees keys ``<= prefix``), an optional boolean visibility mask, softmax with fully masked rows -> 0.
  Pinned by ``tests/golden/attention.npz``, which holds outputs of that reference function itself.
* ``norm`` restates ``scripts/validate_norm.py:104-111``: optional mean removal, rsqrt(mean square + eps),
  gamma, beta, optional BF16 rounding of the normalised value.
* ``gelu_tanh`` is ``0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3)))`` (``native_pi0/dense.cu:53``).
"""
import torch


def _rotate_half(x, tables):
    """x [B,N,H,d] FP32; tables (cos, sin) [B,N,d]: (lo, hi) -> (lo c - hi s, hi c + lo s) with the first-half angles."""
    half = x.shape[-1] // 2
    cos, sin = [t.float().cpu()[..., :half].unsqueeze(2) for t in tables]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1)


def attention(q, k, v, scale, prefix=None, *, bias=None, q_rope=None, k_rope=None, mask=None):
    """q [B,Nq,H,d], k/v [B,Nk,Hk,d] -> FP32 [B,Nq,H,d].  bias: three [heads, d] tensors or Nones (q, k, v);
    q_rope / k_rope: (cos, sin) tables [B, rows, d]; mask: bool [B, Nq, Nk], True = visible."""
    q, k, v = [x.float().cpu().clone() for x in (q, k, v)]
    if bias is not None:
        q, k, v = [x if b is None else x + b.float().cpu() for x, b in zip((q, k, v), bias)]
    if q_rope is not None:
        q = _rotate_half(q, q_rope)
    if k_rope is not None:
        k = _rotate_half(k, k_rope)
    groups = q.shape[2] // k.shape[2]
    k = k.repeat_interleave(groups, 2)
    v = v.repeat_interleave(groups, 2)
    score = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    visible = torch.ones((q.shape[0], q.shape[1], k.shape[1]), dtype=torch.bool)
    if prefix is not None:
        visible[:, 0, prefix + 1:] = False
    if mask is not None:
        visible = visible & mask.cpu()
    score = score.masked_fill(~visible[:, None], float("-inf"))
    prob = torch.softmax(score, dim=-1).nan_to_num(0)
    return torch.einsum("bhqk,bkhd->bqhd", prob, v)


def norm(x, kind, gamma=None, beta=None, eps=1e-6, round_normalized=True):
    y = x.float()
    if kind == "layer":
        y = y - y.mean(-1, keepdim=True)
    y = y * torch.rsqrt(y.square().mean(-1, keepdim=True) + eps)
    if gamma is not None:
        y = y * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.bfloat16().float() if round_normalized else y


def gelu_tanh(x):
    return 0.5 * x * (1 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def rope_interleaved(x, cos, sin):
    """Reference rotate-half RoPE on rows x [rows, hd] in BF16 product rounding, returned in the engine's
    pair-interleaved head layout (column 2i = dim i, column 2i+1 = dim i + hd/2)."""
    hd = x.shape[-1]
    half = hd // 2
    xb = x.bfloat16()
    rot = torch.cat((-xb[..., half:], xb[..., :half]), dim=-1)
    out = (xb * cos.bfloat16()) + (rot * sin.bfloat16())
    idx = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)
    return out[..., idx]
