"""PyTorch restatement of the pi0 forward pass (TEST INFRASTRUCTURE; runs on CPU or GPU).

Two modes over the same state dict (OpenPI ``PI0Pytorch`` parameter names):

* ``mode="bf16"``  - the BF16 eager model the reference compares against
  (``benchmarks/openpi_backend.py:29-81`` ``fixed_sample``: prefix forward with ``use_cache=True``,
  then ``steps`` Euler updates ``x += dt * v`` with ``dt = -1/steps`` from ``t = 1``).
  OpenPI itself (Physical-Intelligence/openpi@215abfb2) is a network dependency of the reference and is
  not available offline, so this is a restatement of its architecture as the reference's own model
  builder walks it (``native_pi0/model.py:154-278``): SigLIP-So400m/14 blocks, PaliGemma projector,
  Gemma-2B prefix, Gemma-300M action expert, state / action / time heads.  **Parity of this mode
  with upstream OpenPI is unpinned** (no golden tensors exist for it).
* ``mode="nvfp4"`` - the same graph with the engine's numerics: every transformer linear consumes an
  NVFP4 fake-quantised activation (``nearest`` block scales, tensor scale 1) and an NVFP4
  fake-quantised weight (``ceil`` block scales, tensor scale amax/(6*448)), accumulates in FP32, and
  applies the epilogue roundings the kernels apply.  This is the "dequantised-NVFP4 math" oracle
  (the reference's per-op form is ``deq(A) @ deq(B).T``, ``scripts/validate_nvfp4.py:49``).

Conventions taken from the reference code: GELU tanh form (``native_pi0/dense.cu:53``); Gemma RMSNorm
gamma = 1 + w (``model.py:129``); attention scale head_dim**-0.5; rotate-half RoPE over the whole head,
base 10000 (``model.py:147-152``); suffix mask: state query sees prefix + itself, action queries see
everything (``attention.cu:342``); time embedding 512 log-spaced periods 0.004..4.0, [sin | cos]
(``model.py:259-263``); token embeddings * sqrt(width) (``model.py:238-239``); patch embedding, norm
parameters and the state / action / time heads in FP32 (``README.md:93-94``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F


@dataclass
class Pi0Dims:
    views: int = 3
    vision_layers: int = 27
    vision_width: int = 1152
    vision_mlp: int = 4304
    vision_heads: int = 16
    width: int = 2048
    mlp: int = 16384
    heads: int = 8
    head_dim: int = 256
    prefix_layers: int = 18
    vocab: int = 257152
    expert_width: int = 1024
    expert_mlp: int = 4096
    expert_layers: int = 18
    action_dim: int = 32
    ln_eps: float = 1e-6
    rms_eps: float = 1e-6
    rope_base: float = 10000.0


VP = "paligemma_with_expert.paligemma.vision_tower.vision_model."
PJ = "paligemma_with_expert.paligemma.multi_modal_projector.linear."
LM = "paligemma_with_expert.paligemma.language_model."
EX = "paligemma_with_expert.gemma_expert.model."


def init_state_dict(dims: Pi0Dims, seed=0, device="cpu", dtype=torch.bfloat16):
    """Random-init parameters: weights, biases and embeddings N(0, 0.02); LayerNorm weight 1 + N(0, 0.02);
    Gemma RMSNorm weight N(0, 0.02) (gamma = 1 + w).  FP32 for patch embedding, norms and the heads."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    sd = {}

    def put(name, shape, base=0.0, fp32=False):
        t = torch.randn(shape, generator=g, dtype=torch.float32) * 0.02 + base
        sd[name] = t.to(device=device, dtype=torch.float32 if fp32 else dtype)

    d = dims
    put(VP + "embeddings.patch_embedding.weight", (d.vision_width, 3, 14, 14), fp32=True)
    put(VP + "embeddings.patch_embedding.bias", (d.vision_width,), fp32=True)
    put(VP + "embeddings.position_embedding.weight", (256, d.vision_width), fp32=True)
    for i in range(d.vision_layers):
        p = f"{VP}encoder.layers.{i}."
        for ln in ("layer_norm1", "layer_norm2"):
            put(p + ln + ".weight", (d.vision_width,), 1.0, fp32=True)
            put(p + ln + ".bias", (d.vision_width,), fp32=True)
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            put(p + f"self_attn.{proj}.weight", (d.vision_width, d.vision_width))
            put(p + f"self_attn.{proj}.bias", (d.vision_width,))
        put(p + "mlp.fc1.weight", (d.vision_mlp, d.vision_width))
        put(p + "mlp.fc1.bias", (d.vision_mlp,))
        put(p + "mlp.fc2.weight", (d.vision_width, d.vision_mlp))
        put(p + "mlp.fc2.bias", (d.vision_width,))
    put(VP + "post_layernorm.weight", (d.vision_width,), 1.0, fp32=True)
    put(VP + "post_layernorm.bias", (d.vision_width,), fp32=True)
    put(PJ + "weight", (d.width, d.vision_width))
    put(PJ + "bias", (d.width,))
    put(LM + "embed_tokens.weight", (d.vocab, d.width))
    for prefix, layers, width, mlp in ((LM, d.prefix_layers, d.width, d.mlp), (EX, d.expert_layers, d.expert_width, d.expert_mlp)):
        for i in range(layers):
            p = f"{prefix}layers.{i}."
            put(p + "input_layernorm.weight", (width,), fp32=True)
            put(p + "post_attention_layernorm.weight", (width,), fp32=True)
            put(p + "self_attn.q_proj.weight", (d.heads * d.head_dim, width))
            put(p + "self_attn.k_proj.weight", (d.head_dim, width))
            put(p + "self_attn.v_proj.weight", (d.head_dim, width))
            put(p + "self_attn.o_proj.weight", (width, d.heads * d.head_dim))
            put(p + "mlp.gate_proj.weight", (mlp, width))
            put(p + "mlp.up_proj.weight", (mlp, width))
            put(p + "mlp.down_proj.weight", (width, mlp))
        put(prefix + "norm.weight", (width,), fp32=True)
    w = d.expert_width
    put("state_proj.weight", (w, d.action_dim), fp32=True)
    put("state_proj.bias", (w,), fp32=True)
    put("action_in_proj.weight", (w, d.action_dim), fp32=True)
    put("action_in_proj.bias", (w,), fp32=True)
    put("action_time_mlp_in.weight", (w, 2 * w), fp32=True)
    put("action_time_mlp_in.bias", (w,), fp32=True)
    put("action_time_mlp_out.weight", (w, w), fp32=True)
    put("action_time_mlp_out.bias", (w,), fp32=True)
    put("action_out_proj.weight", (d.action_dim, w), fp32=True)
    put("action_out_proj.bias", (d.action_dim,), fp32=True)
    return sd


# ---------------------------------------------------------------------------------------------------
# NVFP4 fake quantisation in torch, byte-for-byte the arithmetic of native_pi0/quantization.py:48-93.
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _ue4m3_table(device):
    codes = torch.arange(127, device=device)
    mant = (codes & 7).double()
    expo = (codes >> 3).double()
    return torch.where(expo == 0, mant * 2.0 ** -9, (1 + mant / 8) * torch.pow(torch.tensor(2.0, dtype=torch.float64, device=device), expo - 7)).float()


def _nearest_even(values, table):
    hi = torch.searchsorted(table, values.contiguous()).clamp(0, table.numel() - 1)
    lo = (hi - 1).clamp(min=0)
    dl, dh = values - table[lo], table[hi] - values
    return torch.where((dl < dh) | ((dl == dh) & ((lo & 1) == 0)), lo, hi)


def quantize_codes(x, policy="nearest", global_scale=1.0):
    """FP32 [..., K] (K % 16 == 0) -> (E2M1 codes incl. sign bit, uint8 [..., K]; scale codes uint8 [..., K/16])."""
    x = x.float()
    table = _ue4m3_table(x.device)
    e2m1 = torch.tensor(_E2M1, device=x.device)
    gs = torch.tensor(global_scale, dtype=torch.float32, device=x.device)
    xs = x * (torch.tensor(1.0, device=x.device) / gs)
    blocks = xs.reshape(*x.shape[:-1], x.shape[-1] // 16, 16)
    desired = blocks.abs().amax(-1) * torch.tensor(1 / 6, dtype=torch.float32, device=x.device)
    if policy == "ceil":
        codes = torch.searchsorted(table, desired.contiguous()).clamp(0, 126)
    else:
        codes = _nearest_even(desired, table)
    scale = table[codes]
    recip = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
    normalized = blocks * recip.unsqueeze(-1)
    normalized = torch.where(scale.unsqueeze(-1) > 0, normalized, torch.zeros_like(normalized))
    q = _nearest_even(normalized.abs(), e2m1)
    q = q | (torch.signbit(normalized).long() << 3)
    return q.reshape(x.shape).to(torch.uint8), codes.to(torch.uint8)


def fake_quant(x, policy="nearest", global_scale=1.0):
    """Quantise to NVFP4 and decode again (FP32 result, same shape)."""
    q, codes = quantize_codes(x, policy, global_scale)
    table = _ue4m3_table(x.device)
    e2m1 = torch.tensor(_E2M1, device=x.device)
    mag = e2m1[(q & 7).long()]
    val = torch.where((q & 8) != 0, -mag, mag)
    val = val.reshape(*x.shape[:-1], x.shape[-1] // 16, 16) * table[codes.long()].unsqueeze(-1)
    return (val * torch.tensor(global_scale, dtype=torch.float32, device=x.device)).reshape(x.shape)


def weight_global_scale(w):
    """Tensor scale used for weights: the largest block scale lands on the top E4M3 code."""
    return max(float(w.float().abs().max()) / (6.0 * 448.0), 1e-30)


def pad_cols(x, multiple):
    k = x.shape[-1]
    pk = -(-k // multiple) * multiple
    return x if pk == k else F.pad(x, (0, pk - k))


# ---------------------------------------------------------------------------------------------------
def rope_tables(positions, head_dim, base, dtype=torch.bfloat16, inv_freq_dtype=torch.float32):
    """cos/sin [rows, head_dim] as the Gemma rotary module produces them: angles in FP32, emb = cat(f, f),
    tables cast to the activation dtype.  ``inv_freq_dtype=torch.bfloat16`` reproduces a model whose
    inverse-frequency buffer was cast to BF16 (``native_pi0/model.py:147-152``)."""
    device = positions.device
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    inv = inv.to(inv_freq_dtype).float()
    freqs = positions.float()[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x, cos, sin):
    """x [rows, heads, hd]; BF16 arithmetic as eager PyTorch does it: each product and the sum round to BF16."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos[:, None, :]) + (rot * sin[:, None, :])


def time_embedding(t, width, device):
    """``model.py:259-263``: 512 (width/2) periods log-spaced 0.004..4.0, [sin | cos], FP64 then FP32."""
    fraction = torch.linspace(0.0, 1.0, width // 2, dtype=torch.float64, device=device)
    period = 0.004 * (4.0 / 0.004) ** fraction
    angle = float(t) / period * (2.0 * math.pi)
    return torch.cat((angle.sin(), angle.cos())).float()


_SITE_OF_LEAF = {"q_proj": "qkv", "k_proj": "qkv", "v_proj": "qkv", "out_proj": "out", "o_proj": "o_proj", "fc1": "fc1", "fc2": "fc2",
                 "gate_proj": "gate_up", "up_proj": "gate_up", "down_proj": "down"}


def site_of(parameter):
    """Engine site name of a linear's parameter prefix: ``vision.<i>.{qkv,out,fc1,fc2}``, ``vision.projector``,
    ``prefix.<i>.{qkv,o_proj,gate_up,down}``, ``expert.<i>.{...}``."""
    if parameter.startswith(PJ[:-1]):
        return "vision.projector"
    tower = "vision" if parameter.startswith(VP) else "prefix" if parameter.startswith(LM) else "expert"
    layer = parameter.split("layers.")[1].split(".")[0]
    return f"{tower}.{layer}.{_SITE_OF_LEAF[parameter.rsplit('.', 1)[1]]}"


class Pi0Torch:
    def __init__(self, dims: Pi0Dims, state_dict, mode="bf16", compute_dtype=torch.bfloat16, rope_inv_freq_dtype=torch.float32,
                 precision=None, fold_norms=True, head_blocks=True, fold_layernorms=True):
        """``precision`` (mode "nvfp4" only): dict of fnmatch patterns over site names -> "nvfp4" | "bf16" with an optional
        "default", as the engine takes it; BF16 sites multiply BF16 operands with FP32 accumulation and round the way the
        engine's BF16 epilogues do.  ``fold_norms`` (mode "nvfp4"): an RMSNorm between two NVFP4 projections is evaluated
        the way the engine folds it - the un-normalised BF16 rows are quantised, the weight columns carry ``1 + w`` and
        the accumulator rows are multiplied by ``rsqrt(mean square + eps)``.  ``head_blocks`` (mode "nvfp4"): the SigLIP
        attention rows and the output projection's weight are quantised with every 72-wide head on a pitch of 80 columns,
        i.e. in blocks that do not straddle heads, as the engine's tensor-core attention tiles write them; False keeps
        the plain 16-column partition of the 1152-wide rows (the engine with ``attention_path="mma.sync"``).
        ``fold_layernorms`` (with ``fold_norms``): SigLIP's LayerNorms between two NVFP4 projections are folded the same
        way - un-normalised rows quantised, gamma in the weight columns, ``bias + W beta`` as bias, and the accumulator
        rows turned into ``rstd * (acc - mean * sum_k W'[n, k])`` with the variance as ``E[x^2] - mean^2``."""
        assert mode in ("bf16", "nvfp4")
        self.d, self.sd, self.mode = dims, state_dict, mode
        precision = precision or {}
        if isinstance(precision, str):
            precision = {"default": precision}
        self._precision_map = [(k, v) for k, v in precision.items() if k != "default"]
        self._precision_default = precision.get("default", "nvfp4")
        self._site_cache = {}
        self.fold_norms = bool(fold_norms) and mode == "nvfp4"
        self.head_blocks = bool(head_blocks) and mode == "nvfp4"
        self.fold_layernorms = bool(fold_layernorms) and self.fold_norms
        self.dt = compute_dtype                 # activation dtype of the bf16 mode (float32 for a fast CPU baseline)
        self.rope_inv_freq_dtype = rope_inv_freq_dtype
        self._wq = {}
        self._kv_only = {(f"{LM}layers.{dims.prefix_layers - 1}.self_attn", "kv_only")}
        self.landmarks = {}
        self.record_ops = False                 # also keep every operator's output (``ops``), named like the engine's stages
        self.ops = {}

    def rec(self, name, tensor):
        if self.record_ops:
            self.ops[name] = tensor

    # ----- linear layers ---------------------------------------------------------------------------
    def bf16_site(self, parameter):
        """True when the linear at ``parameter`` runs on BF16 operands in the engine configuration being emulated."""
        if self.mode != "nvfp4":
            return False
        if parameter not in self._site_cache:
            import fnmatch
            site = site_of(parameter)
            chosen = next((v for k, v in self._precision_map if fnmatch.fnmatchcase(site, k)), self._precision_default)
            self._site_cache[parameter] = chosen == "bf16"
        return self._site_cache[parameter]

    def add_residual(self, o, x, parameter):
        """Residual add of a projection ``o`` (FP32 accumulator incl. bias).  NVFP4 sites round once after the sum; BF16
        sites round the projection first (OpenPI's eager ``x + o`` on BF16 tensors), then the sum."""
        if self.mode != "nvfp4":
            return x + o
        if self.bf16_site(parameter):
            return (o.to(torch.bfloat16).float() + x.float()).to(torch.bfloat16)
        return (o + x.float()).to(torch.bfloat16)

    @staticmethod
    def _folded(w, gamma):
        """Weight with the norm weight folded into its columns, stored in BF16 like every weight the engine packs."""
        return w if gamma is None else (w.float() * gamma.float()[None, :]).to(torch.bfloat16)

    def _fused_scale(self, name, w, gamma=None):
        """The engine packs q|k|v (k|v for the last prefix layer) and gate|up as ONE NVFP4 tensor, so the members of
        a fused projection share one tensor scale: amax over the fused matrix / (6*448)."""
        base, leaf = name.rsplit(".", 1)
        if leaf in ("q_proj", "k_proj", "v_proj"):
            members = ["k_proj", "v_proj"] if (base, "kv_only") in self._kv_only else ["q_proj", "k_proj", "v_proj"]
        elif leaf in ("gate_proj", "up_proj"):
            members = ["gate_proj", "up_proj"]
        else:
            return weight_global_scale(self._folded(w, gamma))
        return max(weight_global_scale(self._folded(self.sd[f"{base}.{m}.weight"], gamma)) for m in members)

    def _qweight(self, name, w, gamma=None):
        key = (name, gamma is not None)
        if key not in self._wq:
            gs = self._fused_scale(name, w, gamma)
            self._wq[key] = fake_quant(pad_cols(self._folded(w, gamma).float(), 64), "ceil", gs)
        return self._wq[key]

    def folded_linear(self, x, name, gamma):
        """NVFP4 projection of UN-normalised BF16 rows ``x`` through a weight that carries ``gamma`` (= 1 + norm weight)
        in its columns, times the rows' ``rsqrt(mean square + eps)``: the engine's folded RMSNorm.  FP32, not rounded."""
        xf = x.to(torch.bfloat16).float()
        wq = self._qweight(name, self.sd[name + ".weight"], gamma)
        y = fake_quant(pad_cols(xf, 64), "nearest", 1.0) @ wq.T
        return y * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.d.rms_eps)

    def folded_layernorm_linear(self, x, name, gamma, beta, eps):
        """NVFP4 projection (with its bias) of LayerNorm(x) evaluated the way the engine folds it: the UN-normalised BF16
        rows ``x`` are quantised, the weight columns carry ``gamma``, the bias becomes ``b + W beta`` (BF16), and the
        accumulator rows are centred and scaled afterwards.  FP32, not rounded."""
        xf = x.to(torch.bfloat16).float()
        w, b = self.sd[name + ".weight"], self.sd[name + ".bias"]
        wq = self._qweight(name, w, gamma)
        acc = fake_quant(pad_cols(xf, 64), "nearest", 1.0) @ wq.T
        mean = xf.mean(-1, keepdim=True)
        rstd = torch.rsqrt((xf.square().mean(-1, keepdim=True) - mean * mean).clamp_min(0.0) + eps)
        bias = (b.float() + w.to(torch.bfloat16).float() @ beta.float()).to(torch.bfloat16).float()
        return rstd * (acc - mean * wq.sum(-1)[None, :]) + bias

    def folds(self, producer, consumer):
        """True when the norm between the projections ``producer`` and ``consumer`` (parameter prefixes) is folded."""
        return self.fold_norms and not self.bf16_site(producer) and not self.bf16_site(consumer)

    def linear(self, x, name, bias=True, weight=None, head=None):
        """BF16 mode: y = x W^T + b in the activation dtype.  NVFP4 mode: FP32 accumulator of fake-quantised
        operands (+ bias), *not yet rounded* - the caller applies the epilogue.  ``head=(width, pitch)``: the K axis
        is made of heads ``width`` wide that are quantised on a pitch of ``pitch`` columns (zeros between them)."""
        w = self.sd[name + ".weight"] if weight is None else weight
        b = self.sd.get(name + ".bias") if bias else None
        if self.mode == "bf16":
            return F.linear(x.to(self.dt), w.to(self.dt), None if b is None else b.to(self.dt))
        if self.bf16_site(name):
            y = x.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().T
            return y if b is None else y + b.to(torch.bfloat16).float()
        if head is not None:
            width, pitch = head
            spread = lambda t: F.pad(t.float().reshape(t.shape[0], -1, width), (0, pitch - width)).reshape(t.shape[0], -1)
            x = spread(x)
            if (name, "spread") not in self._wq:
                self._wq[(name, "spread")] = fake_quant(pad_cols(spread(w), 64), "ceil", weight_global_scale(w))
            wq = self._wq[(name, "spread")]
        else:
            wq = self._qweight(name, w)
        xq = fake_quant(pad_cols(x.float(), 64), "nearest", 1.0)
        y = xq @ wq.T
        return y if b is None else y + b.float()

    def act(self, y):
        """Round an FP32 epilogue value to the BF16 activation (identity in bf16 mode)."""
        return y.to(torch.bfloat16) if self.mode == "nvfp4" else y

    # ----- attention -------------------------------------------------------------------------------
    def attention(self, q, k, v, scale, mask=None):
        """q [Nq,H,d], k/v [Nk,Hk,d] -> [Nq,H,d].  BF16 mode mirrors eager: BF16 scores, FP32 softmax, BF16 PV."""
        groups = q.shape[1] // k.shape[1]
        k = k.repeat_interleave(groups, 1)
        v = v.repeat_interleave(groups, 1)
        if self.mode == "nvfp4":
            s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * scale
            if mask is not None:
                s = s.masked_fill(~mask[None], float("-inf"))
            p = torch.softmax(s, dim=-1)
            return torch.einsum("hqk,khd->qhd", p, v.float()).to(torch.bfloat16)
        s = torch.einsum("qhd,khd->hqk", q, k) * scale
        if mask is not None:
            s = s.masked_fill(~mask[None], torch.finfo(s.dtype).min)
        p = torch.softmax(s.float(), dim=-1).to(q.dtype)
        return torch.einsum("hqk,khd->qhd", p, v)

    # ----- SigLIP ----------------------------------------------------------------------------------
    def vision(self, images):
        """images FP32 [views,224,224,3] NHWC in [-1,1] -> tokens [views*256, vision_width]."""
        d, sd = self.d, self.sd
        x = images.permute(0, 3, 1, 2).float()
        x = F.conv2d(x, sd[VP + "embeddings.patch_embedding.weight"].float(), sd[VP + "embeddings.patch_embedding.bias"].float(), stride=14)
        x = x.flatten(2).transpose(1, 2) + sd[VP + "embeddings.position_embedding.weight"].float()[None]
        x = x.reshape(-1, d.vision_width).to(self.dt if self.mode == "bf16" else torch.bfloat16)
        self.landmarks["patch"] = x
        hd = d.vision_width // d.vision_heads
        views = images.shape[0]
        for i in range(d.vision_layers):
            p = f"{VP}encoder.layers.{i}."
            g1, b1 = sd[p + "layer_norm1.weight"].float(), sd[p + "layer_norm1.bias"].float()
            # the first layer's norm reads the patch embedding and stays a norm; later ones fold between fc2 and q|k|v
            if i > 0 and self.fold_layernorms and self.folds(f"{VP}encoder.layers.{i - 1}.mlp.fc2", p + "self_attn.q_proj"):
                q, k, v = [self.act(self.folded_layernorm_linear(x, p + f"self_attn.{n}_proj", g1, b1, d.ln_eps)) for n in "qkv"]
            else:
                y = F.layer_norm(x.float(), (d.vision_width,), g1, b1, d.ln_eps).to(x.dtype)
                self.rec(f"vision.{i}.ln1", y)
                q = self.act(self.linear(y, p + "self_attn.q_proj"))
                k = self.act(self.linear(y, p + "self_attn.k_proj"))
                v = self.act(self.linear(y, p + "self_attn.v_proj"))
            self.rec(f"vision.{i}.qkv", torch.cat((q, k, v), dim=-1))
            outs = []
            for b in range(views):
                sl = slice(b * 256, (b + 1) * 256)
                outs.append(self.attention(q[sl].reshape(256, d.vision_heads, hd), k[sl].reshape(256, d.vision_heads, hd),
                                           v[sl].reshape(256, d.vision_heads, hd), hd ** -0.5))
            a = torch.cat(outs).reshape(-1, d.vision_width)
            self.rec(f"vision.{i}.attention", a)
            o = self.linear(a, p + "self_attn.out_proj", head=(hd, -(-hd // 16) * 16) if self.head_blocks and hd % 16 else None)
            x = self.add_residual(o, x, p + "self_attn.out_proj")
            self.rec(f"vision.{i}.out", x)
            g2, b2 = sd[p + "layer_norm2.weight"].float(), sd[p + "layer_norm2.bias"].float()
            if self.fold_layernorms and self.folds(p + "self_attn.out_proj", p + "mlp.fc1"):
                h = self.folded_layernorm_linear(x, p + "mlp.fc1", g2, b2, d.ln_eps)
            else:
                y = F.layer_norm(x.float(), (d.vision_width,), g2, b2, d.ln_eps).to(x.dtype)
                self.rec(f"vision.{i}.ln2", y)
                h = self.linear(y, p + "mlp.fc1")
            if self.mode != "nvfp4":
                h = F.gelu(h, approximate="tanh")
            elif self.bf16_site(p + "mlp.fc2"):
                h = F.gelu(h.to(torch.bfloat16).float(), approximate="tanh").to(torch.bfloat16)     # BF16 hidden rows for a BF16 consumer
            else:
                h = F.gelu(h.float(), approximate="tanh")
            self.rec(f"vision.{i}.fc1", h)
            o = self.linear(h, p + "mlp.fc2")
            x = self.add_residual(o, x, p + "mlp.fc2")
            self.rec(f"vision.{i}.fc2", x)
            self.landmarks[f"vision.{i}"] = x
        y = F.layer_norm(x.float(), (d.vision_width,), sd[VP + "post_layernorm.weight"].float(), sd[VP + "post_layernorm.bias"].float(), d.ln_eps).to(x.dtype)
        self.rec("vision.post_layernorm", y)
        out = self.act(self.linear(y, PJ[:-1]))
        self.rec("vision.projector", out)
        return out

    # ----- Gemma -----------------------------------------------------------------------------------
    def rms(self, x, w):
        xf = x.float()
        y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.d.rms_eps) * (1.0 + w.float())
        return y.to(x.dtype)

    def gemma_layer(self, x, prefix, i, cos, sin, cache, mask, kv_only=False, name=None):
        """One decoder layer on rows x [N, width].  ``cache`` = (K, V) of earlier rows or None.  Returns (x, (K, V)).
        ``name`` (the engine's stage prefix, e.g. ``prefix.3`` or ``expert.0.3``) labels the operator outputs kept by ``rec``."""
        d, sd = self.d, self.sd
        p = f"{prefix}layers.{i}."
        # the input norm is folded when the previous layer's down projection and this QKV projection are NVFP4 sites
        fold1 = i > 0 and self.folds(f"{prefix}layers.{i - 1}.mlp.down_proj", p + "self_attn.q_proj")
        if fold1:
            g1 = 1.0 + sd[p + "input_layernorm.weight"].float()
            project = lambda leaf: self.folded_linear(x, p + "self_attn." + leaf, g1)
        else:
            y = self.rms(x, sd[p + "input_layernorm.weight"])
            self.rec(f"{name}.norm1", y)
            project = lambda leaf: self.linear(y, p + "self_attn." + leaf, bias=False)
        k = self.act(project("k_proj")).reshape(-1, 1, d.head_dim)
        v = self.act(project("v_proj")).reshape(-1, 1, d.head_dim)
        k = apply_rope(k, cos, sin)
        self.rec(f"{name}.qkv.k", k)
        self.rec(f"{name}.qkv.v", v)
        if cache is not None:
            k_all, v_all = torch.cat((cache[0], k)), torch.cat((cache[1], v))
        else:
            k_all, v_all = k, v
        if kv_only:
            return x, (k, v)
        q = self.act(project("q_proj")).reshape(-1, d.heads, d.head_dim)
        q = apply_rope(q, cos, sin)
        self.rec(f"{name}.qkv.q", q)
        a = self.attention(q, k_all, v_all, d.head_dim ** -0.5, mask).reshape(x.shape[0], -1)
        self.rec(f"{name}.attention", a)
        o = self.linear(a, p + "self_attn.o_proj", bias=False)
        x = self.add_residual(o, x, p + "self_attn.o_proj")
        self.rec(f"{name}.o_proj", x)
        if self.folds(p + "self_attn.o_proj", p + "mlp.gate_proj"):
            g2 = 1.0 + sd[p + "post_attention_layernorm.weight"].float()
            gate = self.folded_linear(x, p + "mlp.gate_proj", g2)
            up = self.folded_linear(x, p + "mlp.up_proj", g2)
        else:
            y = self.rms(x, sd[p + "post_attention_layernorm.weight"])
            self.rec(f"{name}.norm2", y)
            gate = self.linear(y, p + "mlp.gate_proj", bias=False)
            up = self.linear(y, p + "mlp.up_proj", bias=False)
        if self.mode != "nvfp4":
            h = F.gelu(gate, approximate="tanh") * up
        elif self.bf16_site(p + "mlp.down_proj"):
            bf = torch.bfloat16
            h = (F.gelu(gate.to(bf).float(), approximate="tanh").to(bf).float() * up.to(bf).float()).to(bf)
        else:
            h = F.gelu(gate.float(), approximate="tanh") * up.float()
        self.rec(f"{name}.gate_up", h)
        o = self.linear(h, p + "mlp.down_proj", bias=False)
        x = self.add_residual(o, x, p + "mlp.down_proj")
        self.rec(f"{name}.down", x)
        return x, (k, v)

    def prefix(self, images, tokens):
        d, sd = self.d, self.sd
        x = self.vision(images)
        self.landmarks["image_tokens"] = x
        if tokens is not None and tokens.numel():
            emb = sd[LM + "embed_tokens.weight"][tokens.reshape(-1)]
            emb = (emb.to(x.dtype) * math.sqrt(d.width)).to(x.dtype)
            x = torch.cat((x, emb))
        rows = x.shape[0]
        self.landmarks["prefix.input"] = x
        cos, sin = rope_tables(torch.arange(rows, device=x.device), d.head_dim, d.rope_base, torch.bfloat16 if self.mode == "nvfp4" else x.dtype, self.rope_inv_freq_dtype)
        caches = []
        for i in range(d.prefix_layers):
            x, kv = self.gemma_layer(x, LM, i, cos, sin, None, None, kv_only=(i == d.prefix_layers - 1), name=f"prefix.{i}")
            caches.append(kv)
            self.landmarks[f"prefix.{i}"] = x
        return caches

    def denoise_step(self, caches, state_emb, actions, t, prefix_rows, tag=None):
        """One velocity evaluation.  ``tag`` (the Euler step index) makes the expert's rows observable: the assembled
        input as ``expert.<tag>.input`` and every layer's output as ``expert.<tag>.<layer>``."""
        d, sd = self.d, self.sd
        w = d.expert_width
        chunk = actions.shape[0]
        a_emb = F.linear(actions.float(), sd["action_in_proj.weight"].float(), sd["action_in_proj.bias"].float())
        t_emb = time_embedding(t, w, actions.device)[None].expand(chunk, -1)
        h = F.linear(torch.cat((a_emb, t_emb), dim=-1), sd["action_time_mlp_in.weight"].float(), sd["action_time_mlp_in.bias"].float())
        h = F.silu(h)
        self.rec(f"expert.{tag}.time_in", h)
        h = F.linear(h, sd["action_time_mlp_out.weight"].float(), sd["action_time_mlp_out.bias"].float())
        adt = torch.bfloat16 if self.mode == "nvfp4" else self.dt
        x = torch.cat((state_emb, h)).to(adt)
        rows = chunk + 1
        cos, sin = rope_tables(torch.arange(prefix_rows, prefix_rows + rows, device=x.device), d.head_dim, d.rope_base, adt, self.rope_inv_freq_dtype)
        mask = torch.ones(rows, prefix_rows + rows, dtype=torch.bool, device=x.device)
        mask[0, prefix_rows + 1:] = False
        if tag is not None:
            self.landmarks[f"expert.{tag}.input"] = x
        for i in range(d.expert_layers):
            x, _ = self.gemma_layer(x, EX, i, cos, sin, caches[i], mask, name=f"expert.{tag}.{i}")
            if tag is not None:
                self.landmarks[f"expert.{tag}.{i}"] = x
        xf = x[1:].float()
        if self.mode == "nvfp4":
            # engine: FP32 projection of the BF16 rows with (1+w) folded, times the row's 1/rms
            y = (xf * (1.0 + sd[EX + "norm.weight"].float())) * torch.rsqrt(xf.square().mean(-1, keepdim=True) + d.rms_eps)
        else:
            y = self.rms(x[1:], sd[EX + "norm.weight"]).float()
        return F.linear(y, sd["action_out_proj.weight"].float(), sd["action_out_proj.bias"].float())

    @torch.no_grad()
    def sample_actions(self, images, state, noise, tokens=None, steps=10):
        """images [views,224,224,3], state [1,32], noise [1,chunk,32], tokens [1,T] -> actions FP32 [1,chunk,32]."""
        self.landmarks = {}
        caches = self.prefix(images, tokens)
        self.caches = caches
        prefix_rows = caches[0][0].shape[0]
        state_emb = F.linear(state.float(), self.sd["state_proj.weight"].float(), self.sd["state_proj.bias"].float())
        x = noise[0].float().clone()
        # FP32 time and step, kept on the host (no host-to-device copy inside the loop: the pass can be captured in a CUDA graph)
        t, dt = np.float32(1.0), np.float32(-1.0 / steps)
        for step in range(steps):
            v = self.denoise_step(caches, state_emb, x, float(t), prefix_rows, tag=step)
            x = x + float(dt) * v
            self.landmarks[f"actions.{step}"] = x.clone()
            t = np.float32(t + dt)
        return x[None]
