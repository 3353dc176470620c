"""Model dimensions and parameter naming of pi0 (OpenPI ``PI0Pytorch`` state-dict names), plus a
random-initialised parameter set for benchmarks and smoke runs (no checkpoint or network needed).

The names are the module attributes the reference's model builder walks (``native_pi0/model.py:216-278``):
``paligemma_with_expert.paligemma.vision_tower.vision_model.*``, ``...multi_modal_projector.linear``,
``...language_model.{embed_tokens,layers.*}``, ``paligemma_with_expert.gemma_expert.model.{layers.*,norm}``,
``state_proj``, ``action_in_proj``, ``action_time_mlp_in``, ``action_time_mlp_out``, ``action_out_proj``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

VISION = "paligemma_with_expert.paligemma.vision_tower.vision_model."
PROJECTOR = "paligemma_with_expert.paligemma.multi_modal_projector.linear."
LANGUAGE = "paligemma_with_expert.paligemma.language_model."
EXPERT = "paligemma_with_expert.gemma_expert.model."


@dataclass
class Pi0Config:
    """pi0 = SigLIP-So400m/14 + Gemma-2B prefix + Gemma-300M action expert."""
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
    pi05: bool = False

    @classmethod
    def from_state_dict(cls, sd, **overrides):
        """Dimensions read off the tensors of a checkpoint (layer counts, widths, MLP sizes, head_dim from the single
        KV head, action_dim); head counts follow from the widths, everything else keeps its default."""
        def layers(prefix):
            return 1 + max(int(k[len(prefix):].split(".")[0]) for k in sd if k.startswith(prefix))

        vw = sd[VISION + "embeddings.patch_embedding.weight"].shape[0]
        head_dim = sd[LANGUAGE + "layers.0.self_attn.k_proj.weight"].shape[0]
        found = dict(
            vision_layers=layers(VISION + "encoder.layers."), vision_width=vw,
            vision_mlp=sd[VISION + "encoder.layers.0.mlp.fc1.weight"].shape[0],
            width=sd[LANGUAGE + "layers.0.self_attn.o_proj.weight"].shape[0],
            mlp=sd[LANGUAGE + "layers.0.mlp.gate_proj.weight"].shape[0],
            head_dim=head_dim, heads=sd[LANGUAGE + "layers.0.self_attn.q_proj.weight"].shape[0] // head_dim,
            prefix_layers=layers(LANGUAGE + "layers."),
            expert_width=sd[EXPERT + "layers.0.self_attn.o_proj.weight"].shape[0],
            expert_mlp=sd[EXPERT + "layers.0.mlp.gate_proj.weight"].shape[0],
            expert_layers=layers(EXPERT + "layers."),
            action_dim=sd["action_out_proj.weight"].shape[0])
        table = sd.get(LANGUAGE + "embed_tokens.weight")
        if table is not None:
            found["vocab"] = table.shape[0]
        found.update(overrides)
        return cls(**found)


def parameter_shapes(cfg: Pi0Config):
    """name -> (shape, kept_in_fp32, mean) for every parameter of the model."""
    out = {}

    def add(name, shape, fp32=False, mean=0.0):
        out[name] = (tuple(shape), fp32, mean)

    c = cfg
    add(VISION + "embeddings.patch_embedding.weight", (c.vision_width, 3, 14, 14), True)
    add(VISION + "embeddings.patch_embedding.bias", (c.vision_width,), True)
    add(VISION + "embeddings.position_embedding.weight", (256, c.vision_width), True)
    for i in range(c.vision_layers):
        p = f"{VISION}encoder.layers.{i}."
        for ln in ("layer_norm1", "layer_norm2"):
            add(p + ln + ".weight", (c.vision_width,), True, 1.0)
            add(p + ln + ".bias", (c.vision_width,), True)
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            add(p + f"self_attn.{proj}.weight", (c.vision_width, c.vision_width))
            add(p + f"self_attn.{proj}.bias", (c.vision_width,))
        add(p + "mlp.fc1.weight", (c.vision_mlp, c.vision_width))
        add(p + "mlp.fc1.bias", (c.vision_mlp,))
        add(p + "mlp.fc2.weight", (c.vision_width, c.vision_mlp))
        add(p + "mlp.fc2.bias", (c.vision_width,))
    add(VISION + "post_layernorm.weight", (c.vision_width,), True, 1.0)
    add(VISION + "post_layernorm.bias", (c.vision_width,), True)
    add(PROJECTOR + "weight", (c.width, c.vision_width))
    add(PROJECTOR + "bias", (c.width,))
    add(LANGUAGE + "embed_tokens.weight", (c.vocab, c.width))
    for prefix, layers, width, mlp in ((LANGUAGE, c.prefix_layers, c.width, c.mlp),
                                       (EXPERT, c.expert_layers, c.expert_width, c.expert_mlp)):
        for i in range(layers):
            p = f"{prefix}layers.{i}."
            add(p + "input_layernorm.weight", (width,), True)
            add(p + "post_attention_layernorm.weight", (width,), True)
            add(p + "self_attn.q_proj.weight", (c.heads * c.head_dim, width))
            add(p + "self_attn.k_proj.weight", (c.head_dim, width))
            add(p + "self_attn.v_proj.weight", (c.head_dim, width))
            add(p + "self_attn.o_proj.weight", (width, c.heads * c.head_dim))
            add(p + "mlp.gate_proj.weight", (mlp, width))
            add(p + "mlp.up_proj.weight", (mlp, width))
            add(p + "mlp.down_proj.weight", (width, mlp))
        add(prefix + "norm.weight", (width,), True)
    w = c.expert_width
    for name, shape in (("state_proj", (w, c.action_dim)), ("action_in_proj", (w, c.action_dim)),
                        ("action_time_mlp_in", (w, 2 * w)), ("action_time_mlp_out", (w, w)),
                        ("action_out_proj", (c.action_dim, w))):
        add(name + ".weight", shape, True)
        add(name + ".bias", (shape[0],), True)
    return out


def random_state_dict(cfg: Pi0Config, *, seed=0, device="cuda", std=0.02, skip_embedding=False):
    """Random-init parameters N(mean, std) generated on `device` (BF16; FP32 where the model keeps FP32)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    sd = {}
    for name, (shape, fp32, mean) in parameter_shapes(cfg).items():
        if skip_embedding and name.endswith("embed_tokens.weight"):
            continue
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean
        sd[name] = t if fp32 else t.to(torch.bfloat16)
    return sd


class StateDictModel:
    """Minimal stand-in for an OpenPI module: ``config`` + ``state_dict()``; accepted by ``NativePi0.from_model``."""

    def __init__(self, config: Pi0Config, state_dict):
        self.config = config
        self._sd = state_dict

    def state_dict(self):
        return self._sd
