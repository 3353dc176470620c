"""The steps either side of the timed forward: camera frames, robot state and a prompt in, an action chunk in robot
units out.

The reference measures ``forward`` on normalised, device-resident tensors and leaves "resizing, tokenization,
host/device transfers, and robot policy transforms" to the caller (``README.md:72-77``).  ``Pi0Policy`` is that caller
for this engine, shaped like an OpenPI policy's ``infer(observation) -> {"actions": ...}``:

* images: ``uint8 [H, W, 3]`` (or float in [0, 1]) per camera -> aspect-preserving resize to 224 x 224 with black
  padding, mapped to [-1, 1]; cameras missing from the observation are black frames
* state: ``(state - mean) / (std + 1e-6)``, zero-padded to the model's 32 action dimensions
* prompt: ``tokenizer(prompt) -> token ids`` (any callable; a SentencePiece model is a checkpoint asset and is not
  bundled), cut or right-padded with ``pad_token`` to the engine's fixed prompt length
* noise: drawn from a seeded generator unless supplied
* actions: un-normalised ``actions * (std + 1e-6) + mean`` and cut to the robot's action dimensions

Everything here is host / PyTorch plumbing; the forward itself is ``NativePi0.sample_actions``.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

IMAGE_SIZE = 224


def resize_with_pad(image, size=IMAGE_SIZE):
    """``[H, W, 3]`` uint8 or float -> FP32 ``[size, size, 3]`` in [-1, 1]: bilinear resize that keeps the aspect ratio,
    centred on a black canvas."""
    t = torch.as_tensor(np.asarray(image))
    if t.ndim != 3 or t.shape[-1] != 3:
        raise ValueError("images are [H, W, 3]")
    t = t.float() / 255.0 if t.dtype == torch.uint8 else t.float()
    h, w = t.shape[:2]
    ratio = max(h, w) / size
    nh, nw = max(1, min(size, round(h / ratio))), max(1, min(size, round(w / ratio)))
    resized = F.interpolate(t.permute(2, 0, 1)[None], size=(nh, nw), mode="bilinear", align_corners=False, antialias=True)[0]
    canvas = torch.zeros(3, size, size)
    top, left = (size - nh) // 2, (size - nw) // 2
    canvas[:, top:top + nh, left:left + nw] = resized.clamp(0, 1)
    return (canvas * 2.0 - 1.0).permute(1, 2, 0).contiguous()


class Normalizer:
    """``(x - mean) / (std + 1e-6)`` and back, on the leading ``len(mean)`` dimensions."""

    def __init__(self, mean, std):
        self.mean, self.std = np.asarray(mean, np.float32), np.asarray(std, np.float32)
        if self.mean.shape != self.std.shape or self.mean.ndim != 1 or np.any(self.std < 0):
            raise ValueError("mean and std are vectors of one length, std >= 0")

    def __len__(self):
        return len(self.mean)

    def forward(self, x):
        return (np.asarray(x, np.float32)[..., :len(self)] - self.mean) / (self.std + 1e-6)

    def inverse(self, y):
        return np.asarray(y, np.float32)[..., :len(self)] * (self.std + 1e-6) + self.mean


class Pi0Policy:
    def __init__(self, engine, *, cameras=("base_0_rgb", "left_wrist_0_rgb", "right_wrist_0_rgb"), state_norm: Normalizer = None,
                 action_norm: Normalizer = None, tokenizer=None, pad_token=0, seed=0):
        if len(cameras) != engine.num_views:
            raise ValueError(f"the engine was built for {engine.num_views} views, {len(cameras)} camera names given")
        if engine.prompt_len and tokenizer is None:
            raise ValueError("this engine takes a prompt: supply a tokenizer (prompt -> token ids)")
        self.engine, self.cameras = engine, tuple(cameras)
        self.state_norm, self.action_norm = state_norm, action_norm
        self.tokenizer, self.pad_token = tokenizer, int(pad_token)
        self.action_dim = engine.config.action_dim
        self.generator = torch.Generator(device="cpu").manual_seed(seed)
        self._pinned = None

    def _buffers(self):
        if self._pinned is None:
            e = self.engine
            make = lambda shape, dtype: torch.zeros(shape, dtype=dtype).pin_memory() if torch.cuda.is_available() else torch.zeros(shape, dtype=dtype)
            self._pinned = (make((e.num_views, IMAGE_SIZE, IMAGE_SIZE, 3), torch.float32), make((1, self.action_dim), torch.float32),
                            make((1, e.chunk_size, self.action_dim), torch.float32), make((1, e.prompt_len), torch.int64))
        return self._pinned

    def prepare(self, observation, noise=None):
        """Observation dict -> the four host tensors of ``sample_actions`` (pinned, reused between calls)."""
        images, state, noise_buf, tokens = self._buffers()
        frames = observation.get("images", observation)
        for i, name in enumerate(self.cameras):
            images[i] = resize_with_pad(frames[name]) if name in frames else -1.0
        s = np.asarray(observation["state"], np.float32).reshape(-1)
        if self.state_norm is not None:
            s = self.state_norm.forward(s)
        if len(s) > self.action_dim:
            raise ValueError(f"state has {len(s)} dimensions, the model takes {self.action_dim}")
        state.zero_()
        state[0, :len(s)] = torch.from_numpy(np.ascontiguousarray(s))
        if self.engine.prompt_len:
            ids = list(self.tokenizer(observation.get("prompt", "")))[:self.engine.prompt_len]
            ids += [self.pad_token] * (self.engine.prompt_len - len(ids))
            tokens[0] = torch.tensor(ids, dtype=torch.int64)
        if noise is None:
            noise_buf.normal_(generator=self.generator)
        else:
            noise_buf.copy_(torch.as_tensor(np.asarray(noise, np.float32)).reshape(noise_buf.shape))
        return images, state, noise_buf, tokens

    def infer(self, observation, noise=None):
        """One action chunk in robot units: ``{"actions": float32 [chunk, robot action dims]}``."""
        actions = self.engine.sample_actions(*self.prepare(observation, noise))[0].numpy()
        if self.action_norm is not None:
            actions = self.action_norm.inverse(actions)
        return {"actions": np.array(actions, dtype=np.float32, copy=True)}
