"""Caller-side plumbing on CPU: observation -> engine inputs -> robot-unit actions, and the replica pool."""
import numpy as np
import pytest
import torch

from native_pi0.policy import Normalizer, Pi0Policy, resize_with_pad
from native_pi0.replicas import ReplicaPool, requests_for, requests_for_ticket


class FakeConfig:
    action_dim = 32


class FakeEngine:
    """Stands in for NativePi0 on a machine without a GPU: records its inputs, returns state-dependent 'actions'."""
    config = FakeConfig()

    def __init__(self, views=3, prompt=4, chunk=5, offset=0.0):
        self.num_views, self.prompt_len, self.chunk_size, self.offset = views, prompt, chunk, offset
        self.seen = None

    def sample_actions(self, images, state, noise, tokens):
        self.seen = tuple(t.clone() for t in (images, state, noise, tokens))
        return (state[:, None, :] + noise * 0 + self.offset).expand(1, self.chunk_size, 32).clone()


def test_resize_with_pad_keeps_aspect_and_range():
    frame = np.full((100, 200, 3), 255, np.uint8)
    out = resize_with_pad(frame)
    assert out.shape == (224, 224, 3) and out.dtype == torch.float32
    assert float(out.max()) <= 1.0 and float(out.min()) >= -1.0
    assert torch.all(out[:50] == -1.0) and torch.all(out[-50:] == -1.0)          # black bars above and below the 112-row image
    assert torch.allclose(out[112, 10:-10], torch.ones(204, 3), atol=1e-5)
    same = resize_with_pad(np.zeros((224, 224, 3), np.float32) + 0.5)
    assert torch.allclose(same, torch.zeros_like(same), atol=1e-6)
    with pytest.raises(ValueError):
        resize_with_pad(np.zeros((8, 8), np.uint8))


def test_policy_prepares_inputs_and_unnormalises_actions():
    engine = FakeEngine()
    state_norm = Normalizer(mean=[1.0, 2.0, 3.0], std=[2.0, 2.0, 2.0])
    action_norm = Normalizer(mean=[10.0, 20.0], std=[1.0, 3.0])
    policy = Pi0Policy(engine, state_norm=state_norm, action_norm=action_norm, tokenizer=lambda text: [ord(c) for c in text], pad_token=7)
    obs = {"images": {"base_0_rgb": np.zeros((50, 50, 3), np.uint8), "left_wrist_0_rgb": np.full((224, 224, 3), 255, np.uint8)},
           "state": [3.0, 2.0, 1.0], "prompt": "ab"}
    out = policy.infer(obs)
    images, state, noise, tokens = engine.seen
    assert torch.all(images[0] == -1.0) and torch.all(images[1] == 1.0) and torch.all(images[2] == -1.0)   # black, white, missing camera
    np.testing.assert_allclose(state[0, :3].numpy(), [(3 - 1) / (2 + 1e-6), 0.0, (1 - 3) / (2 + 1e-6)], rtol=1e-6)
    assert not state[0, 3:].any() and tokens.tolist() == [[97, 98, 7, 7]]
    assert noise.shape == (1, 5, 32) and float(noise.std()) > 0.5
    assert out["actions"].shape == (5, 2)
    np.testing.assert_allclose(out["actions"][0], [state[0, 0] * (1 + 1e-6) + 10, state[0, 1] * (3 + 1e-6) + 20], rtol=1e-5)
    fixed = policy.infer(obs, noise=np.ones((5, 32)))
    assert torch.all(engine.seen[2] == 1.0) and fixed["actions"].shape == (5, 2)
    with pytest.raises(ValueError):
        Pi0Policy(engine, cameras=("a", "b"))
    with pytest.raises(ValueError):
        Pi0Policy(engine)                                        # prompt length 4 but no tokenizer
    with pytest.raises(ValueError):
        Pi0Policy(engine, tokenizer=len).infer({"images": {}, "state": np.zeros(40)})     # more state dimensions than the model has


def _fake_policy(device):
    engine = FakeEngine(views=1, prompt=0, chunk=2, offset=float(device))
    return Pi0Policy(engine, cameras=("cam",))


def test_replica_pool_deals_requests_round_robin():
    observations = [{"images": {}, "state": [float(i)]} for i in range(5)]
    with ReplicaPool(_fake_policy, devices=[100, 200], start_method="spawn", startup_timeout=300) as pool:
        answers = pool.map(observations)
    for i, answer in enumerate(answers):
        replica = requests_for_ticket(i, 2)
        assert i in requests_for(replica, 2, 5)
        np.testing.assert_allclose(answer["actions"][0, 0], i + (100, 200)[replica])     # served by the replica it was dealt to
