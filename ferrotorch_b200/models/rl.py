"""Actor-critic MLP policy compatible with stable-baselines3 ``MlpPolicy`` checkpoints (PPO / A2C).

Reference parity: ferrotorch-rl/src/{mlp_policy.rs:60,432, loader.rs:66}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .. import nn
from ..errors import InvalidArgument


@dataclass
class MlpPolicyConfig:
    obs_dim: int = 4
    action_dim: int = 2
    discrete: bool = True
    pi_layers: List[int] = field(default_factory=lambda: [64, 64])
    vf_layers: List[int] = field(default_factory=lambda: [64, 64])
    activation: str = "tanh"
    log_std_init: float = 0.0


def _mlp(inp, sizes, act):
    layers, d = [], inp
    for s in sizes:
        layers += [nn.Linear(d, s), act()]
        d = s
    return nn.Sequential(*layers), d


class _Extractor(nn.Module):
    def __init__(self, c, act):
        super().__init__()
        self.policy_net, self.pi_dim = _mlp(c.obs_dim, c.pi_layers, act)
        self.value_net, self.vf_dim = _mlp(c.obs_dim, c.vf_layers, act)


class MlpPolicy(nn.Module):
    def __init__(self, c: MlpPolicyConfig):
        super().__init__()
        act = {"tanh": nn.Tanh, "relu": nn.ReLU}.get(c.activation)
        if act is None:
            raise InvalidArgument(f"unknown activation {c.activation}")
        self.config = c
        self.mlp_extractor = _Extractor(c, act)
        self.action_net = nn.Linear(self.mlp_extractor.pi_dim, c.action_dim)
        self.value_net = nn.Linear(self.mlp_extractor.vf_dim, 1)
        if not c.discrete:
            self.log_std = nn.Parameter(torch.full((c.action_dim,), c.log_std_init))

    def distribution(self, obs):
        from .. import distributions as D
        z = self.action_net(self.mlp_extractor.policy_net(obs))
        return D.Categorical(logits=z) if self.config.discrete else D.Normal(z, self.log_std.exp().expand_as(z))

    def value(self, obs):
        return self.value_net(self.mlp_extractor.value_net(obs)).squeeze(-1)

    def forward(self, obs, deterministic: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns (action, value, log_prob)."""
        dist = self.distribution(obs)
        if deterministic:
            a = dist.logits.argmax(-1) if self.config.discrete else dist.loc
        else:
            a = dist.sample()
        lp = dist.log_prob(a)
        return a, self.value(obs), (lp if self.config.discrete else lp.sum(-1))

    def evaluate_actions(self, obs, actions):
        dist = self.distribution(obs)
        lp, ent = dist.log_prob(actions), dist.entropy()
        if not self.config.discrete:
            lp, ent = lp.sum(-1), ent.sum(-1)
        return self.value(obs), lp, ent

    def predict(self, obs, deterministic: bool = True):
        with torch.no_grad():
            return self.forward(obs, deterministic)[0]


def ppo_loss(policy: MlpPolicy, obs, actions, old_log_prob, advantages, returns, clip_range=0.2, vf_coef=0.5, ent_coef=0.0):
    values, lp, ent = policy.evaluate_actions(obs, actions)
    ratio = (lp - old_log_prob).exp()
    pg = -torch.min(ratio * advantages, ratio.clamp(1 - clip_range, 1 + clip_range) * advantages).mean()
    return pg + vf_coef * torch.nn.functional.mse_loss(values, returns) - ent_coef * ent.mean()


def load_ppo_policy(path: str, config: MlpPolicyConfig) -> MlpPolicy:
    """Loads an sb3 ``policy.pth`` state dict (torch zip format) or a safetensors file with the same names."""
    from ..serialize import load_pytorch_state_dict, load_safetensors
    sd = load_safetensors(path) if path.endswith(".safetensors") else load_pytorch_state_dict(path)
    m = MlpPolicy(config)
    m.load_state_dict({k: v for k, v in sd.items() if k in m.state_dict()}, strict=False)
    return m
