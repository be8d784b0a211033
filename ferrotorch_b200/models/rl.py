"""Actor-critic MLP policy compatible with stable-baselines3 ``MlpPolicy`` checkpoints (PPO / A2C).

Reference parity: ferrotorch-rl/src/{mlp_policy.rs:60,432, loader.rs:66}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .. import nn
from ..errors import InvalidArgument
from .bert import DropReport


@dataclass
class MlpPolicyConfig:
    obs_dim: int = 4
    action_dim: int = 2
    discrete: bool = True
    pi_layers: List[int] = field(default_factory=lambda: [64, 64])
    vf_layers: List[int] = field(default_factory=lambda: [64, 64])
    activation: str = "tanh"
    log_std_init: float = 0.0

    @classmethod
    def cartpole_v1(cls) -> "MlpPolicyConfig":
        """sb3's ``MlpPolicy`` defaults for CartPole-v1: 4 observations, two Tanh layers of 64, 2 actions (ferrotorch-rl/src/mlp_policy.rs:72)."""
        return cls(obs_dim=4, action_dim=2, discrete=True, pi_layers=[64, 64], vf_layers=[64, 64])

    @classmethod
    def discrete_mlp(cls, obs_dim: int, hidden: int, n_actions: int) -> "MlpPolicyConfig":
        """The reference's three-field form ``(obs_dim, hidden, n_actions)`` (mlp_policy.rs:60-67)."""
        return cls(obs_dim=obs_dim, action_dim=n_actions, discrete=True, pi_layers=[hidden, hidden], vf_layers=[hidden, hidden])

    @property
    def hidden(self) -> int:
        return self.pi_layers[-1]

    @property
    def n_actions(self) -> int:
        return self.action_dim


def _mlp(inp, sizes, act):
    layers, d = [], inp
    for s in sizes:
        layers += [nn.Linear(d, s), act()]
        d = s
    return nn.Sequential(*layers), d


class MlpExtractor(nn.Module):
    """sb3's two separate trunks ``policy_net`` / ``value_net`` (``Linear -> act`` per layer, so the linears sit at Sequential slots 0, 2, ...
    and checkpoint keys match). ``MlpExtractor(obs_dim, hidden)`` is the reference's two-Tanh-layer form (ferrotorch-rl/src/mlp_policy.rs:93-170)."""

    def __init__(self, c, act=None):
        super().__init__()
        if not isinstance(c, MlpPolicyConfig):
            c, act = MlpPolicyConfig.discrete_mlp(int(c), int(act if act is not None else 64), 1), nn.Tanh
        self._obs_dim = c.obs_dim
        self.policy_net, self.pi_dim = _mlp(c.obs_dim, c.pi_layers, act or nn.Tanh)
        self.value_net, self.vf_dim = _mlp(c.obs_dim, c.vf_layers, act or nn.Tanh)

    def forward_actor(self, features):
        return self.policy_net(features)

    def forward_critic(self, features):
        return self.value_net(features)

    def forward(self, features):
        return self.policy_net(features), self.value_net(features)

    def obs_dim(self) -> int:
        return self._obs_dim

    def hidden(self) -> int:
        return self.pi_dim


_Extractor = MlpExtractor


class ActionNet(nn.Linear):
    """Policy latent -> action logits (or means) (ferrotorch-rl/src/mlp_policy.rs:249)."""

    def __init__(self, hidden: int, n_actions: int):
        super().__init__(hidden, n_actions)


class ValueHead(nn.Linear):
    """Value latent -> one state value per row, ``[B, 1]`` (ferrotorch-rl/src/mlp_policy.rs:324)."""

    def __init__(self, hidden: int):
        super().__init__(hidden, 1)


@dataclass
class PolicyOutput:
    """Raw action logits ``[B, n_actions]`` and state values ``[B, 1]`` (ferrotorch-rl/src/mlp_policy.rs:392)."""
    action_logits: torch.Tensor
    value: torch.Tensor


class MlpPolicy(nn.Module):
    def __init__(self, c: MlpPolicyConfig):
        super().__init__()
        act = {"tanh": nn.Tanh, "relu": nn.ReLU}.get(c.activation)
        if act is None:
            raise InvalidArgument(f"unknown activation {c.activation}")
        self.config = c
        self.mlp_extractor = _Extractor(c, act)
        self.action_net = ActionNet(self.mlp_extractor.pi_dim, c.action_dim)
        self.value_net = ValueHead(self.mlp_extractor.vf_dim)
        if not c.discrete:
            self.log_std = nn.Parameter(torch.full((c.action_dim,), c.log_std_init))

    def distribution(self, obs):
        from .. import distributions as D
        z = self.action_net(self.mlp_extractor.policy_net(obs))
        return D.Categorical(logits=z) if self.config.discrete else D.Normal(z, self.log_std.exp().expand_as(z))

    def policy_output(self, obs) -> PolicyOutput:
        """Logits and ``[B, 1]`` values in one pass, the reference's ``forward`` (ferrotorch-rl/src/mlp_policy.rs:485)."""
        return PolicyOutput(self.action_net(self.mlp_extractor.policy_net(obs)), self.value_net(self.mlp_extractor.value_net(obs)))

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


def load_ppo_policy(path: str, config: MlpPolicyConfig, strict: Optional[bool] = None):
    """Loads an sb3 ``policy.pth`` state dict (torch zip format) or a safetensors file with the same names. Every parameter of the policy must be
    in the file. With ``strict`` given (the reference's form, ferrotorch-rl/src/safetensors_loader.rs:66) the result is ``(policy, DropReport)``:
    file keys that match no parameter are refused (``True``) or listed in ``report.unmapped`` (``False``); without it, the policy alone."""
    from ..serialize import load_pytorch_state_dict, load_safetensors
    try:
        sd = load_safetensors(path) if str(path).endswith(".safetensors") else load_pytorch_state_dict(path)
    except Exception as e:
        raise InvalidArgument(f"load_ppo_policy: failed to decode {path}: {e}") from None
    m = MlpPolicy(config)
    own = m.state_dict()
    unmapped = sorted(k for k in sd if k not in own)
    if strict and unmapped:
        raise InvalidArgument(f"load_ppo_policy: unmapped upstream keys (strict mode): {unmapped}")
    if strict is not None:
        missing = [k for k in own if k not in sd]
        if missing:
            raise InvalidArgument(f"load_ppo_policy: missing keys {missing}")
    m.load_state_dict({k: v for k, v in sd.items() if k in own}, strict=False)
    return m if strict is None else (m, DropReport(unmapped=tuple(unmapped)))
