"""MuZero-style latent planner over token observations (reference: lib/core/nn/muzero_lm.dart:72-443).

``representation``: tokens ``[T]`` -> embedding + learned positions -> encoder -> mean row ``[1, D]``.
``dynamics``: ``(state [1, D], action id) -> (state + stateHead(relu(fuse([state, emb(action)]))), reward [1, 1])``.
``prediction``: ``state -> (policy logits [1, A], value [1, 1])``.
``MuZeroLM.unroll(obs, actions)`` chains one initial and ``len(actions)`` recurrent inferences.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, NamedTuple, Optional

import torch

from .. import ops as F
from ..nn.layers import Embedding, LearnedPositionalEmbedding, Linear
from ..nn.module import Module
from ..nn.transformer import TransformerEncoder
from .gpt import _as_token_tensor
from .modalities import mean_rows


class MuZeroRepresentation(Module):
    def __init__(self, vocab_size: int, max_obs_len: int, embed_dim: int, num_layers: int = 2, num_heads: int = 4,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.max_obs_len, self.embed_dim = vocab_size, max_obs_len, embed_dim
        self.token_embed = Embedding(vocab_size, embed_dim, device=device, seed=seed, dtype=dtype)
        self.pos_embed = LearnedPositionalEmbedding(max_obs_len, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, dropout_p=dropout_p, device=device,
                                          seed=seed + 100, dtype=dtype)

    def submodules(self):
        return [self.token_embed, self.pos_embed, self.encoder]

    def forward(self, obs_tokens):
        obs_tokens = _as_token_tensor(obs_tokens, self.device)
        if obs_tokens.dim() != 1:
            raise ValueError(f"MuZeroRepresentation: expected [T] token ids; got {list(obs_tokens.shape)}")
        if obs_tokens.shape[0] > self.max_obs_len:
            raise ValueError(f"MuZeroRepresentation: obs length {obs_tokens.shape[0]} exceeds maxObsLen "
                             f"{self.max_obs_len}")
        return mean_rows(self.encoder(self.pos_embed(self.token_embed(obs_tokens))))


class DynamicsOut(NamedTuple):
    next_state: torch.Tensor
    reward: torch.Tensor


class PredictionOut(NamedTuple):
    policy: torch.Tensor
    value: torch.Tensor


class InitialOut(NamedTuple):
    state: torch.Tensor
    policy: torch.Tensor
    value: torch.Tensor


class RecurrentOut(NamedTuple):
    next_state: torch.Tensor
    reward: torch.Tensor
    policy: torch.Tensor
    value: torch.Tensor


class MuZeroDynamics(Module):
    def __init__(self, embed_dim: int, num_actions: int, hidden_dim: Optional[int] = None, device=None, seed: int = 0,
                 dtype=torch.float32):
        super().__init__()
        self.embed_dim, self.num_actions = embed_dim, num_actions
        self.hidden_dim = hidden_dim or embed_dim * 2
        self.action_embed = Embedding(num_actions, embed_dim, device=device, seed=seed, dtype=dtype)
        self.fuse = Linear(embed_dim * 2, self.hidden_dim, device=device, seed=seed + 1, dtype=dtype)
        self.state_head = Linear(self.hidden_dim, embed_dim, device=device, seed=seed + 2, dtype=dtype)
        self.reward_head = Linear(self.hidden_dim, 1, device=device, seed=seed + 3, dtype=dtype)

    def submodules(self):
        return [self.action_embed, self.fuse, self.state_head, self.reward_head]

    def forward(self, state, action_id: int) -> DynamicsOut:
        if state.dim() != 2 or state.shape[0] != 1 or state.shape[1] != self.embed_dim:
            raise ValueError(f"MuZeroDynamics: expected state [1, {self.embed_dim}]; got {list(state.shape)}")
        if not (0 <= action_id < self.num_actions):
            raise ValueError(f"MuZeroDynamics: action {action_id} out of [0, {self.num_actions})")
        a_emb = self.action_embed(torch.tensor([action_id], dtype=torch.long, device=state.device))
        h = self.fuse(F.concat([state, a_emb], axis=1), activation="relu")
        nxt = self.state_head(h, residual=state)
        return DynamicsOut(nxt, self.reward_head(h))


class MuZeroPrediction(Module):
    def __init__(self, embed_dim: int, num_actions: int, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.embed_dim, self.num_actions = embed_dim, num_actions
        self.policy_head = Linear(embed_dim, num_actions, device=device, seed=seed, dtype=dtype)
        self.value_head = Linear(embed_dim, 1, device=device, seed=seed + 1, dtype=dtype)

    def submodules(self):
        return [self.policy_head, self.value_head]

    def forward(self, state) -> PredictionOut:
        if state.dim() != 2 or state.shape[0] != 1 or state.shape[1] != self.embed_dim:
            raise ValueError(f"MuZeroPrediction: expected state [1, {self.embed_dim}]; got {list(state.shape)}")
        return PredictionOut(self.policy_head(state), self.value_head(state))


@dataclass
class MuZeroUnroll:
    states: List[torch.Tensor] = field(default_factory=list)
    policies: List[torch.Tensor] = field(default_factory=list)
    values: List[torch.Tensor] = field(default_factory=list)
    rewards: List[torch.Tensor] = field(default_factory=list)


class MuZeroLM(Module):
    def __init__(self, vocab_size: int, max_obs_len: int, embed_dim: int, num_actions: int, num_layers: int = 2,
                 num_heads: int = 4, dynamics_hidden_dim: Optional[int] = None, dropout_p: float = 0.0, device=None,
                 seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.max_obs_len, self.embed_dim, self.num_actions = (vocab_size, max_obs_len, embed_dim,
                                                                               num_actions)
        self.representation = MuZeroRepresentation(vocab_size, max_obs_len, embed_dim, num_layers, num_heads,
                                                   dropout_p, device=device, seed=seed + 1000, dtype=dtype)
        self.dynamics = MuZeroDynamics(embed_dim, num_actions, dynamics_hidden_dim, device=device, seed=seed + 2000,
                                       dtype=dtype)
        self.prediction = MuZeroPrediction(embed_dim, num_actions, device=device, seed=seed + 3000, dtype=dtype)

    def submodules(self):
        return [self.representation, self.dynamics, self.prediction]

    def initial_inference(self, obs_tokens) -> InitialOut:
        state = self.representation(obs_tokens)
        pv = self.prediction(state)
        return InitialOut(state, pv.policy, pv.value)

    def recurrent_inference(self, state, action: int) -> RecurrentOut:
        d = self.dynamics(state, action)
        pv = self.prediction(d.next_state)
        return RecurrentOut(d.next_state, d.reward, pv.policy, pv.value)

    def unroll(self, obs_tokens, actions: List[int]) -> MuZeroUnroll:
        init = self.initial_inference(obs_tokens)
        u = MuZeroUnroll([init.state], [init.policy], [init.value], [])
        for a in actions:
            r = self.recurrent_inference(u.states[-1], int(a))
            u.states.append(r.next_state)
            u.policies.append(r.policy)
            u.values.append(r.value)
            u.rewards.append(r.reward)
        return u

    initialInference, recurrentInference = initial_inference, recurrent_inference

    def forward(self, obs_tokens):
        return self.initial_inference(obs_tokens)
