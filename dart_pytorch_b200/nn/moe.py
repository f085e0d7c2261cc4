"""Mixture-of-experts feed-forward (reference: lib/core/nn/moe.dart:70-583).

Kept from the reference: router ``gateW [D, E]``; softmax or sigmoid gate; top-K chosen on ``score + routingBias`` (the
bias only steers the choice, never the combine weights); optional DeepSeek-V3 grouped routing (group score = max, or
sum of the top two for the sigmoid gate); optional renormalisation of the K weights; ``routeScale``; always-on shared
experts; dense execution (every expert on every token) and sparse execution (gather routed rows -> expert -> weight ->
scatter-add); aux-loss-free bias update from the load counters.

Added (options the benchmark configuration asks for, off by default): ``capacity_factor`` (each expert processes at
most ``ceil(cf * T * K / E)`` tokens, the rest are dropped for that expert), a Switch-style load-balance auxiliary loss
(``aux_loss_coef``; read it from ``last_aux_loss``), and bias-free experts.  Routing decisions are made on the device
(no score download); only the sparse path without a capacity reads the per-expert counts back.
"""
from __future__ import annotations

import math
from enum import Enum
from typing import List, Optional

import torch

from .. import ops as F
from .layers import Linear
from .module import Module, make_param, uniform_, normal_


class GateFunction(str, Enum):
    softmax = "softmax"
    sigmoid = "sigmoid"


class BiasUpdateRule(str, Enum):
    sign = "sign"
    proportional = "proportional"


class ExpertActivation(str, Enum):
    relu = "relu"
    silu = "silu"


class ExpertVariant(str, Enum):
    mlp = "mlp"
    swiGlu = "swiGlu"


class Expert(Module):
    """``w2(act(w1 x))`` or, for SwiGLU, ``w2(silu(w1 x) * w3 x)``; parameter order w1, w2, (w3)
    (reference: lib/core/nn/moe.dart:70-130).  For SwiGLU, ``w1`` and ``w3`` are stored as one ``[2H, D]`` weight."""

    def __init__(self, dim: int, hidden_dim: int, device=None, seed: int = 0, activation=ExpertActivation.relu,
                 variant=ExpertVariant.mlp, bias: bool = True, dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        self.dim, self.hidden_dim = dim, hidden_dim
        self.activation, self.variant = ExpertActivation(activation), ExpertVariant(variant)
        self.has_bias = bias
        w1 = Linear(dim, hidden_dim, bias=bias, device=device, seed=seed, dtype=dtype, init_std=init_std)
        self.w2 = Linear(hidden_dim, dim, bias=bias, device=device, seed=seed + 1, dtype=dtype, init_std=init_std)
        if self.variant == ExpertVariant.swiGlu:
            w3 = Linear(dim, hidden_dim, bias=bias, device=device, seed=seed + 2, dtype=dtype, init_std=init_std)
            self.w13 = make_param(torch.cat([w1.weight.data, w3.weight.data], 0))
            self.b13 = make_param(torch.cat([w1.bias.data, w3.bias.data], 0)) if bias else None
            self.w1 = None
        else:
            self.w1 = w1
            self.w13 = self.b13 = None

    def own_parameters(self):
        if self.w13 is None:
            return []
        return [self.w13] + ([self.b13] if self.b13 is not None else [])

    def submodules(self):
        return ([self.w1] if self.w1 is not None else []) + [self.w2]

    def _walk_params(self, reference: bool):
        H = self.hidden_dim
        if self.w13 is None:
            yield from self.w1._walk_params(reference)
            yield from self.w2._walk_params(reference)
            return
        if not reference:
            yield self.w13
            if self.b13 is not None:
                yield self.b13
            yield from self.w2._walk_params(False)
            return
        yield self.w13.data[:H]
        if self.b13 is not None:
            yield self.b13.data[:H].view(1, H)
        yield from self.w2._walk_params(True)
        yield self.w13.data[H:]
        if self.b13 is not None:
            yield self.b13.data[H:].view(1, H)

    def forward(self, x):
        if self.variant == ExpertVariant.swiGlu:
            return self.w2(F.swiglu(F.linear(x, self.w13, self.b13)))
        return self.w2(self.w1(x, activation=self.activation.value))


class MoEFeedForward(Module):
    def __init__(self, embed_dim: int, num_routed_experts: int, num_shared_experts: int, top_k: int,
                 expert_hidden_dim: int, bias_update_rate: float = 0.001, device=None, seed: int = 0,
                 activation=ExpertActivation.relu, expert_variant=ExpertVariant.mlp,
                 gate_function=GateFunction.softmax, bias_update_rule=BiasUpdateRule.sign, num_expert_groups: int = 1,
                 top_k_groups: Optional[int] = None, route_scale: float = 1.0, sparse_execution: bool = False,
                 renormalize_top_k: Optional[bool] = None, capacity_factor: Optional[float] = None,
                 aux_loss_coef: float = 0.0, expert_bias: bool = True, dtype=torch.float32,
                 init_std: Optional[float] = None):
        super().__init__()
        self.embed_dim, self.num_routed_experts, self.num_shared_experts = embed_dim, num_routed_experts, num_shared_experts
        self.top_k, self.expert_hidden_dim = top_k, expert_hidden_dim
        self.bias_update_rate = bias_update_rate
        self.gate_function = GateFunction(gate_function)
        self.bias_update_rule = BiasUpdateRule(bias_update_rule)
        self.num_expert_groups = num_expert_groups
        self.top_k_groups = num_expert_groups if top_k_groups is None else top_k_groups
        self.route_scale = route_scale
        self.sparse_execution = sparse_execution
        self.renormalize_top_k = (self.gate_function == GateFunction.sigmoid) if renormalize_top_k is None \
            else renormalize_top_k
        self.capacity_factor = capacity_factor
        self.aux_loss_coef = aux_loss_coef
        E = num_routed_experts
        if top_k <= 0 or top_k > E:
            raise ValueError(f"MoEFeedForward: topK ({top_k}) must be in [1, numRoutedExperts ({E})]")
        if num_expert_groups <= 0:
            raise ValueError(f"MoEFeedForward: numExpertGroups ({num_expert_groups}) must be >= 1")
        if E % num_expert_groups:
            raise ValueError("MoEFeedForward: numRoutedExperts must be divisible by numExpertGroups")
        if self.top_k_groups <= 0 or self.top_k_groups > num_expert_groups:
            raise ValueError("MoEFeedForward: topKGroups must be in [1, numExpertGroups]")
        if num_expert_groups > 1 and top_k > self.top_k_groups * (E // num_expert_groups):
            raise ValueError("MoEFeedForward: topK exceeds topKGroups * expertsPerGroup")
        bound = 1.0 / math.sqrt(embed_dim)
        gw = uniform_((embed_dim, E), bound, seed, device, dtype) if init_std is None else \
            normal_((embed_dim, E), init_std, seed, device, dtype)
        self.gate_w = make_param(gw)
        mk = lambda s: Expert(embed_dim, expert_hidden_dim, device=device, seed=s, activation=activation,  # noqa: E731
                              variant=expert_variant, bias=expert_bias, dtype=dtype, init_std=init_std)
        self.routed_experts: List[Expert] = [mk(seed + 1000 + i * 100) for i in range(E)]
        self.shared_experts: List[Expert] = [mk(seed + 500000 + i * 100) for i in range(num_shared_experts)]
        self.routing_bias = torch.zeros(E, dtype=torch.float32, device=device)
        self._expert_load = torch.zeros(E, dtype=torch.long, device=device)
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.last_dropped = 0

    def own_parameters(self):
        return [self.gate_w]

    def submodules(self):
        return list(self.routed_experts) + list(self.shared_experts)

    def _moved(self, device, dtype):
        if device is not None:
            self.routing_bias = self.routing_bias.to(device)
            self._expert_load = self._expert_load.to(device)

    @property
    def expert_load(self) -> List[int]:
        return [int(v) for v in self._expert_load.tolist()]

    expertLoad = expert_load

    @property
    def routingBias(self) -> List[float]:
        return [float(v) for v in self.routing_bias.tolist()]

    # ---- routing ---------------------------------------------------------------------------------
    def route(self, scores: torch.Tensor) -> torch.Tensor:
        """0/1 mask ``[T, E]`` of the top-K experts per token chosen on ``scores + routingBias`` (grouped when
        configured).  No gradient flows through the choice."""
        T, E = scores.shape
        with torch.no_grad():
            biased = scores.detach().float() + self.routing_bias.to(scores.device)
            G = self.num_expert_groups
            if G > 1:
                per = E // G
                grp = biased.view(T, G, per)
                if self.gate_function == GateFunction.sigmoid and per >= 2:
                    gscore = grp.topk(2, dim=-1).values.sum(-1)
                else:
                    gscore = grp.max(dim=-1).values
                keep_g = torch.zeros(T, G, dtype=torch.bool, device=scores.device)
                keep_g.scatter_(1, gscore.topk(self.top_k_groups, dim=-1).indices, True)
                biased = torch.where(keep_g.unsqueeze(-1).expand(T, G, per).reshape(T, E), biased,
                                     torch.full_like(biased, float("-inf")))
            idx = biased.topk(self.top_k, dim=-1).indices
            mask = torch.zeros(T, E, dtype=scores.dtype, device=scores.device)
            mask.scatter_(1, idx, 1.0)
            if self.capacity_factor is not None:
                cap = int(math.ceil(self.capacity_factor * T * self.top_k / E))
                rank_in_expert = torch.cumsum(mask.float(), dim=0) * mask.float()   # 1-based arrival order per expert
                kept = (rank_in_expert <= cap) & (mask > 0)
                self.last_dropped = int((mask.sum() - kept.sum()).item()) if not scores.is_cuda else -1
                mask = kept.to(scores.dtype)
            self._expert_load += mask.sum(0).to(torch.long)
        return mask

    def forward(self, x):
        if x.dim() != 2 or x.shape[1] != self.embed_dim:
            raise ValueError(f"MoEFeedForward: expected 2D input [T, {self.embed_dim}]; got {list(x.shape)}")
        T, E = x.shape[0], self.num_routed_experts
        logits = F.matmul(x, self.gate_w)
        scores = F.softmax(logits) if self.gate_function == GateFunction.softmax else F.sigmoid(logits)
        mask = self.route(scores)
        masked = F.mul(scores, mask)
        if self.aux_loss_coef > 0.0:
            # Switch-style balance term: E * sum_j (fraction of routed slots on j) * (mean gate probability of j).
            frac = (mask.float().sum(0) / max(1.0, float(T * self.top_k))).to(scores.dtype).detach()
            prob = scores.float().mean(0) if not scores.is_cuda else \
                F.mul(F.matmul(torch.ones(1, T, dtype=scores.dtype, device=scores.device), scores), 1.0 / T).reshape(-1)
            self.last_aux_loss = (prob.float() * frac.float()).sum() * (E * self.aux_loss_coef)
        else:
            self.last_aux_loss = None
        if self.renormalize_top_k:
            ones_e1 = torch.ones(E, 1, dtype=masked.dtype, device=masked.device)
            ones_1e = torch.ones(1, E, dtype=masked.dtype, device=masked.device)
            row = F.matmul(F.matmul(masked, ones_e1), ones_1e)
            masked = F.div(masked, F.add(row, 1e-9))
        if self.route_scale != 1.0:
            masked = F.mul(masked, self.route_scale)
        acc = None
        if self.sparse_execution:
            counts = mask.sum(0).to(torch.long).tolist()
            for j in range(E):
                if counts[j] == 0:
                    continue
                idx = torch.nonzero(mask[:, j] > 0, as_tuple=False).reshape(-1)
                xs = F.embedding(x, idx)
                onehot = torch.zeros(E, 1, dtype=masked.dtype, device=masked.device)
                onehot[j, 0] = 1.0
                w = F.embedding(F.matmul(masked, onehot), idx)                      # [K_j, 1]
                wb = F.matmul(w, torch.ones(1, self.embed_dim, dtype=w.dtype, device=w.device))
                contrib = F.scatter_rows_add(F.mul(self.routed_experts[j](xs), wb), idx, T)
                acc = contrib if acc is None else F.add(acc, contrib)
            if acc is None:
                acc = torch.zeros(T, self.embed_dim, dtype=x.dtype, device=x.device)
        else:
            for j in range(E):
                sel = torch.zeros(E, self.embed_dim, dtype=masked.dtype, device=masked.device)
                sel[j] = 1.0
                gate_col = F.matmul(masked, sel)
                weighted = F.mul(gate_col, self.routed_experts[j](x))
                acc = weighted if acc is None else F.add(acc, weighted)
        for s in self.shared_experts:
            o = s(x)
            acc = o if acc is None else F.add(acc, o)
        return acc

    def update_routing_bias(self) -> None:
        """Aux-loss-free balancing: raise the bias of under-loaded experts, lower it for over-loaded ones, then reset
        the load counters (reference: lib/core/nn/moe.dart:550-569)."""
        load = self._expert_load.float()
        total = float(load.sum().item())
        if total == 0:
            return
        mean = total / self.num_routed_experts
        e = mean - load
        delta = torch.sign(e) if self.bias_update_rule == BiasUpdateRule.sign else e / mean
        self.routing_bias += self.bias_update_rate * delta.to(self.routing_bias.device)
        self._expert_load.zero_()

    updateRoutingBias = update_routing_bias
