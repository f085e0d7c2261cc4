"""Model presets of cooperative training (reference: lib/core/coop/lm_factory.dart:29-174): ``tiny`` (ctx 32, D 32,
2 layers, 4 heads) and ``small`` (ctx 64, D 128, 4 layers, 8 heads) for the GPT and AFT architectures."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable

from ..models.gpt import GPT, GPTConfig
from ..models.seq_models import AFTLanguageModel
from ..nn.module import Module


class Arch(str, Enum):
    gpt = "gpt"
    aft = "aft"


def parse_arch(s: str) -> Arch:
    try:
        return Arch(s.lower())
    except ValueError:
        raise ValueError(f'unknown arch "{s}" (expected gpt|aft)') from None


def arch_to_string(a: Arch) -> str:
    return Arch(a).value


@dataclass
class CoopLM:
    arch: Arch
    model_size: str
    module: Module
    forward: Callable
    max_len: int

    def __call__(self, tokens):
        return self.forward(tokens)

    def loss(self, tokens, targets):
        return self.module.loss(tokens, targets)

    @property
    def scalar_count(self) -> int:
        return sum(p.numel() for p in self.module.parameters())

    scalarCount = scalar_count


_GPT = {"tiny": dict(max_ctx=32, embed_dim=32, num_layers=2, num_heads=4),
        "small": dict(max_ctx=64, embed_dim=128, num_layers=4, num_heads=8)}
_AFT = {"tiny": dict(max_len=32, embed_dim=32, num_layers=2, ffn_dim=128),
        "small": dict(max_len=64, embed_dim=128, num_layers=4, ffn_dim=512)}


def build_coop_lm(arch, model_size: str, vocab_size: int, device=None, seed: int = 0) -> CoopLM:
    arch = Arch(arch)
    if model_size not in _GPT:
        raise ValueError(f'unknown model size "{model_size}" (expected tiny|small)')
    if arch == Arch.gpt:
        cfg = GPTConfig(vocab_size=vocab_size, dropout_p=0.0, tie_weights=True, device=device, seed=seed,
                        **_GPT[model_size])
        gpt = GPT(cfg)
        return CoopLM(arch, model_size, gpt, gpt, cfg.max_ctx)
    dims = _AFT[model_size]
    aft = AFTLanguageModel(vocab_size=vocab_size, dropout_p=0.0, device=device, seed=seed, **dims)
    return CoopLM(arch, model_size, aft, aft, dims["max_len"])


parseArch, archToString, buildCoopLM = parse_arch, arch_to_string, build_coop_lm
