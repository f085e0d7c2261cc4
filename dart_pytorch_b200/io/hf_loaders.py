"""HuggingFace weight loaders for GPT-2 and Llama checkpoints
(reference: lib/core/nn/gpt2_hf_loader.dart:57-372, lib/core/nn/llama_hf_loader.dart:43-221).

Both take a ``{name: tensor}`` state dict (from ``SafeTensors.load_file`` / ``load_sharded``), check every shape, copy
in place and return a report ``{consumed_count, unused_keys, missing_keys}``; a missing or mis-shaped tensor raises.
Because projections are stored fused here, the reference's per-head slicing disappears: GPT-2's Conv1D ``c_attn``
``[D, 3D]`` transposes straight into the fused ``[3D, D]`` QKV weight, and Llama's ``q_proj / k_proj / v_proj`` rows
concatenate into it (rows of head ``h`` are ``[h*hd, (h+1)*hd)``, the same split the reference makes).
``dump_*`` produce HF-named state dicts from a model (round-trip tests, exports).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..models.gpt import GPT, GPTConfig
from ..models.llama import Llama, LlamaConfig
from ..nn.transformer import Activation
from .safetensors import SafeTensors


@dataclass
class LoadReport:
    consumed_count: int = 0
    unused_keys: List[str] = field(default_factory=list)
    missing_keys: List[str] = field(default_factory=list)

    consumedCount = property(lambda self: self.consumed_count)
    unusedKeys = property(lambda self: self.unused_keys)
    missingKeys = property(lambda self: self.missing_keys)


class _Taker:
    def __init__(self, state: Dict[str, torch.Tensor], who: str):
        self.state, self.who = state, who
        self.consumed = set()

    def take(self, name: str, shape) -> torch.Tensor:
        t = self.state.get(name)
        if t is None:
            raise ValueError(f'{self.who} loader: missing tensor "{name}"')
        if list(t.shape) != list(shape):
            raise ValueError(f'{self.who} loader: "{name}" has shape {list(t.shape)}, expected {list(shape)}')
        self.consumed.add(name)
        return t

    def has(self, name: str) -> bool:
        return name in self.state

    def report(self, ignorable=()) -> LoadReport:
        unused = sorted(k for k in self.state if k not in self.consumed)
        return LoadReport(len(self.consumed), unused, [])


def _copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    with torch.no_grad():
        dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
    arena = getattr(dst, "_dptb_arena", None)
    if arena is not None and arena.master is not None:
        arena.master_view(dst).copy_(src.to(arena.master.device, torch.float32))


class GPT2HFLoader:
    @staticmethod
    def _cfg(embed, layers, heads, device=None, seed=0, dtype=torch.float32) -> GPTConfig:
        return GPTConfig(vocab_size=50257, max_ctx=1024, embed_dim=embed, num_layers=layers, num_heads=heads,
                         dropout_p=0.0, tie_weights=True, attn_bias=True, activation=Activation.geluTanh,
                         device=device, seed=seed, dtype=dtype)

    @staticmethod
    def gpt2_small_config(**kw):
        return GPT2HFLoader._cfg(768, 12, 12, **kw)

    @staticmethod
    def distil_gpt2_config(**kw):
        return GPT2HFLoader._cfg(768, 6, 12, **kw)

    @staticmethod
    def gpt2_medium_config(**kw):
        return GPT2HFLoader._cfg(1024, 24, 16, **kw)

    @staticmethod
    def gpt2_large_config(**kw):
        return GPT2HFLoader._cfg(1280, 36, 20, **kw)

    @staticmethod
    def gpt2_xl_config(**kw):
        return GPT2HFLoader._cfg(1600, 48, 25, **kw)

    gpt2SmallConfig, distilGpt2Config, gpt2MediumConfig = gpt2_small_config, distil_gpt2_config, gpt2_medium_config
    gpt2LargeConfig, gpt2XLConfig = gpt2_large_config, gpt2_xl_config

    @staticmethod
    def load_file(gpt: GPT, path: str, keep_fp16: bool = False) -> LoadReport:
        return GPT2HFLoader.load_map(gpt, SafeTensors.load_file(path, keep_fp16=keep_fp16))

    @staticmethod
    def load_sharded(gpt: GPT, index_path: str, keep_fp16: bool = False) -> LoadReport:
        return GPT2HFLoader.load_map(gpt, SafeTensors.load_sharded(index_path, keep_fp16=keep_fp16))

    @staticmethod
    def load_map(gpt: GPT, state_in: Dict[str, torch.Tensor]) -> LoadReport:
        state = state_in
        if state_in and all(k.startswith("transformer.") or k.startswith("lm_head.") for k in state_in):
            state = {(k[len("transformer."):] if k.startswith("transformer.") else k): v for k, v in state_in.items()}
        t = _Taker(state, "gpt2")
        c = gpt.config
        d, ffn = c.embed_dim, c.ffn_dim or 4 * c.embed_dim
        if not c.attn_bias:
            raise ValueError("gpt2 loader: the target GPT must be built with attnBias: true")
        _copy(gpt.token_emb.weight, t.take("wte.weight", [c.vocab_size, d]))
        _copy(gpt.pos_emb.table.weight, t.take("wpe.weight", [c.max_ctx, d]))
        for i, blk in enumerate(gpt.encoder.blocks):
            p = f"h.{i}"
            _copy(blk.ln1.gamma, t.take(f"{p}.ln_1.weight", [d]))
            _copy(blk.ln1.beta, t.take(f"{p}.ln_1.bias", [d]))
            # Conv1D stores [in, out]: transpose into the fused [3D, D] projection (rows: q heads, k heads, v heads).
            _copy(blk.mha.w_qkv, t.take(f"{p}.attn.c_attn.weight", [d, 3 * d]).float().t())
            _copy(blk.mha.b_qkv, t.take(f"{p}.attn.c_attn.bias", [3 * d]))
            _copy(blk.mha.wo.weight, t.take(f"{p}.attn.c_proj.weight", [d, d]).float().t())
            _copy(blk.mha.wo.bias, t.take(f"{p}.attn.c_proj.bias", [d]))
            _copy(blk.ln2.gamma, t.take(f"{p}.ln_2.weight", [d]))
            _copy(blk.ln2.beta, t.take(f"{p}.ln_2.bias", [d]))
            _copy(blk.ffn1.weight, t.take(f"{p}.mlp.c_fc.weight", [d, ffn]).float().t())
            _copy(blk.ffn1.bias, t.take(f"{p}.mlp.c_fc.bias", [ffn]))
            _copy(blk.ffn2.weight, t.take(f"{p}.mlp.c_proj.weight", [ffn, d]).float().t())
            _copy(blk.ffn2.bias, t.take(f"{p}.mlp.c_proj.bias", [d]))
        _copy(gpt.encoder.final_norm.gamma, t.take("ln_f.weight", [d]))
        _copy(gpt.encoder.final_norm.beta, t.take("ln_f.bias", [d]))
        if gpt.untied_head is not None:   # HF saves no separate head: fall back to wte
            _copy(gpt.untied_head.weight, state["wte.weight"])
        return t.report()

    @staticmethod
    def dump(gpt: GPT, prefix: str = "") -> Dict[str, torch.Tensor]:
        out = {prefix + "wte.weight": gpt.token_emb.weight.detach().float().cpu(),
               prefix + "wpe.weight": gpt.pos_emb.table.weight.detach().float().cpu()}
        for i, blk in enumerate(gpt.encoder.blocks):
            p = f"{prefix}h.{i}"
            f32 = lambda x: x.detach().float().cpu()  # noqa: E731
            out.update({f"{p}.ln_1.weight": f32(blk.ln1.gamma), f"{p}.ln_1.bias": f32(blk.ln1.beta),
                        f"{p}.attn.c_attn.weight": f32(blk.mha.w_qkv).t().contiguous(),
                        f"{p}.attn.c_attn.bias": f32(blk.mha.b_qkv),
                        f"{p}.attn.c_proj.weight": f32(blk.mha.wo.weight).t().contiguous(),
                        f"{p}.attn.c_proj.bias": f32(blk.mha.wo.bias),
                        f"{p}.ln_2.weight": f32(blk.ln2.gamma), f"{p}.ln_2.bias": f32(blk.ln2.beta),
                        f"{p}.mlp.c_fc.weight": f32(blk.ffn1.weight).t().contiguous(),
                        f"{p}.mlp.c_fc.bias": f32(blk.ffn1.bias),
                        f"{p}.mlp.c_proj.weight": f32(blk.ffn2.weight).t().contiguous(),
                        f"{p}.mlp.c_proj.bias": f32(blk.ffn2.bias)})
        out[prefix + "ln_f.weight"] = gpt.encoder.final_norm.gamma.detach().float().cpu()
        out[prefix + "ln_f.bias"] = gpt.encoder.final_norm.beta.detach().float().cpu()
        return out

    loadFile, loadSharded, loadMap = load_file, load_sharded, load_map


class LlamaHFLoader:
    @staticmethod
    def _cfg(embed, layers, heads, ffn, tie, max_ctx=None, device=None, seed=0, dtype=torch.float32) -> LlamaConfig:
        return LlamaConfig(vocab_size=128256, max_ctx=max_ctx or 131072, embed_dim=embed, num_layers=layers,
                           num_heads=heads, num_kv_heads=8, ffn_dim=ffn, rope_base=500000.0, rms_norm_eps=1e-5,
                           tie_weights=tie, device=device, seed=seed, dtype=dtype)

    @staticmethod
    def llama32_1b_config(**kw):
        return LlamaHFLoader._cfg(2048, 16, 32, 8192, True, **kw)

    @staticmethod
    def llama32_3b_config(**kw):
        return LlamaHFLoader._cfg(3072, 28, 24, 8192, True, **kw)

    @staticmethod
    def llama31_8b_config(**kw):
        return LlamaHFLoader._cfg(4096, 32, 32, 14336, False, **kw)

    llama32_1BConfig, llama32_3BConfig, llama31_8BConfig = llama32_1b_config, llama32_3b_config, llama31_8b_config

    @staticmethod
    def load_file(model: Llama, path: str, keep_fp16: bool = False) -> LoadReport:
        return LlamaHFLoader.load_map(model, SafeTensors.load_file(path, keep_fp16=keep_fp16))

    @staticmethod
    def load_sharded(model: Llama, index_path: str, keep_fp16: bool = False) -> LoadReport:
        """Shards are streamed: at most one shard is resident beside the model."""
        t_all = _Taker({}, "llama")
        total = LoadReport()

        def on_shard(part):
            t_all.state.update({k: v for k, v in part.items()})
        SafeTensors.stream_sharded(index_path, on_shard, keep_fp16=keep_fp16)
        return LlamaHFLoader.load_map(model, t_all.state)

    @staticmethod
    def load_map(model: Llama, state: Dict[str, torch.Tensor]) -> LoadReport:
        t = _Taker(state, "llama")
        c = model.config
        d, hd, H, Hkv, F_ = c.embed_dim, c.head_dim, c.num_heads, c.num_kv_heads, c.ffn_dim
        _copy(model.embed_in.weight, t.take("model.embed_tokens.weight", [c.vocab_size, d]))
        for i, blk in enumerate(model.blocks):
            p = f"model.layers.{i}"
            _copy(blk.attn_norm.gamma, t.take(f"{p}.input_layernorm.weight", [d]))
            q = t.take(f"{p}.self_attn.q_proj.weight", [H * hd, d])
            k = t.take(f"{p}.self_attn.k_proj.weight", [Hkv * hd, d])
            v = t.take(f"{p}.self_attn.v_proj.weight", [Hkv * hd, d])
            _copy(blk.attn.w_qkv, torch.cat([q.float(), k.float(), v.float()], 0))
            _copy(blk.attn.wo.weight, t.take(f"{p}.self_attn.o_proj.weight", [d, H * hd]))
            _copy(blk.ffn_norm.gamma, t.take(f"{p}.post_attention_layernorm.weight", [d]))
            g = t.take(f"{p}.mlp.gate_proj.weight", [F_, d])
            u = t.take(f"{p}.mlp.up_proj.weight", [F_, d])
            _copy(blk.ffn.w_gate_up, torch.cat([g.float(), u.float()], 0))
            _copy(blk.ffn.down.weight, t.take(f"{p}.mlp.down_proj.weight", [d, F_]))
        _copy(model.final_norm.gamma, t.take("model.norm.weight", [d]))
        if model.untied_head is not None:
            if t.has("lm_head.weight"):
                _copy(model.untied_head.weight, t.take("lm_head.weight", [c.vocab_size, d]))
            else:
                _copy(model.untied_head.weight, state["model.embed_tokens.weight"])
        rep = t.report()
        rep.unused_keys = [k for k in rep.unused_keys if not k.endswith("rotary_emb.inv_freq")
                           and not (k == "lm_head.weight" and model.untied_head is None)]
        return rep

    @staticmethod
    def dump(model: Llama) -> Dict[str, torch.Tensor]:
        c = model.config
        H, Hkv, hd, F_ = c.num_heads, c.num_kv_heads, c.head_dim, c.ffn_dim
        f32 = lambda x: x.detach().float().cpu().contiguous()  # noqa: E731
        out = {"model.embed_tokens.weight": f32(model.embed_in.weight)}
        for i, blk in enumerate(model.blocks):
            p = f"model.layers.{i}"
            w = f32(blk.attn.w_qkv)
            gu = f32(blk.ffn.w_gate_up)
            out.update({f"{p}.input_layernorm.weight": f32(blk.attn_norm.gamma),
                        f"{p}.self_attn.q_proj.weight": w[:H * hd].contiguous(),
                        f"{p}.self_attn.k_proj.weight": w[H * hd:(H + Hkv) * hd].contiguous(),
                        f"{p}.self_attn.v_proj.weight": w[(H + Hkv) * hd:].contiguous(),
                        f"{p}.self_attn.o_proj.weight": f32(blk.attn.wo.weight),
                        f"{p}.post_attention_layernorm.weight": f32(blk.ffn_norm.gamma),
                        f"{p}.mlp.gate_proj.weight": gu[:F_].contiguous(), f"{p}.mlp.up_proj.weight": gu[F_:].contiguous(),
                        f"{p}.mlp.down_proj.weight": f32(blk.ffn.down.weight)})
        out["model.norm.weight"] = f32(model.final_norm.gamma)
        if model.untied_head is not None:
            out["lm_head.weight"] = f32(model.untied_head.weight)
        return out

    loadFile, loadSharded, loadMap = load_file, load_sharded, load_map
