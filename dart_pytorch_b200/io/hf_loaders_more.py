"""HuggingFace weight loaders for Pythia (GPT-NeoX), GPT-J, BERT / MiniLM and the CLIP vision tower
(reference: lib/core/nn/pythia_hf_loader.dart:1-402, gptj_hf_loader.dart:1-387, bert_hf_loader.dart:1-355,
clip_hf_loader.dart:1-472).

All take a ``{name: tensor}`` state dict, check every shape, copy in place and return a ``LoadReport``; a missing or
mis-shaped tensor raises.  Layout conversions:

* Pythia ``query_key_value`` rows are ``[heads, 3, head_dim]``-interleaved; they are regrouped into the fused
  ``[q heads | k heads | v heads]`` projection.
* GPT-J rotates *interleaved* pairs; the rows of the first ``rotary_dim`` outputs of every q / k head are permuted
  ``2i -> i, 2i+1 -> i + rotary_dim/2`` so the half-split rotary used here produces the same scores.
* BERT ``query / key / value`` concatenate into the fused projection; the token-type table collapses to its row 0.
* CLIP's patch ``Conv2d`` weight ``[D, C, P, P]`` is permuted to ``[D, P*P*C]`` (``(dy, dx, c)`` per patch).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..models.bert import BertConfig, BertModel
from ..models.neox import GPTJConfig, GPTJModel, PythiaConfig, PythiaModel
from ..models.vision_language import CLIPVisionConfig, CLIPVisionModel
from .hf_loaders import LoadReport, _copy, _Taker
from .safetensors import SafeTensors


def _strip_prefix(state: Dict[str, torch.Tensor], prefix: str, keep=()):
    if any(k.startswith(prefix) for k in state):
        return {(k[len(prefix):] if k.startswith(prefix) else k): v for k, v in state.items()}
    return state


class _FileEntry:
    """``load_file`` / ``load_sharded`` on top of a ``load_map``."""

    @classmethod
    def load_file(cls, model, path: str, keep_fp16: bool = False) -> LoadReport:
        return cls.load_map(model, SafeTensors.load_file(path, keep_fp16=keep_fp16))

    @classmethod
    def load_sharded(cls, model, index_path: str, keep_fp16: bool = False) -> LoadReport:
        return cls.load_map(model, SafeTensors.load_sharded(index_path, keep_fp16=keep_fp16))

    loadFile, loadSharded = load_file, load_sharded


# ------------------------------------------------------------------------------------------------- Pythia ----
class PythiaHFLoader(_FileEntry):
    @staticmethod
    def _cfg(embed, layers, heads, **kw) -> PythiaConfig:
        return PythiaConfig(vocab_size=50304, max_ctx=2048, embed_dim=embed, num_layers=layers, num_heads=heads, **kw)

    @staticmethod
    def pythia_14m_config(**kw): return PythiaHFLoader._cfg(128, 6, 8, **kw)
    @staticmethod
    def pythia_70m_config(**kw): return PythiaHFLoader._cfg(512, 6, 8, **kw)
    @staticmethod
    def pythia_160m_config(**kw): return PythiaHFLoader._cfg(768, 12, 12, **kw)
    @staticmethod
    def pythia_410m_config(**kw): return PythiaHFLoader._cfg(1024, 24, 16, **kw)
    @staticmethod
    def pythia_1b_config(**kw): return PythiaHFLoader._cfg(2048, 16, 8, **kw)

    pythia14mConfig, pythia70mConfig, pythia160mConfig = pythia_14m_config, pythia_70m_config, pythia_160m_config
    pythia410mConfig, pythia1bConfig = pythia_410m_config, pythia_1b_config

    @staticmethod
    def _deinterleave(t: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
        """``[heads, 3, hd, ...] -> [3, heads, hd, ...]`` flattened back to rows."""
        rest = t.shape[1:]
        return t.reshape(heads, 3, hd, *rest).transpose(0, 1).reshape(3 * heads * hd, *rest)

    @staticmethod
    def _interleave(t: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
        rest = t.shape[1:]
        return t.reshape(3, heads, hd, *rest).transpose(0, 1).reshape(3 * heads * hd, *rest)

    @classmethod
    def load_map(cls, model: PythiaModel, state_in: Dict[str, torch.Tensor]) -> LoadReport:
        state = _strip_prefix(state_in, "gpt_neox.")
        t = _Taker(state, "pythia")
        c = model.config
        d, f, H = c.embed_dim, c.ffn_dim, c.num_heads
        hd = d // H
        _copy(model.embed_in.weight, t.take("embed_in.weight", [c.vocab_size, d]))
        for i, blk in enumerate(model.blocks):
            p = f"layers.{i}"
            for ln, name in ((blk.input_ln, "input_layernorm"), (blk.post_attn_ln, "post_attention_layernorm")):
                _copy(ln.gamma, t.take(f"{p}.{name}.weight", [d]))
                _copy(ln.beta, t.take(f"{p}.{name}.bias", [d]))
            _copy(blk.attn.w_qkv, cls._deinterleave(t.take(f"{p}.attention.query_key_value.weight", [3 * d, d]).float(),
                                                    H, hd))
            _copy(blk.attn.b_qkv, cls._deinterleave(t.take(f"{p}.attention.query_key_value.bias", [3 * d]).float(),
                                                    H, hd))
            _copy(blk.attn.wo.weight, t.take(f"{p}.attention.dense.weight", [d, d]))
            _copy(blk.attn.wo.bias, t.take(f"{p}.attention.dense.bias", [d]))
            _copy(blk.ffn1.weight, t.take(f"{p}.mlp.dense_h_to_4h.weight", [f, d]))
            _copy(blk.ffn1.bias, t.take(f"{p}.mlp.dense_h_to_4h.bias", [f]))
            _copy(blk.ffn2.weight, t.take(f"{p}.mlp.dense_4h_to_h.weight", [d, f]))
            _copy(blk.ffn2.bias, t.take(f"{p}.mlp.dense_4h_to_h.bias", [d]))
        _copy(model.final_ln.gamma, t.take("final_layer_norm.weight", [d]))
        _copy(model.final_ln.beta, t.take("final_layer_norm.bias", [d]))
        _copy(model.embed_out.weight, t.take("embed_out.weight", [c.vocab_size, d]))
        return t.report()

    loadMap = load_map

    @classmethod
    def dump(cls, model: PythiaModel) -> Dict[str, torch.Tensor]:
        c = model.config
        H, hd = c.num_heads, c.embed_dim // c.num_heads
        f32 = lambda x: x.detach().float().cpu().contiguous()  # noqa: E731
        out = {"gpt_neox.embed_in.weight": f32(model.embed_in.weight), "embed_out.weight": f32(model.embed_out.weight),
               "gpt_neox.final_layer_norm.weight": f32(model.final_ln.gamma),
               "gpt_neox.final_layer_norm.bias": f32(model.final_ln.beta)}
        for i, blk in enumerate(model.blocks):
            p = f"gpt_neox.layers.{i}"
            out.update({
                f"{p}.input_layernorm.weight": f32(blk.input_ln.gamma), f"{p}.input_layernorm.bias": f32(blk.input_ln.beta),
                f"{p}.post_attention_layernorm.weight": f32(blk.post_attn_ln.gamma),
                f"{p}.post_attention_layernorm.bias": f32(blk.post_attn_ln.beta),
                f"{p}.attention.query_key_value.weight": f32(cls._interleave(f32(blk.attn.w_qkv), H, hd)),
                f"{p}.attention.query_key_value.bias": f32(cls._interleave(f32(blk.attn.b_qkv), H, hd)),
                f"{p}.attention.dense.weight": f32(blk.attn.wo.weight), f"{p}.attention.dense.bias": f32(blk.attn.wo.bias),
                f"{p}.mlp.dense_h_to_4h.weight": f32(blk.ffn1.weight), f"{p}.mlp.dense_h_to_4h.bias": f32(blk.ffn1.bias),
                f"{p}.mlp.dense_4h_to_h.weight": f32(blk.ffn2.weight), f"{p}.mlp.dense_4h_to_h.bias": f32(blk.ffn2.bias)})
        return out


# -------------------------------------------------------------------------------------------------- GPT-J ----
class GPTJHFLoader(_FileEntry):
    @staticmethod
    def gpt_j_6b_config(device=None, seed: int = 0, **kw) -> GPTJConfig:
        return GPTJConfig(vocab_size=50400, max_ctx=2048, embed_dim=4096, num_layers=28, num_heads=16, rotary_dim=64,
                          device=device, seed=seed, **kw)

    @staticmethod
    def gpt_j_6b_hybrid_config(gpu_layers: int, embed_on_gpu: bool = False, lm_head_on_gpu: bool = False,
                               seed: int = 0, gpu="cuda", cpu="cpu", **kw) -> GPTJConfig:
        """First ``gpu_layers`` blocks on the GPU, the rest (and by default the embedding / head) on the CPU."""
        n = 28
        if not (0 <= gpu_layers <= n):
            raise ValueError(f"gptJ6bHybridConfig: gpuLayers ({gpu_layers}) must be in [0, {n}]")
        return GPTJConfig(vocab_size=50400, max_ctx=2048, embed_dim=4096, num_layers=n, num_heads=16, rotary_dim=64,
                          device=cpu, layer_devices=[gpu if i < gpu_layers else cpu for i in range(n)],
                          embedding_device=gpu if embed_on_gpu else cpu,
                          lm_head_device=gpu if lm_head_on_gpu else cpu, seed=seed, **kw)

    gptJ6bConfig, gptJ6bHybridConfig = gpt_j_6b_config, gpt_j_6b_hybrid_config

    @staticmethod
    def rotary_row_permutation(head_dim: int, rotary_dim: int, inverse: bool = False) -> torch.Tensor:
        """Index ``idx`` with ``out[r] = src[idx[r]]``: ``out[i] = src[2i]``, ``out[i + R/2] = src[2i + 1]`` for the first
        ``R = rotary_dim`` rows of a head, identity above."""
        if rotary_dim <= 0 or rotary_dim > head_dim or rotary_dim % 2:
            raise ValueError(f"_permuteRotaryRows: rDim={rotary_dim} invalid for headDim={head_dim}")
        half = rotary_dim // 2
        idx = torch.arange(head_dim)
        idx[:half] = torch.arange(0, rotary_dim, 2)
        idx[half:rotary_dim] = torch.arange(1, rotary_dim, 2)
        if inverse:
            inv = torch.empty_like(idx)
            inv[idx] = torch.arange(head_dim)
            return inv
        return idx

    @classmethod
    def _permute_heads(cls, w: torch.Tensor, heads: int, hd: int, rdim: int, inverse: bool = False) -> torch.Tensor:
        idx = cls.rotary_row_permutation(hd, rdim, inverse)
        return w.reshape(heads, hd, -1)[:, idx, :].reshape(heads * hd, -1)

    @classmethod
    def load_map(cls, model: GPTJModel, state_in: Dict[str, torch.Tensor]) -> LoadReport:
        state = _strip_prefix(state_in, "transformer.")
        t = _Taker(state, "gpt-j")
        c = model.config
        d, f, H = c.embed_dim, c.ffn_dim, c.num_heads
        hd = d // H
        _copy(model.wte.weight, t.take("wte.weight", [c.vocab_size, d]))
        for i, blk in enumerate(model.blocks):
            p = f"h.{i}"
            _copy(blk.ln.gamma, t.take(f"{p}.ln_1.weight", [d]))
            _copy(blk.ln.beta, t.take(f"{p}.ln_1.bias", [d]))
            q = cls._permute_heads(t.take(f"{p}.attn.q_proj.weight", [d, d]).float(), H, hd, c.rotary_dim)
            k = cls._permute_heads(t.take(f"{p}.attn.k_proj.weight", [d, d]).float(), H, hd, c.rotary_dim)
            v = t.take(f"{p}.attn.v_proj.weight", [d, d]).float()
            _copy(blk.attn.w_qkv, torch.cat([q, k, v], 0))
            _copy(blk.attn.wo.weight, t.take(f"{p}.attn.out_proj.weight", [d, d]))
            _copy(blk.ffn1.weight, t.take(f"{p}.mlp.fc_in.weight", [f, d]))
            _copy(blk.ffn1.bias, t.take(f"{p}.mlp.fc_in.bias", [f]))
            _copy(blk.ffn2.weight, t.take(f"{p}.mlp.fc_out.weight", [d, f]))
            _copy(blk.ffn2.bias, t.take(f"{p}.mlp.fc_out.bias", [d]))
        _copy(model.final_ln.gamma, t.take("ln_f.weight", [d]))
        _copy(model.final_ln.beta, t.take("ln_f.bias", [d]))
        _copy(model.lm_head.weight, t.take("lm_head.weight", [c.vocab_size, d]))
        _copy(model.lm_head.bias, t.take("lm_head.bias", [c.vocab_size]))
        return t.report()

    loadMap = load_map

    @classmethod
    def dump(cls, model: GPTJModel) -> Dict[str, torch.Tensor]:
        c = model.config
        d, H = c.embed_dim, c.num_heads
        hd = d // H
        f32 = lambda x: x.detach().float().cpu().contiguous()  # noqa: E731
        out = {"transformer.wte.weight": f32(model.wte.weight), "transformer.ln_f.weight": f32(model.final_ln.gamma),
               "transformer.ln_f.bias": f32(model.final_ln.beta), "lm_head.weight": f32(model.lm_head.weight),
               "lm_head.bias": f32(model.lm_head.bias)}
        for i, blk in enumerate(model.blocks):
            p = f"transformer.h.{i}"
            w = f32(blk.attn.w_qkv)
            out.update({
                f"{p}.ln_1.weight": f32(blk.ln.gamma), f"{p}.ln_1.bias": f32(blk.ln.beta),
                f"{p}.attn.q_proj.weight": cls._permute_heads(w[:d], H, hd, c.rotary_dim, inverse=True).contiguous(),
                f"{p}.attn.k_proj.weight": cls._permute_heads(w[d:2 * d], H, hd, c.rotary_dim, inverse=True).contiguous(),
                f"{p}.attn.v_proj.weight": w[2 * d:].contiguous(),
                f"{p}.attn.out_proj.weight": f32(blk.attn.wo.weight),
                f"{p}.mlp.fc_in.weight": f32(blk.ffn1.weight), f"{p}.mlp.fc_in.bias": f32(blk.ffn1.bias),
                f"{p}.mlp.fc_out.weight": f32(blk.ffn2.weight), f"{p}.mlp.fc_out.bias": f32(blk.ffn2.bias)})
        return out


# --------------------------------------------------------------------------------------------------- BERT ----
class BertHFLoader(_FileEntry):
    @staticmethod
    def mini_lm_l6_v2_config(**kw) -> BertConfig:
        return BertConfig(vocab_size=30522, max_position_embeddings=512, embed_dim=384, num_layers=6, num_heads=12,
                          intermediate_size=1536, **kw)

    @staticmethod
    def bert_base_uncased_config(**kw) -> BertConfig:
        return BertConfig(vocab_size=30522, max_position_embeddings=512, embed_dim=768, num_layers=12, num_heads=12,
                          intermediate_size=3072, **kw)

    miniLmL6V2Config, bertBaseUncasedConfig = mini_lm_l6_v2_config, bert_base_uncased_config

    @classmethod
    def load_map(cls, model: BertModel, state_in: Dict[str, torch.Tensor]) -> LoadReport:
        state = _strip_prefix(state_in, "bert.")
        t = _Taker(state, "bert")
        c = model.config
        d, f = c.embed_dim, c.intermediate_size
        e = model.embeddings
        _copy(e.word_embeddings.weight, t.take("embeddings.word_embeddings.weight", [c.vocab_size, d]))
        _copy(e.position_embeddings.weight, t.take("embeddings.position_embeddings.weight",
                                                   [c.max_position_embeddings, d]))
        tt = t.state.get("embeddings.token_type_embeddings.weight")
        if tt is None or tt.dim() != 2 or tt.shape[1] != d:
            raise ValueError('bert loader: missing or mis-shaped "embeddings.token_type_embeddings.weight"')
        t.consumed.add("embeddings.token_type_embeddings.weight")
        _copy(e.token_type_bias, tt[0:1])
        _copy(e.layer_norm.gamma, t.take("embeddings.LayerNorm.weight", [d]))
        _copy(e.layer_norm.beta, t.take("embeddings.LayerNorm.bias", [d]))
        for i, layer in enumerate(model.layers):
            p = f"encoder.layer.{i}"
            ws = [t.take(f"{p}.attention.self.{n}.weight", [d, d]).float() for n in ("query", "key", "value")]
            bs = [t.take(f"{p}.attention.self.{n}.bias", [d]).float() for n in ("query", "key", "value")]
            _copy(layer.attention.w_qkv, torch.cat(ws, 0))
            _copy(layer.attention.b_qkv, torch.cat(bs, 0))
            _copy(layer.attention.wo.weight, t.take(f"{p}.attention.output.dense.weight", [d, d]))
            _copy(layer.attention.wo.bias, t.take(f"{p}.attention.output.dense.bias", [d]))
            _copy(layer.attention_output_ln.gamma, t.take(f"{p}.attention.output.LayerNorm.weight", [d]))
            _copy(layer.attention_output_ln.beta, t.take(f"{p}.attention.output.LayerNorm.bias", [d]))
            _copy(layer.intermediate.weight, t.take(f"{p}.intermediate.dense.weight", [f, d]))
            _copy(layer.intermediate.bias, t.take(f"{p}.intermediate.dense.bias", [f]))
            _copy(layer.output.weight, t.take(f"{p}.output.dense.weight", [d, f]))
            _copy(layer.output.bias, t.take(f"{p}.output.dense.bias", [d]))
            _copy(layer.output_ln.gamma, t.take(f"{p}.output.LayerNorm.weight", [d]))
            _copy(layer.output_ln.beta, t.take(f"{p}.output.LayerNorm.bias", [d]))
        return t.report()

    loadMap = load_map

    @classmethod
    def dump(cls, model: BertModel, type_vocab: int = 2) -> Dict[str, torch.Tensor]:
        d = model.config.embed_dim
        f32 = lambda x: x.detach().float().cpu().contiguous()  # noqa: E731
        e = model.embeddings
        tt = torch.zeros(type_vocab, d)
        tt[0] = f32(e.token_type_bias)[0]
        out = {"embeddings.word_embeddings.weight": f32(e.word_embeddings.weight),
               "embeddings.position_embeddings.weight": f32(e.position_embeddings.weight),
               "embeddings.token_type_embeddings.weight": tt,
               "embeddings.LayerNorm.weight": f32(e.layer_norm.gamma), "embeddings.LayerNorm.bias": f32(e.layer_norm.beta)}
        for i, layer in enumerate(model.layers):
            p = f"encoder.layer.{i}"
            w, b = f32(layer.attention.w_qkv), f32(layer.attention.b_qkv)
            for j, n in enumerate(("query", "key", "value")):
                out[f"{p}.attention.self.{n}.weight"] = w[j * d:(j + 1) * d].contiguous()
                out[f"{p}.attention.self.{n}.bias"] = b[j * d:(j + 1) * d].contiguous()
            out.update({
                f"{p}.attention.output.dense.weight": f32(layer.attention.wo.weight),
                f"{p}.attention.output.dense.bias": f32(layer.attention.wo.bias),
                f"{p}.attention.output.LayerNorm.weight": f32(layer.attention_output_ln.gamma),
                f"{p}.attention.output.LayerNorm.bias": f32(layer.attention_output_ln.beta),
                f"{p}.intermediate.dense.weight": f32(layer.intermediate.weight),
                f"{p}.intermediate.dense.bias": f32(layer.intermediate.bias),
                f"{p}.output.dense.weight": f32(layer.output.weight), f"{p}.output.dense.bias": f32(layer.output.bias),
                f"{p}.output.LayerNorm.weight": f32(layer.output_ln.gamma),
                f"{p}.output.LayerNorm.bias": f32(layer.output_ln.beta)})
        return out


# --------------------------------------------------------------------------------------------------- CLIP ----
class ClipHFLoader(_FileEntry):
    @staticmethod
    def base32_config(**kw) -> CLIPVisionConfig:
        return CLIPVisionConfig(image_size=224, patch_size=32, embed_dim=768, num_layers=12, num_heads=12,
                                ffn_dim=3072, **kw)

    @staticmethod
    def base16_config(**kw) -> CLIPVisionConfig:
        return CLIPVisionConfig(image_size=224, patch_size=16, embed_dim=768, num_layers=12, num_heads=12,
                                ffn_dim=3072, **kw)

    @staticmethod
    def large14_config(**kw) -> CLIPVisionConfig:
        return CLIPVisionConfig(image_size=224, patch_size=14, embed_dim=1024, num_layers=24, num_heads=16,
                                ffn_dim=4096, **kw)

    base32Config, base16Config, large14Config = base32_config, base16_config, large14_config

    @staticmethod
    def conv_to_linear(conv: torch.Tensor) -> torch.Tensor:
        """``[D, C, P, P] -> [D, P*P*C]`` with per-patch order ``(dy, dx, c)``."""
        return conv.permute(0, 2, 3, 1).reshape(conv.shape[0], -1).contiguous()

    @classmethod
    def load_map(cls, model: CLIPVisionModel, state_in: Dict[str, torch.Tensor]) -> LoadReport:
        # full CLIPModel bundles prefix every vision tensor with "vision_model."; standalone vision checkpoints and
        # some re-exports carry bare names (reference: lib/core/nn/clip_hf_loader.dart:343-355)
        candidates = ("vision_model.", "")
        prefix = next((p for p in candidates if p + "embeddings.patch_embedding.weight" in state_in), None)
        if prefix is None:
            raise ValueError('clip loader: cannot find "embeddings.patch_embedding.weight" in the state dict (checked '
                             f'prefixes {list(candidates)}); is this a CLIP vision checkpoint?')
        t = _Taker(state_in, "clip")
        c = model.config
        d, f, P, C = c.embed_dim, c.ffn_dim, c.patch_size, c.num_channels
        conv = t.take(prefix + "embeddings.patch_embedding.weight", [d, C, P, P]).float()
        _copy(model.patch_projection.weight, cls.conv_to_linear(conv))
        _copy(model.cls_token, t.take(prefix + "embeddings.class_embedding", [d]).reshape(1, d))
        _copy(model.pos_embeddings, t.take(prefix + "embeddings.position_embedding.weight", [c.num_patches + 1, d]))
        _copy(model.pre_layer_norm.gamma, t.take(prefix + "pre_layrnorm.weight", [d]))
        _copy(model.pre_layer_norm.beta, t.take(prefix + "pre_layrnorm.bias", [d]))
        for i, blk in enumerate(model.encoder.blocks):
            p = f"{prefix}encoder.layers.{i}"
            ws = [t.take(f"{p}.self_attn.{n}_proj.weight", [d, d]).float() for n in "qkv"]
            bs = [t.take(f"{p}.self_attn.{n}_proj.bias", [d]).float() for n in "qkv"]
            _copy(blk.mha.w_qkv, torch.cat(ws, 0))
            _copy(blk.mha.b_qkv, torch.cat(bs, 0))
            _copy(blk.mha.wo.weight, t.take(f"{p}.self_attn.out_proj.weight", [d, d]))
            _copy(blk.mha.wo.bias, t.take(f"{p}.self_attn.out_proj.bias", [d]))
            for ln, name in ((blk.ln1, "layer_norm1"), (blk.ln2, "layer_norm2")):
                _copy(ln.gamma, t.take(f"{p}.{name}.weight", [d]))
                _copy(ln.beta, t.take(f"{p}.{name}.bias", [d]))
            _copy(blk.ffn1.weight, t.take(f"{p}.mlp.fc1.weight", [f, d]))
            _copy(blk.ffn1.bias, t.take(f"{p}.mlp.fc1.bias", [f]))
            _copy(blk.ffn2.weight, t.take(f"{p}.mlp.fc2.weight", [d, f]))
            _copy(blk.ffn2.bias, t.take(f"{p}.mlp.fc2.bias", [d]))
        _copy(model.encoder.final_norm.gamma, t.take(prefix + "post_layernorm.weight", [d]))
        _copy(model.encoder.final_norm.beta, t.take(prefix + "post_layernorm.bias", [d]))
        return t.report()

    loadMap = load_map

    @classmethod
    def dump(cls, model: CLIPVisionModel) -> Dict[str, torch.Tensor]:
        c = model.config
        d, P, C = c.embed_dim, c.patch_size, c.num_channels
        f32 = lambda x: x.detach().float().cpu().contiguous()  # noqa: E731
        pre = "vision_model."
        out = {pre + "embeddings.patch_embedding.weight":
               f32(model.patch_projection.weight).reshape(d, P, P, C).permute(0, 3, 1, 2).contiguous(),
               pre + "embeddings.class_embedding": f32(model.cls_token).reshape(d),
               pre + "embeddings.position_embedding.weight": f32(model.pos_embeddings),
               pre + "pre_layrnorm.weight": f32(model.pre_layer_norm.gamma),
               pre + "pre_layrnorm.bias": f32(model.pre_layer_norm.beta),
               pre + "post_layernorm.weight": f32(model.encoder.final_norm.gamma),
               pre + "post_layernorm.bias": f32(model.encoder.final_norm.beta)}
        for i, blk in enumerate(model.encoder.blocks):
            p = f"{pre}encoder.layers.{i}"
            w, b = f32(blk.mha.w_qkv), f32(blk.mha.b_qkv)
            for j, n in enumerate("qkv"):
                out[f"{p}.self_attn.{n}_proj.weight"] = w[j * d:(j + 1) * d].contiguous()
                out[f"{p}.self_attn.{n}_proj.bias"] = b[j * d:(j + 1) * d].contiguous()
            out.update({f"{p}.self_attn.out_proj.weight": f32(blk.mha.wo.weight),
                        f"{p}.self_attn.out_proj.bias": f32(blk.mha.wo.bias),
                        f"{p}.layer_norm1.weight": f32(blk.ln1.gamma), f"{p}.layer_norm1.bias": f32(blk.ln1.beta),
                        f"{p}.layer_norm2.weight": f32(blk.ln2.gamma), f"{p}.layer_norm2.bias": f32(blk.ln2.beta),
                        f"{p}.mlp.fc1.weight": f32(blk.ffn1.weight), f"{p}.mlp.fc1.bias": f32(blk.ffn1.bias),
                        f"{p}.mlp.fc2.weight": f32(blk.ffn2.weight), f"{p}.mlp.fc2.bias": f32(blk.ffn2.bias)})
        return out
