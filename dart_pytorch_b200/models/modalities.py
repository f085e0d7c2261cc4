"""Text / audio / video encoders and their multimodal combinations
(reference: lib/core/nn/modalities/{text,audio,video}_transformer.dart, multi_modal_classifier.dart:1-81,
multi_modal_encoder.dart:1-99, multi_modal_generator.dart:1-298, multi_modal_lm.dart:1-380).

* ``TextTransformer`` / ``AudioTransformer`` / ``VideoTransformer``: embed or project the input to ``[N, D]``, add a learned
  positional table, run a pre-LN ``TransformerEncoder``; ``pool_mean`` returns the ``[1, D]`` mean row.
* ``MultiModalClassifier`` (late fusion: concatenate pooled features), ``MultiModalEncoder`` (mid fusion: concatenate
  token sequences, run a fusion encoder), ``MultiModalGenerator`` (encoder memory + causal ``TransformerDecoder``),
  ``MultiModalLM`` (one packed causal stream with per-modality type embeddings); greedy ``generate`` on the last two.
"""
from __future__ import annotations

import math
import random as _random
from typing import List, Optional

import torch

from .. import ops as F
from ..nn.layers import Embedding, LearnedPositionalEmbedding, Linear, SinusoidalPositionalEncoding
from ..nn.module import Module, make_param
from ..nn.transformer import TransformerDecoder, TransformerEncoder
from .gpt import _as_token_tensor


def mean_rows(x):
    """``[N, D] -> [1, D]`` as ``(1/N) 1^T x`` (differentiable; reference: audio_transformer.dart:100-112)."""
    if x.dim() != 2:
        raise ValueError(f"meanRows: expected 2D [N, D]; got {list(x.shape)}")
    n = x.shape[0]
    if n == 0:
        raise ValueError("meanRows: cannot pool an empty sequence")
    ones = torch.full((1, n), 1.0 / n, device=x.device, dtype=x.dtype)
    return F.matmul(ones, x)


meanRows = mean_rows


def _argmax_last_row(logits, vocab: int) -> int:
    row = logits.reshape(-1, logits.shape[-1])[-1:, :]
    if row.is_cuda:
        from ..ops import kernels as K
        return int(K.argmax_rows(row.contiguous(), n_cols=vocab).item())
    return int(torch.argmax(row[0, :vocab]).item())


class _SeqEncoder(Module):
    embed_dim: int

    @property
    def embedDim(self):
        return self.embed_dim

    def pool_mean(self, x):
        return mean_rows(self(x))

    poolMean = pool_mean


class TextTransformer(_SeqEncoder):
    def __init__(self, vocab_size: int, max_seq_len: int, embed_dim: int, num_layers: int = 4, num_heads: int = 4,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.max_seq_len, self.embed_dim = vocab_size, max_seq_len, embed_dim
        self.num_layers, self.num_heads = num_layers, num_heads
        self.token_embed = Embedding(vocab_size, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.pos_embed = LearnedPositionalEmbedding(max_seq_len, embed_dim, device=device, seed=seed + 2, dtype=dtype)
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, dropout_p=dropout_p, device=device,
                                          seed=seed + 100, dtype=dtype)

    def submodules(self):
        return [self.token_embed, self.pos_embed, self.encoder]

    def forward(self, tokens):
        tokens = _as_token_tensor(tokens, self.device)
        if tokens.dim() != 1:
            raise ValueError(f"TextTransformer: expected 1D [seqLen]; got {list(tokens.shape)}")
        return self.encoder(self.pos_embed(self.token_embed(tokens)))


class AudioTransformer(_SeqEncoder):
    def __init__(self, feature_dim: int, max_seq_len: int, embed_dim: int, num_layers: int = 4, num_heads: int = 4,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.feature_dim, self.max_seq_len, self.embed_dim = feature_dim, max_seq_len, embed_dim
        self.feature_projection = Linear(feature_dim, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.pos_embed = LearnedPositionalEmbedding(max_seq_len, embed_dim, device=device, seed=seed + 2, dtype=dtype)
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, dropout_p=dropout_p, device=device,
                                          seed=seed + 100, dtype=dtype)

    def submodules(self):
        return [self.feature_projection, self.pos_embed, self.encoder]

    def forward(self, features):
        if features.dim() != 2 or features.shape[1] != self.feature_dim:
            raise ValueError(f"AudioTransformer: expected [seqLen, {self.feature_dim}]; got {list(features.shape)}")
        return self.encoder(self.pos_embed(self.feature_projection(features)))


class VideoTransformer(_SeqEncoder):
    """Per-frame feature vectors -> temporal encoder; the projection is skipped when the widths already match."""

    def __init__(self, frame_feature_dim: int, max_frames: int, embed_dim: int, num_layers: int = 2,
                 num_heads: int = 4, dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.frame_feature_dim, self.max_frames, self.embed_dim = frame_feature_dim, max_frames, embed_dim
        self.frame_projection = None if frame_feature_dim == embed_dim else Linear(
            frame_feature_dim, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.pos_embed = LearnedPositionalEmbedding(max_frames, embed_dim, device=device, seed=seed + 2, dtype=dtype)
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, dropout_p=dropout_p, device=device,
                                          seed=seed + 100, dtype=dtype)

    def submodules(self):
        return ([self.frame_projection] if self.frame_projection is not None else []) + [self.pos_embed, self.encoder]

    def forward(self, frames):
        if frames.dim() != 2 or frames.shape[1] != self.frame_feature_dim:
            raise ValueError(f"VideoTransformer: expected [numFrames, {self.frame_feature_dim}]; "
                             f"got {list(frames.shape)}")
        x = frames if self.frame_projection is None else self.frame_projection(frames)
        return self.encoder(self.pos_embed(x))


def _check_pair(owner: str, name: str, enc, inp):
    if (enc is None) != (inp is None):
        raise ValueError(f"{owner}: {name} encoder present={enc is not None} but {name} input present={inp is not None}")


class MultiModalClassifier(Module):
    """Late fusion: ``head(concat(pool(audio), pool(video)[, pool(text)]))``."""

    def __init__(self, audio: AudioTransformer, video: VideoTransformer, num_classes: int,
                 text: Optional[TextTransformer] = None, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.audio, self.video, self.text, self.num_classes = audio, video, text, num_classes
        width = audio.embed_dim + video.embed_dim + (text.embed_dim if text is not None else 0)
        self.head = Linear(width, num_classes, device=device, seed=seed, dtype=dtype)

    def submodules(self):
        return [self.audio, self.video] + ([self.text] if self.text is not None else []) + [self.head]

    def forward(self, audio_in, video_in, text_in=None):
        _check_pair("MultiModalClassifier", "text", self.text, text_in)
        feats = [self.audio.pool_mean(audio_in), self.video.pool_mean(video_in)]
        if text_in is not None:
            feats.append(self.text.pool_mean(text_in))
        return self.head(F.concat(feats, axis=1))


class MultiModalEncoder(Module):
    """Mid fusion: token sequences of every modality concatenated along time, then a fusion encoder."""

    def __init__(self, audio: AudioTransformer, video: VideoTransformer, joint_embed_dim: int,
                 text: Optional[TextTransformer] = None, fusion_layers: int = 2, fusion_heads: int = 4,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        for m in (audio, video, text):
            if m is not None and m.embed_dim != joint_embed_dim:
                raise ValueError(f"MultiModalEncoder: all unimodal encoders must share jointEmbedDim={joint_embed_dim}")
        self.audio, self.video, self.text, self.joint_embed_dim = audio, video, text, joint_embed_dim
        self.fusion = TransformerEncoder(fusion_layers, joint_embed_dim, fusion_heads, dropout_p=dropout_p,
                                         device=device, seed=seed, dtype=dtype)

    def submodules(self):
        return [self.audio, self.video] + ([self.text] if self.text is not None else []) + [self.fusion]

    def forward(self, audio_in, video_in, text_in=None):
        _check_pair("MultiModalEncoder", "text", self.text, text_in)
        parts = [self.audio(audio_in), self.video(video_in)]
        if text_in is not None:
            parts.append(self.text(text_in))
        return self.fusion(F.concat(parts, axis=0))


class MultiModalGenerator(Module):
    """Any subset of {image, audio, video, text} encoders -> (optional fusion) memory -> causal decoder with
    cross-attention -> token logits; greedy ``generate`` re-decodes the growing target each step."""

    def __init__(self, target_vocab_size: int, max_target_len: int, joint_embed_dim: int, image=None, audio=None,
                 video=None, text=None, decoder_layers: int = 2, decoder_heads: int = 4,
                 decoder_ffn_dim: Optional[int] = None, fusion_layers: int = 1, fusion_heads: int = 4,
                 use_fusion: bool = True, dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        if image is None and audio is None and video is None and text is None:
            raise ValueError("MultiModalGenerator: at least one modality encoder must be provided")
        for name, m in (("image", image), ("audio", audio), ("video", video), ("text", text)):
            if m is not None and m.embed_dim != joint_embed_dim:
                raise ValueError(f"MultiModalGenerator: {name} encoder embedDim must equal "
                                 f"jointEmbedDim={joint_embed_dim}")
        self.image, self.audio, self.video, self.text = image, audio, video, text
        self.joint_embed_dim, self.target_vocab_size, self.max_target_len = (joint_embed_dim, target_vocab_size,
                                                                             max_target_len)
        self.fusion = TransformerEncoder(fusion_layers, joint_embed_dim, fusion_heads, dropout_p=dropout_p,
                                         device=device, seed=seed + 200000, dtype=dtype) if use_fusion else None
        self.target_emb = Embedding(target_vocab_size, joint_embed_dim, device=device, seed=seed + 300000, dtype=dtype)
        self.tgt_pos_enc = SinusoidalPositionalEncoding(joint_embed_dim)
        self.decoder = TransformerDecoder(decoder_layers, joint_embed_dim, decoder_heads, ffn_dim=decoder_ffn_dim,
                                          dropout_p=dropout_p, memory_dim=joint_embed_dim, device=device,
                                          seed=seed + 400000, dtype=dtype)
        self.head = Linear(joint_embed_dim, target_vocab_size, device=device, seed=seed + 500000, dtype=dtype)

    def submodules(self):
        mods = [m for m in (self.image, self.audio, self.video, self.text) if m is not None]
        if self.fusion is not None:
            mods.append(self.fusion)
        return mods + [self.target_emb, self.decoder, self.head]

    def encode(self, image_patches=None, audio_features=None, video_frames=None, text_in=None):
        for name, enc, inp in (("image", self.image, image_patches), ("audio", self.audio, audio_features),
                               ("video", self.video, video_frames), ("text", self.text, text_in)):
            _check_pair("MultiModalGenerator", name, enc, inp)
        parts = []
        if image_patches is not None:
            parts.append(self.image(image_patches))
        if audio_features is not None:
            parts.append(self.audio(audio_features))
        if video_frames is not None:
            parts.append(self.video(video_frames))
        if text_in is not None:
            parts.append(self.text(text_in))
        if not parts:
            raise ValueError("MultiModalGenerator.encode: no modality inputs were provided")
        joint = parts[0] if len(parts) == 1 else F.concat(parts, axis=0)
        return self.fusion(joint) if self.fusion is not None else joint

    def decode(self, target_tokens, memory):
        target_tokens = _as_token_tensor(target_tokens, self.device)
        if target_tokens.dim() != 1:
            raise ValueError(f"MultiModalGenerator.decode: targetTokens must be 1D [seqTgt]; "
                             f"got {list(target_tokens.shape)}")
        n = target_tokens.shape[-1]
        if n > self.max_target_len:
            raise ValueError(f"MultiModalGenerator.decode: seqLen {n} exceeds maxTargetLen {self.max_target_len}")
        y = self.tgt_pos_enc(self.target_emb(target_tokens))
        return self.head(self.decoder(y, memory, causal=True))

    def forward(self, target_tokens, image_patches=None, audio_features=None, video_frames=None, text_in=None):
        return self.decode(target_tokens, self.encode(image_patches, audio_features, video_frames, text_in))

    def generate(self, prompt: List[int], max_new_tokens: int, eos_id: Optional[int] = None, image_patches=None,
                 audio_features=None, video_frames=None, text_in=None) -> List[int]:
        if not prompt:
            raise ValueError("MultiModalGenerator.generate: prompt must have at least one token (typically a BOS)")
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                memory = self.encode(image_patches, audio_features, video_frames, text_in)
                out = [int(t) for t in prompt]
                for _ in range(max_new_tokens):
                    if len(out) >= self.max_target_len:
                        break
                    best = _argmax_last_row(self.decode(out, memory), self.target_vocab_size)
                    out.append(best)
                    if eos_id is not None and best == eos_id:
                        break
                return out
        finally:
            if was_training:
                self.train()


def _type_embedding(embed_dim: int, device, seed: int, dtype, scale: float = 0.02):
    rng = _random.Random(seed)
    vals = []
    for _ in range(embed_dim):
        u1 = min(max(rng.random(), 1e-9), 1.0)
        u2 = rng.random()
        vals.append(math.sqrt(-2.0 * math.log(u1)) * math.cos(2.0 * math.pi * u2) * scale)
    return make_param(torch.tensor(vals, dtype=torch.float32).reshape(1, embed_dim).to(device=device, dtype=dtype))


class MultiModalLM(Module):
    """One causal stream ``[image | audio | video | text prompt | target]``: continuous inputs are projected, every
    segment gets a learned type embedding, positions are sinusoidal over the packed stream, logits are returned for
    the target segment only."""

    def __init__(self, vocab_size: int, embed_dim: int, max_total_seq_len: int, image_patch_pixels: Optional[int] = None,
                 audio_feature_dim: Optional[int] = None, video_frame_feature_dim: Optional[int] = None,
                 use_text_prompt: bool = True, num_layers: int = 4, num_heads: int = 4, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.embed_dim, self.max_total_seq_len = vocab_size, embed_dim, max_total_seq_len
        self.image_patch_pixels, self.audio_feature_dim = image_patch_pixels, audio_feature_dim
        self.video_frame_feature_dim, self.use_text_prompt = video_frame_feature_dim, use_text_prompt

        def proj(width, s):
            return None if width is None else Linear(width, embed_dim, device=device, seed=seed + s, dtype=dtype)

        def typ(enabled, s):
            return _type_embedding(embed_dim, device, seed + s, dtype) if enabled else None
        self.image_proj, self.audio_proj, self.video_proj = (proj(image_patch_pixels, 1), proj(audio_feature_dim, 2),
                                                             proj(video_frame_feature_dim, 3))
        self.token_embed = Embedding(vocab_size, embed_dim, device=device, seed=seed + 4, dtype=dtype)
        self.image_type_emb = typ(image_patch_pixels is not None, 11)
        self.audio_type_emb = typ(audio_feature_dim is not None, 12)
        self.video_type_emb = typ(video_frame_feature_dim is not None, 13)
        self.text_prompt_type_emb = typ(use_text_prompt, 14)
        self.target_type_emb = typ(True, 15)
        self.pos_enc = SinusoidalPositionalEncoding(embed_dim)
        self.decoder = TransformerEncoder(num_layers, embed_dim, num_heads, ffn_dim=ffn_dim, dropout_p=dropout_p,
                                          device=device, seed=seed + 100000, dtype=dtype)
        self.head = Linear(embed_dim, vocab_size, device=device, seed=seed + 200000, dtype=dtype)

    def submodules(self):
        mods = [m for m in (self.image_proj, self.audio_proj, self.video_proj) if m is not None]
        return mods + [self.token_embed, self.decoder, self.head]

    def _walk_params(self, reference: bool):
        # order: projections, token embedding, type embeddings (image, audio, video, prompt, target), decoder, head
        for m in (self.image_proj, self.audio_proj, self.video_proj):
            if m is not None:
                yield from m._walk_params(reference)
        yield from self.token_embed._walk_params(reference)
        for t in (self.image_type_emb, self.audio_type_emb, self.video_type_emb, self.text_prompt_type_emb,
                  self.target_type_emb):
            if t is not None:
                yield t.data if reference else t
        yield from self.decoder._walk_params(reference)
        yield from self.head._walk_params(reference)

    def forward_all(self, target_input_tokens, image_patches=None, audio_features=None, video_frames=None,
                    text_prompt=None):
        for name, dim, inp in (("image", self.image_patch_pixels, image_patches),
                               ("audio", self.audio_feature_dim, audio_features),
                               ("video", self.video_frame_feature_dim, video_frames)):
            if (dim is None) != (inp is None):
                raise ValueError(f"MultiModalLM: {name} enabled={dim is not None} but {name} input "
                                 f"present={inp is not None}")
        if self.use_text_prompt and text_prompt is None:
            raise ValueError("MultiModalLM: useTextPrompt=true but textPrompt input is null")
        if not self.use_text_prompt and text_prompt is not None:
            raise ValueError("MultiModalLM: useTextPrompt=false but textPrompt input was given")
        parts = []
        for inp, prj, typ in ((image_patches, self.image_proj, self.image_type_emb),
                              (audio_features, self.audio_proj, self.audio_type_emb),
                              (video_frames, self.video_proj, self.video_type_emb)):
            if inp is not None:
                parts.append(F.add(prj(inp), typ.reshape(-1)))
        if text_prompt is not None:
            parts.append(F.add(self.token_embed(_as_token_tensor(text_prompt, self.device)),
                               self.text_prompt_type_emb.reshape(-1)))
        tgt_tokens = _as_token_tensor(target_input_tokens, self.device)
        parts.append(F.add(self.token_embed(tgt_tokens), self.target_type_emb.reshape(-1)))
        x = parts[0] if len(parts) == 1 else F.concat(parts, axis=0)
        total = x.shape[0]
        if total > self.max_total_seq_len:
            raise ValueError(f"MultiModalLM.forwardAll: total sequence length {total} exceeds maxTotalSeqLen "
                             f"{self.max_total_seq_len}")
        logits = self.head(self.decoder(self.pos_enc(x), causal=True))
        return logits, total - tgt_tokens.shape[0], total

    forwardAll = forward_all

    def forward(self, target_input_tokens, image_patches=None, audio_features=None, video_frames=None,
                text_prompt=None):
        logits, start, _ = self.forward_all(target_input_tokens, image_patches, audio_features, video_frames,
                                            text_prompt)
        return logits if start == 0 else logits[start:]

    def generate(self, prompt: List[int], max_new_tokens: int, eos_id: Optional[int] = None, image_patches=None,
                 audio_features=None, video_frames=None, text_prompt=None) -> List[int]:
        if not prompt:
            raise ValueError("MultiModalLM.generate: prompt must have at least one token (typically a BOS)")
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                out = [int(t) for t in prompt]
                for _ in range(max_new_tokens):
                    logits = self.forward(out, image_patches, audio_features, video_frames, text_prompt)
                    best = _argmax_last_row(logits, self.vocab_size)
                    out.append(best)
                    if eos_id is not None and best == eos_id:
                        break
                return out
        finally:
            if was_training:
                self.train()
