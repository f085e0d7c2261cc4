"""Smaller sequence models of the reference zoo: ``TransformerLM``, the attention-free ``AFTLanguageModel`` (with its
``AFTAttention`` / ``AFTBlock``) and the ``EncoderDecoderTransformer``
(reference: lib/core/nn/transformer_lm.dart:25-94, aft_transformer.dart:23-159, attention/aft_attention.dart:26-106,
encoder_decoder.dart:32-185)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops as F
from ..nn.layers import Dropout, Embedding, LayerNorm, Linear, SinusoidalPositionalEncoding
from ..nn.module import Module, make_param, uniform_
from ..nn.transformer import TransformerDecoder, TransformerEncoder
from .gpt import _as_token_tensor


class TransformerLM(Module):
    """Token embedding + sinusoidal positions + pre-LN encoder (ReLU FFN) + biased untied head."""

    def __init__(self, vocab_size: int, embed_dim: int, num_layers: int, num_heads: int, max_len: int,
                 ffn_dim: Optional[int] = None, dropout_p: float = 0.0, device=None, seed: int = 0,
                 dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.embed_dim, self.max_len = vocab_size, embed_dim, max_len
        self.token_emb = Embedding(vocab_size, embed_dim, device=device, seed=seed, dtype=dtype)
        self.pos_enc = SinusoidalPositionalEncoding(embed_dim)
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, ffn_dim=ffn_dim, dropout_p=dropout_p,
                                          device=device, seed=seed + 100000, dtype=dtype)
        self.head = Linear(embed_dim, vocab_size, device=device, seed=seed + 900000, dtype=dtype)

    def submodules(self):
        return [self.token_emb, self.encoder, self.head]

    def forward(self, tokens):
        tokens = _as_token_tensor(tokens, self.device)
        if tokens.dim() not in (1, 2):
            raise ValueError("TransformerLM: tokens must be [N] or [B, N]")
        n = tokens.shape[-1]
        if n > self.max_len:
            raise ValueError(f"TransformerLM: seqLen {n} exceeds maxLen {self.max_len}")
        x = self.pos_enc(F.embedding(self.token_emb.weight, tokens))
        return self.head(self.encoder(x, causal=n > 1))

    def loss(self, tokens, targets):
        logits = self.forward(tokens)
        targets = _as_token_tensor(targets, self.device)
        return F.mean(F.cross_entropy(logits.reshape(-1, self.vocab_size), targets.reshape(-1))).reshape(())


class AFTAttention(Module):
    """AFT-full: ``sigmoid(q) * softmax_t'(k + w[t, t']) v`` with a learned pairwise position bias ``[maxSeq, maxSeq]``
    ~ U(+-0.02), sliced to ``[T, T]``."""

    def __init__(self, embed_dim: int, max_seq_len: int, masked: bool = False, bias: bool = False, device=None,
                 seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.embed_dim, self.max_seq_len, self.masked = embed_dim, max_seq_len, masked
        self.wq = Linear(embed_dim, embed_dim, bias=bias, device=device, seed=seed, dtype=dtype)
        self.wk = Linear(embed_dim, embed_dim, bias=bias, device=device, seed=seed + 1000, dtype=dtype)
        self.wv = Linear(embed_dim, embed_dim, bias=bias, device=device, seed=seed + 2000, dtype=dtype)
        self.pos_bias = make_param(uniform_((max_seq_len, max_seq_len), 0.02, seed + 3000, device, dtype))

    def submodules(self):
        return [self.wq, self.wk, self.wv]

    def _walk_params(self, reference: bool):
        for m in (self.wq, self.wk, self.wv):
            yield from m._walk_params(reference)
        yield self.pos_bias.data if reference else self.pos_bias

    def forward(self, x):
        if x.dim() != 2:
            raise ValueError(f"AFTAttention: expected 2D input [T, embedDim]; got {list(x.shape)}")
        if x.shape[1] != self.embed_dim:
            raise ValueError(f"AFTAttention: last dim {x.shape[1]} != embedDim {self.embed_dim}")
        t = x.shape[0]
        if t > self.max_seq_len:
            raise ValueError(f"AFTAttention: seqLen {t} exceeds maxSeqLen {self.max_seq_len}")
        w = self.pos_bias if t == self.max_seq_len else F.slice_top_left(self.pos_bias, t, t)
        return F.aft_full(self.wq(x), self.wk(x), self.wv(x), w, causal=self.masked)


class AFTBlock(Module):
    def __init__(self, embed_dim: int, max_seq_len: int, masked: bool = False, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.ffn_dim = ffn_dim or embed_dim * 4
        self.ln1 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.ln2 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.attn = AFTAttention(embed_dim, max_seq_len, masked=masked, device=device, seed=seed, dtype=dtype)
        self.ffn1 = Linear(embed_dim, self.ffn_dim, device=device, seed=seed + 4000, dtype=dtype)
        self.ffn2 = Linear(self.ffn_dim, embed_dim, device=device, seed=seed + 5000, dtype=dtype)
        self.dropout = Dropout(dropout_p)

    def submodules(self):
        return [self.ln1, self.ln2, self.attn, self.ffn1, self.ffn2, self.dropout]

    def forward(self, x):
        h = F.add(x, self.dropout(self.attn(self.ln1(x))))
        return F.add(h, self.dropout(self.ffn2(self.ffn1(self.ln2(h), activation="relu"))))


class AFTLanguageModel(Module):
    def __init__(self, vocab_size: int, embed_dim: int, num_layers: int, max_len: int, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.vocab_size, self.embed_dim, self.num_layers, self.max_len = vocab_size, embed_dim, num_layers, max_len
        self.token_emb = Embedding(vocab_size, embed_dim, device=device, seed=seed, dtype=dtype)
        self.pos_enc = SinusoidalPositionalEncoding(embed_dim)
        self.blocks: List[AFTBlock] = [
            AFTBlock(embed_dim, max_len, masked=True, ffn_dim=ffn_dim, dropout_p=dropout_p, device=device,
                     seed=seed + 100000 + i * 10000, dtype=dtype) for i in range(num_layers)]
        self.final_ln = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.head = Linear(embed_dim, vocab_size, device=device, seed=seed + 900000, dtype=dtype)

    def submodules(self):
        return [self.token_emb] + list(self.blocks) + [self.final_ln, self.head]

    def forward(self, tokens):
        tokens = _as_token_tensor(tokens, self.device)
        if tokens.dim() != 1:
            raise ValueError(f"AFTLanguageModel: tokens must be 1D [seqLen]; got {list(tokens.shape)}")
        n = tokens.shape[0]
        if n > self.max_len:
            raise ValueError(f"AFTLanguageModel: seqLen {n} exceeds maxLen {self.max_len}")
        x = self.pos_enc(F.embedding(self.token_emb.weight, tokens))
        for b in self.blocks:
            x = b(x)
        return self.head(self.final_ln(x))

    def loss(self, tokens, targets):
        logits = self.forward(tokens)
        targets = _as_token_tensor(targets, self.device)
        return F.mean(F.cross_entropy(logits, targets.reshape(-1))).reshape(())


class EncoderDecoderTransformer(Module):
    """Sequence-to-sequence transformer: source encoder (bidirectional), target decoder (causal self-attention + cross
    attention), biased head over the target vocabulary; ``encode``, ``decode`` and ``call(src, tgt)``."""

    def __init__(self, src_vocab_size: int, tgt_vocab_size: int, embed_dim: int, num_heads: int,
                 num_encoder_layers: int, num_decoder_layers: int, max_len: int, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.max_len, self.tgt_vocab_size = max_len, tgt_vocab_size
        self.src_emb = Embedding(src_vocab_size, embed_dim, device=device, seed=seed, dtype=dtype)
        self.tgt_emb = Embedding(tgt_vocab_size, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.pos_enc = SinusoidalPositionalEncoding(embed_dim)
        self.encoder = TransformerEncoder(num_encoder_layers, embed_dim, num_heads, ffn_dim=ffn_dim,
                                          dropout_p=dropout_p, device=device, seed=seed + 100000, dtype=dtype)
        self.decoder = TransformerDecoder(num_decoder_layers, embed_dim, num_heads, ffn_dim=ffn_dim,
                                          dropout_p=dropout_p, device=device, seed=seed + 500000, dtype=dtype)
        self.head = Linear(embed_dim, tgt_vocab_size, device=device, seed=seed + 900000, dtype=dtype)

    def submodules(self):
        return [self.src_emb, self.tgt_emb, self.encoder, self.decoder, self.head]

    def _check(self, t, what):
        if t.dim() not in (1, 2):
            raise ValueError(f"EncoderDecoderTransformer: {what} tokens must be [N] or [B, N]")
        if t.shape[-1] > self.max_len:
            raise ValueError(f"EncoderDecoderTransformer: {what} length {t.shape[-1]} exceeds maxLen {self.max_len}")

    def encode(self, src):
        src = _as_token_tensor(src, self.device)
        self._check(src, "source")
        return self.encoder(self.pos_enc(F.embedding(self.src_emb.weight, src)))

    def decode(self, tgt, memory):
        tgt = _as_token_tensor(tgt, self.device)
        self._check(tgt, "target")
        x = self.pos_enc(F.embedding(self.tgt_emb.weight, tgt))
        return self.head(self.decoder(x, memory, causal=True))

    def forward(self, src, tgt):
        return self.decode(tgt, self.encode(src))

    def loss(self, src, tgt_in, tgt_out):
        logits = self.forward(src, tgt_in)
        tgt_out = _as_token_tensor(tgt_out, self.device)
        return F.mean(F.cross_entropy(logits.reshape(-1, self.tgt_vocab_size), tgt_out.reshape(-1))).reshape(())

    def greedy_decode(self, src, bos: int, eos: Optional[int], max_new_tokens: int) -> List[int]:
        with torch.no_grad():
            memory = self.encode(src)
            out = [int(bos)]
            for _ in range(max_new_tokens):
                logits = self.decode(torch.tensor(out, dtype=torch.long, device=self.device), memory)
                nxt = int(torch.argmax(logits[-1].float()).item())
                out.append(nxt)
                if eos is not None and nxt == eos:
                    break
            return out
