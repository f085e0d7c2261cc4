"""HuggingFace ``tokenizer.json`` byte-level BPE and BERT WordPiece tokenizers
(reference: lib/core/data/hf_bpe_tokenizer.dart:1-445, lib/core/data/wordpiece_tokenizer.dart:1-318).

HF BPE: GPT-2 ``bytes_to_unicode`` table; pre-tokenizer regex taken from a ``Split`` pre-tokenizer when the file has
one (also inside a ``Sequence``; a leading ``(?i:...)`` is lifted to a case-insensitive flag), else the GPT-2 default;
``added_tokens`` matched as literals, longest first, before pre-tokenising; per word: whole-word vocabulary hit, else
lowest-rank pair merging; merges accepted as ``"a b"`` strings or ``[a, b]`` lists; unknown ids are skipped on decode.

WordPiece: clean -> lowercase -> strip accents -> split punctuation, greedy longest-match with ``##`` continuations and
a whole-word ``[UNK]`` fallback; ``[CLS] ... [SEP]`` framing with truncation that keeps the trailing ``[SEP]``.
"""
from __future__ import annotations

import json
import unicodedata
from typing import Dict, List, Optional, Sequence, Tuple

import regex

GPT2_PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"


def bytes_to_unicode() -> List[str]:
    """GPT-2's reversible byte -> printable code point table."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    table = [""] * 256
    for b, c in zip(bs, cs):
        table[b] = chr(c)
    return table


def _find_split_pattern(pre) -> Optional[str]:
    if not isinstance(pre, dict):
        return None
    if pre.get("type") == "Split":
        pat = pre.get("pattern")
        if isinstance(pat, dict):
            return pat.get("Regex") or pat.get("String")
    if pre.get("type") == "Sequence":
        for sub in pre.get("pretokenizers", []):
            found = _find_split_pattern(sub)
            if found:
                return found
    return None


class HFBpeTokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence, added_tokens: Sequence[dict] = (),
                 pattern: Optional[str] = None):
        self.vocab: Dict[str, int] = dict(vocab)
        self._rank: Dict[Tuple[str, str], int] = {}
        for r, m in enumerate(merges):
            if isinstance(m, str):
                parts = m.split(" ")
                if len(parts) != 2:
                    continue
                a, b = parts
            else:
                a, b = m[0], m[1]
            self._rank[(a, b)] = r
        self._byte_encoder = bytes_to_unicode()
        self._byte_decoder = {c: b for b, c in enumerate(self._byte_encoder)}
        self._specials: List[Tuple[str, int]] = []
        for t in added_tokens:
            content, tid = t.get("content"), t.get("id")
            if isinstance(content, str) and isinstance(tid, int):
                self._specials.append((content, tid))
                self.vocab.setdefault(content, tid)
        self._specials.sort(key=lambda s: -len(s[0]))
        self._id_to_token: Dict[int, str] = {i: t for t, i in self.vocab.items()}
        self._special_ids = {tid for _, tid in self._specials}
        flags = 0
        pat = pattern or GPT2_PATTERN
        if pat.startswith("(?i:") and pat.endswith(")"):
            # keep the group but make the whole expression case-insensitive, as the reference does
            flags |= regex.IGNORECASE
        self._pre = regex.compile(pat, flags)

    @classmethod
    def from_json(cls, text: str) -> "HFBpeTokenizer":
        data = json.loads(text)
        model = data.get("model")
        if not isinstance(model, dict) or "vocab" not in model:
            raise ValueError('HFBpeTokenizer: tokenizer.json has no "model.vocab"')
        if model.get("type") not in (None, "BPE"):
            raise ValueError(f"HFBpeTokenizer: unsupported model type {model.get('type')}")
        return cls(model["vocab"], model.get("merges", []), data.get("added_tokens", []) or [],
                   _find_split_pattern(data.get("pre_tokenizer")))

    @classmethod
    def load_file(cls, path: str) -> "HFBpeTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_json(f.read())

    fromJson, loadFile = from_json, load_file

    @property
    def vocab_size(self) -> int:
        return max(self.vocab.values()) + 1 if self.vocab else 0

    vocabSize = vocab_size

    def token_id(self, content: str) -> Optional[int]:
        return self.vocab.get(content)

    tokenId = token_id

    @property
    def end_of_text_id(self):
        return self.token_id("<|endoftext|>")

    @property
    def llama_eot_id(self):
        return self.token_id("<|eot_id|>")

    @property
    def llama_begin_of_text_id(self):
        return self.token_id("<|begin_of_text|>")

    endOfTextId, llamaEotId, llamaBeginOfTextId = end_of_text_id, llama_eot_id, llama_begin_of_text_id

    def _bpe_word(self, word: str) -> List[int]:
        if word in self.vocab:
            return [self.vocab[word]]
        parts = list(word)
        while len(parts) >= 2:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self._rank.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            parts = parts[:best_i] + [parts[best_i] + parts[best_i + 1]] + parts[best_i + 2:]
        return [self.vocab[p] for p in parts if p in self.vocab]

    def _encode_plain(self, text: str) -> List[int]:
        out: List[int] = []
        for m in self._pre.finditer(text):
            mapped = "".join(self._byte_encoder[b] for b in m.group(0).encode("utf-8"))
            out.extend(self._bpe_word(mapped))
        return out

    def encode(self, text: str) -> List[int]:
        if not self._specials:
            return self._encode_plain(text)
        out: List[int] = []
        i, start = 0, 0
        while i < len(text):
            hit = None
            for content, tid in self._specials:
                if text.startswith(content, i):
                    hit = (content, tid)
                    break
            if hit is None:
                i += 1
                continue
            if start < i:
                out.extend(self._encode_plain(text[start:i]))
            out.append(hit[1])
            i += len(hit[0])
            start = i
        if start < len(text):
            out.extend(self._encode_plain(text[start:]))
        return out

    def decode(self, ids: Sequence[int], skip_special: bool = False) -> str:
        buf = bytearray()
        out: List[str] = []

        def flush():
            if buf:
                out.append(bytes(buf).decode("utf-8", errors="replace"))
                buf.clear()
        for tid in ids:
            tok = self._id_to_token.get(int(tid))
            if tok is None:
                continue
            if int(tid) in self._special_ids:
                flush()
                if not skip_special:
                    out.append(tok)
                continue
            for ch in tok:
                b = self._byte_decoder.get(ch)
                if b is None:
                    flush()
                    out.append(ch)
                else:
                    buf.append(b)
        flush()
        return "".join(out)


def _is_punct(ch: str) -> bool:
    cp = ord(ch)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(ch).startswith("P")


class WordPieceTokenizer:
    def __init__(self, vocab: Sequence[str], unk: str = "[UNK]", cls: str = "[CLS]", sep: str = "[SEP]",
                 pad: str = "[PAD]", do_lower_case: bool = True, max_input_chars_per_word: int = 100):
        self.tokens: List[str] = list(vocab)
        self.vocab: Dict[str, int] = {t: i for i, t in enumerate(self.tokens)}
        for name, tok in (("unk", unk), ("cls", cls), ("sep", sep), ("pad", pad)):
            if tok not in self.vocab:
                raise ValueError(f'WordPieceTokenizer: vocab has no "{tok}" ({name}) token')
        self.unk_id, self.cls_id, self.sep_id, self.pad_id = (self.vocab[t] for t in (unk, cls, sep, pad))
        self.do_lower_case, self.max_chars = do_lower_case, max_input_chars_per_word

    @classmethod
    def from_vocab_file(cls, path: str, **kw) -> "WordPieceTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return cls([line.rstrip("\n") for line in f if line.rstrip("\n") != ""], **kw)

    fromVocabFile = from_vocab_file

    @property
    def vocab_size(self) -> int:
        return len(self.tokens)

    def _basic(self, text: str) -> List[str]:
        cleaned = []
        for ch in text:
            cp = ord(ch)
            if cp == 0 or cp == 0xFFFD or (unicodedata.category(ch) in ("Cc", "Cf") and ch not in "\t\n\r"):
                continue
            cleaned.append(" " if ch.isspace() else ch)
        text = "".join(cleaned)
        if self.do_lower_case:
            text = text.lower()
            text = "".join(c for c in unicodedata.normalize("NFD", text) if unicodedata.category(c) != "Mn")
        words: List[str] = []
        for w in text.split():
            cur = ""
            for ch in w:
                if _is_punct(ch):
                    if cur:
                        words.append(cur)
                        cur = ""
                    words.append(ch)
                else:
                    cur += ch
            if cur:
                words.append(cur)
        return words

    def tokenize(self, text: str) -> List[str]:
        out: List[str] = []
        for word in self._basic(text):
            if len(word) > self.max_chars:
                out.append(self.tokens[self.unk_id])
                continue
            pieces, start, bad = [], 0, False
            while start < len(word):
                end, cur = len(word), None
                while start < end:
                    sub = word[start:end]
                    if start > 0:
                        sub = "##" + sub
                    if sub in self.vocab:
                        cur = sub
                        break
                    end -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(cur)
                start = end
            out.extend([self.tokens[self.unk_id]] if bad else pieces)
        return out

    def encode(self, text: str, add_special_tokens: bool = True, max_length: Optional[int] = None) -> List[int]:
        ids = [self.vocab[t] for t in self.tokenize(text)]
        if add_special_tokens:
            ids = [self.cls_id] + ids + [self.sep_id]
        if max_length is not None and len(ids) > max_length:
            ids = ids[:max_length - 1] + [self.sep_id] if add_special_tokens else ids[:max_length]
        return ids

    def encode_pair(self, a: str, b: str, max_length: Optional[int] = None) -> List[int]:
        ia = [self.vocab[t] for t in self.tokenize(a)]
        ib = [self.vocab[t] for t in self.tokenize(b)]
        if max_length is not None:
            budget = max(0, max_length - 3)
            while len(ia) + len(ib) > budget:      # trim the longer side first
                if len(ia) >= len(ib) and ia:
                    ia.pop()
                elif ib:
                    ib.pop()
                else:
                    break
        return [self.cls_id] + ia + [self.sep_id] + ib + [self.sep_id]

    encodePair = encode_pair

    def decode(self, ids: Sequence[int]) -> str:
        words: List[str] = []
        for i in ids:
            i = int(i)
            if i in (self.cls_id, self.sep_id, self.pad_id) or not (0 <= i < len(self.tokens)):
                continue
            tok = self.tokens[i]
            if tok.startswith("##") and words:
                words[-1] += tok[2:]
            else:
                words.append(tok)
        return " ".join(words)


def debug_preview(ids: Sequence[int], max_items: int) -> str:
    """JSON list of the first ``max_items`` ids, with the total appended when the list is longer
    (reference: lib/core/data/wordpiece_tokenizer.dart:315-318)."""
    ids = [int(i) for i in ids]
    if len(ids) <= max_items:
        return json.dumps(ids, separators=(",", ":"))
    return f"{json.dumps(ids[:max_items], separators=(',', ':'))} ...({len(ids)} total)"


debugPreview = debug_preview
