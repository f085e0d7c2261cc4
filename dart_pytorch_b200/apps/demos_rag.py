"""Retrieval, question-answering and Hugging Face loading demos (third part of the reference's ``bin/`` demos).

With ``--model-dir`` pointing at a downloaded ``sentence-transformers/all-MiniLM-L6-v2`` (``model.safetensors`` +
``vocab.txt``) the sentence demos use the pretrained encoder, as the originals do.  Without it they build a small
BERT over a WordPiece vocabulary made from the demo corpus, so that every command runs offline.

Reference programs: bin/rag_learn.dart, bin/rag_demo.dart, bin/rag_gpu_demo.dart, bin/rag_qa_demo.dart, bin/qa.dart,
bin/vector_store_demo.dart, bin/gpt2_hf_demo.dart.
"""
from __future__ import annotations

import json
import os
import random
import re
import tempfile
import time
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from .demos import _dev, _train

FACTS = [
    "The Eiffel Tower is a wrought iron lattice tower in Paris, France.",
    "Mount Kilimanjaro in Tanzania is the highest mountain in Africa.",
    "Python is a programming language created by Guido van Rossum.",
    "The Great Barrier Reef off Australia is the largest coral reef system.",
    "A car seat keeps small children safe in a vehicle.",
    "Minivans are popular family vehicles with sliding doors.",
    "Simmer the tomato sauce slowly and season it with basil.",
    "Knead the bread dough until it is smooth and elastic.",
    "Gravity bends light that passes near a massive star.",
    "Electrons carry a negative electric charge.",
]
QUERIES = [("Which tower stands in Paris?", 0), ("What is the tallest mountain in Africa?", 1),
           ("Who created the Python language?", 2), ("How do I keep children safe in a vehicle?", 4),
           ("How should the dough be kneaded?", 7), ("What charge do electrons carry?", 9)]


def _words(text: str) -> List[str]:
    return re.findall(r"[a-z0-9]+", text.lower())


def _sentence_stack(args, extra_text: Sequence[str] = ()):
    """(SentenceEncoder over a BERT backbone, WordPiece tokenizer, label)."""
    from ..data.hf_tokenizers import WordPieceTokenizer
    from ..io.hf_loaders_more import BertHFLoader
    from ..models import BertConfig, BertModel, SentenceEncoder
    dev = _dev(args)
    model_dir = getattr(args, "model_dir", None)
    if model_dir:
        tok = WordPieceTokenizer.from_vocab_file(os.path.join(model_dir, "vocab.txt"))
        bert = BertModel(BertHFLoader.mini_lm_l6_v2_config(device=dev))
        rep = BertHFLoader.load_file(bert, os.path.join(model_dir, "model.safetensors"))
        return SentenceEncoder.wrap(bert), tok, f"all-MiniLM-L6-v2 ({rep.consumed_count} tensors)"
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]"] + sorted({w for s in list(FACTS) + [q for q, _ in QUERIES] +
                                                          list(extra_text) for w in _words(s)})
    tok = WordPieceTokenizer(vocab)
    bert = BertModel(BertConfig(len(vocab), 64, 32, 2, 4, 64, device=dev, seed=getattr(args, "seed", 0)))
    return SentenceEncoder.wrap(bert), tok, "tiny random BERT (no --model-dir)"


def _encode(enc, tok, texts: Sequence[str], dev: str, grad: bool = False) -> torch.Tensor:
    rows = []
    for t in texts:
        ids = torch.tensor(tok.encode(t, max_length=64), device=dev)
        rows.append(enc(ids) if grad else enc(ids).detach())
    return torch.cat([r.reshape(1, -1) for r in rows], 0)


def _top1(enc, tok, dev) -> Tuple[float, float]:
    with torch.no_grad():
        c = _encode(enc, tok, FACTS, dev)
        q = _encode(enc, tok, [t for t, _ in QUERIES], dev)
    sim = q @ c.t()
    gold = torch.tensor([g for _, g in QUERIES], device=sim.device)
    acc = float((sim.argmax(-1) == gold).float().mean())
    return acc, float(sim[torch.arange(len(QUERIES)), gold].mean())


def demo_rag_learn(args) -> Dict:
    """Fine-tune the sentence encoder with the in-batch multiple-negatives ranking loss; retrieval before / after."""
    from ..models import SentenceLosses
    dev = _dev(args)
    enc, tok, label = _sentence_stack(args)
    acc0, pos0 = _top1(enc, tok, dev)
    rng = random.Random(args.seed)

    def loss_fn(_):
        batch = rng.sample(QUERIES, 4)
        a = _encode(enc, tok, [q for q, _ in batch], dev, grad=True)
        p = _encode(enc, tok, [FACTS[g] for _, g in batch], dev, grad=True)
        return SentenceLosses.multiple_negatives_ranking_loss(a, p).mean()
    losses = _train(enc, enc.parameters(), loss_fn, args.steps, lr=1e-3)
    acc1, pos1 = _top1(enc, tok, dev)
    print(f"{label}: top-1 {acc0:.2f} -> {acc1:.2f}; cosine to the gold passage {pos0:.3f} -> {pos1:.3f}; "
          f"loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return {"acc_before": acc0, "acc_after": acc1, "pos_before": pos0, "pos_after": pos1,
            "loss_first": losses[0], "loss_last": losses[-1]}


def demo_rag_demo(args) -> Dict:
    """Index the factlets, print the top-3 passages per query and a quoted answer."""
    from ..models import Similarity
    dev = _dev(args)
    enc, tok, label = _sentence_stack(args)
    with torch.no_grad():
        corpus = _encode(enc, tok, FACTS, dev)
        queries = _encode(enc, tok, [q for q, _ in QUERIES], dev)
    hits = Similarity.semantic_search(queries, corpus, top_k=3)
    answers = []
    for (q, _), row in zip(QUERIES, hits):
        print(f"Q: {q}")
        for h in row:
            print(f"   {h.score:+.3f}  {FACTS[h.corpus_index]}")
        answers.append(FACTS[row[0].corpus_index])
        print(f"A: {answers[-1]}")
    return {"encoder": label, "answers": answers, "top_k": len(hits[0])}


def demo_rag_gpu_demo(args) -> Dict:
    """The same sentences encoded on the CPU and (when there is one) on the GPU: per-sentence time and agreement."""
    out = {}
    embs = {}
    devices = ["cpu"] + (["cuda"] if torch.cuda.is_available() else [])
    for dev in devices:
        a = type(args)(**{**vars(args), "device": dev})
        enc, tok, _ = _sentence_stack(a)
        with torch.no_grad():
            _encode(enc, tok, FACTS[:2], dev)
            t0 = time.perf_counter()
            for _ in range(max(1, args.steps)):
                e = _encode(enc, tok, FACTS, dev)
            if dev == "cuda":
                torch.cuda.synchronize()
        out[dev + "_ms_per_sentence"] = 1e3 * (time.perf_counter() - t0) / max(1, args.steps) / len(FACTS)
        embs[dev] = e.float().cpu()
    if "cuda" in embs:
        out["max_abs_diff"] = float((embs["cpu"] - embs["cuda"]).abs().max())
    print(out)
    return out


# ---------------------------------------------------------------------------------- causal-LM retrieval + QA ---
def _char_lm(args, text: str):
    from ..coop.lm_factory import build_coop_lm
    from ..data.tokenizers import CharTokenizer
    tok = CharTokenizer.from_text(text + "".join(chr(c) for c in range(32, 127)) + "\n")
    return build_coop_lm("gpt", "small", tok.vocab_size, device=_dev(args)).module, tok


def demo_rag_qa_demo(args) -> Dict:
    """Retrieval-augmented QA where one causal LM is both the encoder (last-token hidden state, corpus-mean
    centred, L2-normalised) and the generator; with ``--model-dir`` that LM is a Hugging Face GPT-2."""
    from .servers import RagChatService, load_hf_model
    if getattr(args, "model_dir", None):
        model, tok, _ = load_hf_model("gpt2", args.model_dir, device=_dev(args))
        label = "gpt2"
    else:
        model, tok = _char_lm(args, " ".join(FACTS))
        label = "char-gpt (untrained)"
    svc = RagChatService(model, tok, arch_label="gpt", preset_label=label, max_new_tokens=16)
    code, up = svc.upload("facts.txt", "\n\n".join(FACTS))
    code, res = svc.chat(QUERIES[0][0])
    print(f"{label}: indexed {up.get('chunks', up)} chunks; sources for {QUERIES[0][0]!r}:")
    for s in res["sources"]:
        print(f"   {s['score']:+.3f}  {s['preview']}")
    print("answer:", repr(res["answer"]))
    return {"status": code, "sources": len(res["sources"]), "prompt_tokens": res["promptTokens"]}


def _chunks(text: str, chunk_words: int, overlap: int) -> List[str]:
    out = []
    for para in re.split(r"\n\s*\n", text):
        w = para.split()
        if not w:
            continue
        if len(w) <= chunk_words:
            out.append(" ".join(w))
            continue
        step = max(1, chunk_words - overlap)
        for s in range(0, len(w), step):
            out.append(" ".join(w[s:s + chunk_words]))
            if s + chunk_words >= len(w):
                break
    return out


def demo_qa(args) -> Dict:
    """The semantic-QA tool's two phases with the file backend: ``build`` chunks a corpus (blank-line paragraphs,
    long ones in overlapping word windows), encodes every chunk and saves index + chunk table to a directory;
    ``ask`` reloads both and ranks the chunks for a question."""
    from .. import vector_store as vs
    dev = _dev(args)
    corpus_path = getattr(args, "corpus", None)
    text = open(corpus_path, encoding="utf-8").read() if corpus_path else "\n\n".join(FACTS)
    chunks = _chunks(text, getattr(args, "chunk_words", 120), getattr(args, "overlap_words", 20))
    enc, tok, label = _sentence_stack(args, extra_text=chunks)
    question = getattr(args, "question", None) or QUERIES[1][0]
    with tempfile.TemporaryDirectory() as tmp:
        out_dir = getattr(args, "out", None) or tmp
        os.makedirs(out_dir, exist_ok=True)
        index = vs.IndexFlatIP(enc.embed_dim)
        index.add(_encode(enc, tok, chunks, dev).float().cpu().numpy())
        vs.write_index(index, os.path.join(out_dir, "chunks.dvi"))
        with open(os.path.join(out_dir, "chunks.json"), "w", encoding="utf-8") as f:
            json.dump(chunks, f)
        # ask: a fresh process would start here
        index2 = vs.read_index(os.path.join(out_dir, "chunks.dvi"))
        with open(os.path.join(out_dir, "chunks.json"), encoding="utf-8") as f:
            table = json.load(f)
        res = index2.search(_encode(enc, tok, [question], dev).float().cpu().numpy(), min(3, len(table)))
    print(f"{label}: {len(chunks)} chunks indexed; Q: {question}")
    for cid, score in zip(res.ids[0], res.distances[0]):
        print(f"   {float(score):+.3f}  {table[int(cid)][:100]}")
    return {"chunks": len(chunks), "reloaded": index2.ntotal, "top": int(res.ids[0][0])}


def demo_vector_store_demo(args) -> Dict:
    """Word-hash tokens -> TextTransformer -> mean pool -> L2 normalise; cosine search by ``query @ index^T``;
    triplet-loss fine-tuning pulls the semantic groups apart."""
    from ..models import SentenceEncoder, SentenceLosses
    dev = _dev(args)
    groups = {"vehicles": [4, 5], "cooking": [6, 7], "physics": [8, 9]}
    docs = [FACTS[i] for g in groups.values() for i in g]
    group_of = [name for name, g in groups.items() for _ in g]
    buckets, seq = 256, 12

    def hash_ids(text: str) -> torch.Tensor:
        ids = [1 + (sum(ord(c) * 31 ** k for k, c in enumerate(w)) % (buckets - 1)) for w in _words(text)][:seq]
        return torch.tensor(ids + [0] * (seq - len(ids)), device=dev)
    enc = SentenceEncoder(buckets, seq, 32, 1, 4, device=dev, seed=args.seed)
    query = "What is a safe vehicle for kids?"

    def rank() -> List[str]:
        with torch.no_grad():
            index = torch.cat([enc(hash_ids(d)).reshape(1, -1) for d in docs], 0)
            scores = (enc(hash_ids(query)).reshape(1, -1) @ index.t()).reshape(-1)
        return [group_of[i] for i in torch.argsort(scores, descending=True).tolist()]
    before = rank()
    rng = random.Random(args.seed)

    def loss_fn(_):
        g = rng.choice(list(groups))
        other = rng.choice([x for x in groups if x != g])
        a, p = (FACTS[i] for i in groups[g])
        n = FACTS[rng.choice(groups[other])]
        e = [enc(hash_ids(t)).reshape(1, -1) for t in (a, p, n)]
        return SentenceLosses.triplet_loss(e[0], e[1], e[2], margin=0.5).mean()
    losses = _train(enc, enc.parameters(), loss_fn, args.steps, lr=2e-3)
    after = rank()
    print(f"triplet loss {losses[0]:.3f} -> {losses[-1]:.3f}\nranking before: {before}\nranking after:  {after}")
    return {"before": before, "after": after, "loss_first": losses[0], "loss_last": losses[-1]}


def demo_gpt2_hf_demo(args) -> Dict:
    """Load Hugging Face GPT-2 ``.safetensors`` weights into ``GPT`` and run a forward pass.  With no file given, a
    small GPT-2-layout checkpoint is written first (Conv1D ``[in, out]`` weights, ``h.N.`` names), so the loader's
    whole path (name mapping, transposes, tied head) runs offline."""
    from .. import GPT, GPTConfig
    from ..io.hf_loaders import GPT2HFLoader
    from ..io.safetensors import SafeTensors
    from ..nn.transformer import Activation
    dev = _dev(args)
    path = getattr(args, "weights", None)
    with tempfile.TemporaryDirectory() as tmp:
        if path:
            cfg = GPT2HFLoader.gpt2_small_config(device=dev)
        else:
            cfg = GPTConfig(vocab_size=96, max_ctx=32, embed_dim=32, num_layers=2, num_heads=4, attn_bias=True,
                            activation=Activation.geluTanh, seed=args.seed + 5, device=dev)
            donor = GPT(cfg)
            path = os.path.join(tmp, "model.safetensors")
            SafeTensors.save_file({k: v.detach().cpu() for k, v in GPT2HFLoader.dump(donor).items()}, path)
            want = donor(torch.arange(8, device=dev)).detach()
            cfg = GPTConfig(vocab_size=96, max_ctx=32, embed_dim=32, num_layers=2, num_heads=4, attn_bias=True,
                            activation=Activation.geluTanh, seed=args.seed + 6, device=dev)
        model = GPT(cfg)
        t0 = time.perf_counter()
        rep = GPT2HFLoader.load_file(model, path)
        dt = time.perf_counter() - t0
    logits = model(torch.arange(8, device=dev)).detach()
    out = {"loaded": rep.consumed_count, "logits_shape": tuple(logits.shape), "load_s": dt}
    if "want" in locals():
        out["max_abs_diff"] = float((logits.float() - want.float()).abs().max())
    nxt = model.generate([0.0, 1.0, 2.0], 5, temperature=0.0)
    print(f"loaded {rep.consumed_count} tensors in {dt:.2f} s; logits {out['logits_shape']}; greedy continuation {nxt[3:]}")
    return out
