"""Vector-store application demos and the small debug programs (last part of the reference's ``bin/`` demos).

Sentence embeddings come from ``demos_rag._sentence_stack``: the pretrained MiniLM when ``--model-dir`` is given, a
small random BERT otherwise (its mean-pooled embeddings still follow word overlap, which is what the toy corpora
below are built around).

Reference programs: bin/vector_chunked_rag_demo.dart, bin/vector_cluster_demo.dart, bin/vector_dedup_demo.dart,
bin/vector_image_search_demo.dart, bin/vector_index_benchmark_demo.dart, bin/vector_zero_shot_classify_demo.dart,
bin/_bug_repro.dart, bin/_gpt2_debug.dart, bin/_prep_coco_pairs.dart, bin/dart_pytorch.dart.
"""
from __future__ import annotations

import json
import os
import tempfile
import time
from typing import Dict, List

import numpy as np
import torch

from .demos import _dev, _toy_images, _train
from .demos_rag import _chunks, _encode, _sentence_stack

TOPICS = {
    "astronomy": ["The telescope observed a distant galaxy and its stars.",
                  "Stars in the galaxy orbit a black hole.",
                  "The telescope tracked a comet near the stars."],
    "cooking": ["Bake the bread in a hot oven with butter.",
                "Stir butter and flour, then bake the cake in the oven.",
                "The oven must be hot before you bake bread."],
    "football": ["The striker scored a goal in the football match.",
                 "The football team won the match with a late goal.",
                 "A goal in extra time decided the football final."],
}


def _topic_docs():
    docs = [d for ds in TOPICS.values() for d in ds]
    labels = [name for name, ds in TOPICS.items() for _ in ds]
    return docs, labels


class _Centred:
    """Encoder wrapper of the offline fallback: a random BERT puts every sentence in one narrow cone, so embeddings
    are centred on the corpus mean and re-normalised (the trick bin/rag_qa_demo.dart uses for causal-LM vectors)."""

    def __init__(self, enc, mean):
        self.enc, self.mean, self.embed_dim = enc, mean, enc.embed_dim

    def __call__(self, ids):
        v = self.enc(ids).reshape(1, -1) - self.mean
        return v / v.norm().clamp_min(1e-9)


def _embed(args, texts, extra=()):
    enc, tok, label = _sentence_stack(args, extra_text=list(texts) + list(extra))
    with torch.no_grad():
        e = _encode(enc, tok, texts, _dev(args))
        if not getattr(args, "model_dir", None):
            enc = _Centred(enc, e.mean(0, keepdim=True))
            e = _encode(enc, tok, texts, _dev(args))
    return e.float().cpu().numpy(), enc, tok, label


def demo_vector_cluster_demo(args) -> Dict:
    """Topic discovery: k-means over sentence embeddings; each cluster is printed with its members."""
    from .. import vector_store as vs
    docs, labels = _topic_docs()
    e, _, _, label = _embed(args, docs)
    res = vs.Kmeans(e.shape[1], len(TOPICS), niter=20, seed=args.seed + 1).train(e)
    purity = 0
    for c in range(len(TOPICS)):
        members = [i for i, a in enumerate(res.assignments) if a == c]
        names = [labels[i] for i in members]
        if names:
            purity += max(names.count(n) for n in set(names))
        print(f"cluster {c}: {names}")
    print(f"{label}: purity {purity / len(docs):.2f}, objective {res.objective:.3f}")
    return {"purity": purity / len(docs), "clusters": len(TOPICS), "objective": float(res.objective)}


def demo_vector_dedup_demo(args) -> Dict:
    """Near-duplicate detection: range search around every document, pairs joined into connected components."""
    from .. import vector_store as vs
    docs, _ = _topic_docs()
    docs = docs + [docs[0].replace("observed", "saw"), docs[3] + " Enjoy.", docs[6].replace("The striker", "A striker")]
    e, _, _, label = _embed(args, docs)
    index = vs.IndexFlatIP(e.shape[1])
    index.add(e)
    # the centred fallback embeddings spread out much further than MiniLM's, hence its lower default threshold
    threshold = getattr(args, "threshold", None) or (0.9 if getattr(args, "model_dir", None) else 0.6)
    rr = index.range_search(e, threshold)
    parent = list(range(len(docs)))

    def find(i):
        while parent[i] != i:
            parent[i] = parent[parent[i]]
            i = parent[i]
        return i
    for q in range(rr.nq):
        for j in rr.ids[rr.limits[q]:rr.limits[q + 1]]:
            if int(j) != q:
                parent[find(q)] = find(int(j))
    groups: Dict[int, List[int]] = {}
    for i in range(len(docs)):
        groups.setdefault(find(i), []).append(i)
    dup = sorted(g for g in groups.values() if len(g) > 1)
    for g in dup:
        print("duplicates:", [docs[i][:50] for i in g])
    print(f"{label}: {len(dup)} duplicate groups at cosine > {threshold}")
    return {"groups": dup, "n_docs": len(docs)}


def demo_vector_zero_shot_classify_demo(args) -> Dict:
    """No classifier is trained: every label is a sentence, documents take the label whose embedding is nearest."""
    from .. import vector_store as vs
    docs, gold = _topic_docs()
    prompts = {"astronomy": "This text is about stars, a galaxy and the telescope.",
               "cooking": "This text is about the oven, bread and how to bake.",
               "football": "This text is about a football match and a goal."}
    names = list(prompts)
    e, enc, tok, label = _embed(args, docs, extra=list(prompts.values()))
    with torch.no_grad():
        le = _encode(enc, tok, [prompts[n] for n in names], _dev(args)).float().cpu().numpy()
    index = vs.IndexFlatIP(e.shape[1])
    index.add(le)
    pred = [names[int(i)] for i in index.search(e, 1).ids[:, 0]]
    acc = sum(p == g for p, g in zip(pred, gold)) / len(gold)
    print(f"{label}: zero-shot accuracy {acc:.2f}; predictions {pred}")
    return {"accuracy": acc, "pred": pred}


def demo_vector_image_search_demo(args) -> Dict:
    """Image-to-image search: patchify -> ViT face embedder -> L2-normalised vectors -> inner-product index."""
    from .. import vector_store as vs
    from ..models import ViTFaceEmbedding
    dev = _dev(args)
    model = ViTFaceEmbedding(image_size=16, patch_size=8, embed_dim=32, num_layers=1, device=dev, seed=args.seed)
    gallery, labels = _toy_images(24, 4, 16, args.seed, dev)
    with torch.no_grad():
        e = model(gallery).float().cpu().numpy()
    index = vs.IndexFlatIP(e.shape[1])
    index.add(e)
    q = 5
    noisy = gallery[q:q + 1] + 0.02 * torch.randn(gallery[q:q + 1].shape, generator=torch.Generator().manual_seed(3)).to(dev)
    with torch.no_grad():
        qe = model(noisy).float().cpu().numpy()
    res = index.search(qe, 4)
    hits = [int(i) for i in res.ids[0]]
    print(f"query = noisy image {q} (class {int(labels[q])}); hits {hits} classes {[int(labels[i]) for i in hits]}")
    return {"hits": hits, "top_is_source": hits[0] == q, "same_class_top4": sum(int(labels[i] == labels[q]) for i in hits)}


def demo_vector_index_benchmark_demo(args) -> Dict:
    """Same vectors, same queries, every index type: build time, search time, recall@10 against the flat scan."""
    from .. import vector_store as vs
    n, d, nq, k = getattr(args, "n", 2000), 32, 40, 10
    rng = np.random.default_rng(args.seed)
    centers = rng.normal(size=(16, d)).astype(np.float32)
    xs = (centers[rng.integers(0, 16, n)] + 0.3 * rng.normal(size=(n, d))).astype(np.float32)
    qs = (centers[rng.integers(0, 16, nq)] + 0.3 * rng.normal(size=(nq, d))).astype(np.float32)
    flat = vs.IndexFlatL2(d)
    flat.add(xs)
    truth = flat.search(qs, k)
    rows = []
    for desc in ("Flat", "IVF16,Flat", "HNSW16", "PQ8", "SQ8", "IVF16,PQ8"):
        idx = vs.index_factory(d, desc)
        t0 = time.perf_counter()
        idx.train(xs)
        idx.add(xs)
        build = time.perf_counter() - t0
        r = vs.bench_index(idx, qs, k, truth, label=desc)
        rows.append(r)
        print(f"{desc:12s} build {build * 1e3:7.1f} ms   recall@{k} {r.recall:.3f}")
    print(vs.format_bench_table(rows))
    return {"recall": {r.label: r.recall for r in rows}}


def demo_vector_chunked_rag_demo(args) -> Dict:
    """Long documents are split into overlapping word windows, every chunk is embedded and indexed with the id of
    its document; a query retrieves chunks, which are then grouped back by document."""
    from .. import vector_store as vs
    docs, labels = _topic_docs()
    long_docs = {name: " ".join(TOPICS[name] * 6) for name in TOPICS}
    chunks, owner = [], []
    for name, text in long_docs.items():
        for c in _chunks(text, 24, 6):
            chunks.append(c)
            owner.append(name)
    query = "Which team scored the late goal in the football match?"
    e, enc, tok, label = _embed(args, chunks, extra=[query])
    index = vs.IndexIDMap(vs.IndexFlatIP(e.shape[1]))
    index.add_with_ids(e, np.arange(1000, 1000 + len(chunks), dtype=np.int64))
    with torch.no_grad():
        qe = _encode(enc, tok, [query], _dev(args)).float().cpu().numpy()
    res = index.search(qe, 5)
    votes: Dict[str, float] = {}
    for cid, score in zip(res.ids[0], res.distances[0]):
        votes[owner[int(cid) - 1000]] = votes.get(owner[int(cid) - 1000], 0.0) + float(score)
    best = max(votes, key=votes.get)
    print(f"{label}: {len(chunks)} chunks from {len(long_docs)} documents; query -> document '{best}' (votes {votes})")
    return {"chunks": len(chunks), "best": best}


# ------------------------------------------------------------------------------------------- debug programs ---
def demo_bug_repro(args) -> Dict:
    """Regression for the all-parameters-become-zero failure: a mid-size GPT trained for many optimizer steps keeps
    finite, non-zero parameters and a non-zero loss."""
    from .. import GPT, GPTConfig
    dev = _dev(args)
    model = GPT(GPTConfig(vocab_size=64, max_ctx=32, embed_dim=64, num_layers=2, num_heads=4, seed=args.seed, device=dev))
    g = torch.Generator().manual_seed(args.seed)
    seq = torch.randint(0, 64, (33,), generator=g).to(dev)
    losses = _train(model, model.parameters(), lambda s: model.loss(seq[:-1], seq[1:]), max(args.steps, 12))
    finite = all(bool(torch.isfinite(p).all()) for p in model.parameters())
    nonzero = all(float(p.detach().abs().sum()) > 0 for p in model.parameters() if p.numel() > 1 and p.dim() > 1)
    print(f"{len(losses)} steps: loss {losses[0]:.4f} -> {losses[-1]:.4f}; parameters finite {finite}, non-zero {nonzero}")
    return {"finite": finite, "nonzero": nonzero, "loss_last": losses[-1]}


def demo_gpt2_debug(args) -> Dict:
    """Per-stage statistics (mean, variance, non-finite count) of a GPT forward pass: embeddings, every block's
    output, final norm, logits — the tool that isolates where a NaN first appears after loading weights."""
    from .. import GPT, GPTConfig
    from ..io.hf_loaders import GPT2HFLoader
    from ..nn.transformer import Activation
    dev = _dev(args)
    path = getattr(args, "weights", None)
    if path:
        model = GPT(GPT2HFLoader.gpt2_small_config(device=dev))
        GPT2HFLoader.load_file(model, path)
    else:
        model = GPT(GPTConfig(vocab_size=96, max_ctx=32, embed_dim=32, num_layers=2, num_heads=4, attn_bias=True,
                              activation=Activation.geluTanh, seed=args.seed, device=dev))
    tokens = torch.arange(8, device=dev)
    rows = []

    def stat(label, t):
        x = t.detach().float()
        bad = int((~torch.isfinite(x)).sum())
        rows.append((label, bad))
        print(f"{label:14s} shape={list(x.shape)} mean={float(x.mean()):+.6f} var={float(x.var(unbiased=False)):.6f} "
              f"nonfinite={bad}")
    with torch.no_grad():
        stat("hidden", model.hidden(tokens))
        stat("logits", model(tokens))
        for i, p in enumerate(model.parameters()[:6]):
            stat(f"param[{i}]", p)
    return {"stages": [r[0] for r in rows], "nonfinite": sum(r[1] for r in rows)}


def demo_prep_coco_pairs(args) -> Dict:
    """Turn a COCO ``captions_*.json`` into the ``img.jpg`` + ``img.txt`` folder layout of the projector trainer.
    Without ``--json`` a three-image annotation file is generated first so that the conversion can be shown."""
    from PIL import Image
    with tempfile.TemporaryDirectory() as tmp:
        src = getattr(args, "json", None)
        images_dir = getattr(args, "images", None)
        if not src:
            images_dir = os.path.join(tmp, "val")
            os.makedirs(images_dir)
            ann = {"images": [], "annotations": []}
            for i in range(3):
                name = f"{i:012d}.jpg"
                Image.new("RGB", (16, 16), (40 * i, 80, 120)).save(os.path.join(images_dir, name))
                ann["images"].append({"id": i, "file_name": name})
                ann["annotations"].append({"image_id": i, "caption": f"a synthetic picture number {i}"})
                ann["annotations"].append({"image_id": i, "caption": "a second caption that is ignored"})
            src = os.path.join(tmp, "captions.json")
            with open(src, "w", encoding="utf-8") as f:
                json.dump(ann, f)
        out = getattr(args, "out", None) or os.path.join(tmp, "pairs")
        os.makedirs(out, exist_ok=True)
        with open(src, encoding="utf-8") as f:
            ann = json.load(f)
        first_caption = {}
        for a in ann["annotations"]:
            first_caption.setdefault(a["image_id"], a["caption"].strip())
        n = 0
        for im in ann["images"][:getattr(args, "n", 200)]:
            if im["id"] not in first_caption:
                continue
            src_img = os.path.join(images_dir or os.path.dirname(src), im["file_name"])
            if not os.path.exists(src_img):
                continue
            with open(src_img, "rb") as fi, open(os.path.join(out, im["file_name"]), "wb") as fo:
                fo.write(fi.read())
            with open(os.path.join(out, os.path.splitext(im["file_name"])[0] + ".txt"), "w", encoding="utf-8") as f:
                f.write(first_caption[im["id"]] + "\n")
            n += 1
        files = sorted(os.listdir(out))
    print(f"wrote {n} (image, caption) pairs: {files[:4]} ...")
    return {"pairs": n, "files": files}


def demo_hello(args) -> Dict:
    """The package's hello-world: version, device, one tensor op."""
    import dart_pytorch_b200 as pkg
    dev = _dev(args)
    x = torch.arange(6, dtype=torch.float32, device=dev).reshape(2, 3)
    print(f"dart_pytorch_b200 {getattr(pkg, '__version__', '')} on {dev}: sum of {x.tolist()} = {float(x.sum())}")
    return {"sum": float(x.sum())}
