"""Multimodal, world-model and vision-language demo programs (second half of the reference's ``bin/`` demos).

Same conventions as ``demos.py``: every ``demo_*`` function takes the parsed CLI arguments (``device``, ``steps``,
``seed``), runs on small synthetic data offline and returns a dict of results.

Reference programs: bin/multi_modal_demo.dart, bin/train_multimodal_demo.dart, bin/train_muzero_shakespeare.dart,
bin/train_llama_vision_demo.dart, bin/train_llava_projector.dart, bin/llama_llava_demo.dart,
bin/llama_image_rag.dart, bin/_clip_smoke.dart, bin/_lc0_bench_batch.dart.
"""
from __future__ import annotations

import random
import time
from typing import Dict, List

import numpy as np
import torch

from .demos import _dev, _train
from .util import load_corpus


# ------------------------------------------------------------------------------------------------ multimodal ---
def _modal_batch(n: int, classes: int, seed: int, dev: str):
    """Synthetic (audio [20,10], video [8,32], text [16]) triples whose class shifts every modality's mean."""
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, classes, (n,), generator=g)
    audio = torch.randn(n, 20, 10, generator=g) + labels.view(n, 1, 1).float()
    video = torch.randn(n, 8, 32, generator=g) - labels.view(n, 1, 1).float()
    text = (torch.randint(0, 10, (n, 16), generator=g) + 10 * labels.view(n, 1)).clamp_max(49)
    return audio.to(dev), video.to(dev), text.to(dev), labels.to(dev)


def demo_multi_modal_demo(args) -> Dict:
    """Forward shapes of the three modality encoders, the late-fusion classifier, the fusion encoder and the
    cross-attention generator."""
    from ..models import (AudioTransformer, MultiModalClassifier, MultiModalEncoder, MultiModalGenerator,
                          TextTransformer, VideoTransformer)
    dev = _dev(args)
    au = AudioTransformer(10, 20, 32, 1, 4, device=dev, seed=args.seed)
    vi = VideoTransformer(32, 8, 32, 1, 4, device=dev, seed=args.seed + 1)
    tx = TextTransformer(50, 16, 32, 1, 4, device=dev, seed=args.seed + 2)
    audio, video, text, _ = _modal_batch(1, 5, args.seed, dev)
    out = {"audio": tuple(au(audio[0]).shape), "video": tuple(vi(video[0]).shape), "text": tuple(tx(text[0]).shape)}
    clf = MultiModalClassifier(au, vi, 5, text=tx, device=dev, seed=args.seed)
    out["classifier"] = tuple(clf(audio[0], video[0], text[0]).shape)
    enc = MultiModalEncoder(au, vi, 32, text=tx, fusion_layers=1, device=dev, seed=args.seed)
    out["fused"] = tuple(enc(audio[0], video[0], text[0]).shape)
    gen = MultiModalGenerator(50, 12, 32, audio=au, video=vi, decoder_layers=1, device=dev, seed=args.seed)
    out["generator_logits"] = tuple(gen(text[0][:6], audio_features=audio[0], video_frames=video[0]).shape)
    out["generated"] = gen.generate([1], 4, audio_features=audio[0], video_frames=video[0])
    print(out)
    return out


def demo_train_multimodal_demo(args) -> Dict:
    """Train the late-fusion classifier and the single-stream multimodal LM on synthetic triples."""
    from .. import ops as F
    from ..models import AudioTransformer, MultiModalClassifier, MultiModalLM, TextTransformer, VideoTransformer
    dev = _dev(args)
    clf = MultiModalClassifier(AudioTransformer(10, 20, 32, 1, 4, device=dev, seed=1),
                               VideoTransformer(32, 8, 32, 1, 4, device=dev, seed=2), 4,
                               text=TextTransformer(50, 16, 32, 1, 4, device=dev, seed=3), device=dev, seed=args.seed)
    audio, video, text, labels = _modal_batch(16, 4, args.seed, dev)

    def clf_loss(step):
        i = step % 16
        return F.mean(F.cross_entropy(clf(audio[i], video[i], text[i]), labels[i:i + 1]))
    a = _train(clf, clf.parameters(), clf_loss, args.steps, lr=2e-3)
    lm = MultiModalLM(50, 32, 48, audio_feature_dim=10, num_layers=1, device=dev, seed=args.seed)

    def lm_loss(step):
        i = step % 16
        logits = lm(text[i][:-1], audio_features=audio[i], text_prompt=text[i][:4])
        return F.mean(F.cross_entropy(logits, text[i][1:]))
    b = _train(lm, lm.parameters(), lm_loss, args.steps, lr=2e-3)
    print(f"classifier loss {a[0]:.3f} -> {a[-1]:.3f}; multimodal LM loss {b[0]:.3f} -> {b[-1]:.3f}")
    return {"clf_first": a[0], "clf_last": a[-1], "lm_first": b[0], "lm_last": b[-1]}


def demo_train_muzero_shakespeare(args) -> Dict:
    """MuZero-style world model over characters: observation window -> latent state; action = next character;
    policy learns the next character, reward = 1 for the right one, value = discounted return of the unroll."""
    from .. import ops as F
    from ..data.tokenizers import CharTokenizer
    from ..models import MuZeroLM
    dev = _dev(args)
    text = load_corpus(4000)
    tok = CharTokenizer.from_text(text)
    ids = tok.encode(text)
    v = tok.vocab_size
    model = MuZeroLM(v, 16, 32, v, num_layers=1, device=dev, seed=args.seed)
    rng = random.Random(args.seed)
    unroll, gamma = 3, 0.9

    def loss_fn(_):
        s = rng.randrange(0, len(ids) - 16 - unroll - 1)
        obs = torch.tensor(ids[s:s + 16], device=dev)
        acts = ids[s + 16:s + 16 + unroll]
        nxt = ids[s + 16:s + 16 + unroll + 1]
        u = model.unroll(obs, acts)
        total = 0
        for k in range(unroll + 1):
            target = torch.tensor([nxt[k]], device=dev)
            total = total + F.mean(F.cross_entropy(u.policies[k].reshape(1, -1), target))
            ret = sum(gamma ** j for j in range(unroll - k))
            total = total + ((u.values[k].reshape(-1) - ret) ** 2).mean()
        for r in u.rewards:
            total = total + ((r.reshape(-1) - 1.0) ** 2).mean()
        return total / (unroll + 1)
    losses = _train(model, model.parameters(), loss_fn, args.steps, lr=2e-3)
    ctx = ids[:16]
    out = []
    with torch.no_grad():
        for _ in range(12):
            pol = model.initial_inference(torch.tensor(ctx[-16:], device=dev)).policy
            nxt = int(torch.argmax(pol.reshape(-1)))
            out.append(nxt)
            ctx.append(nxt)
    print(f"world-model loss {losses[0]:.3f} -> {losses[-1]:.3f}; greedy rollout: {tok.decode(out)!r}")
    return {"loss_first": losses[0], "loss_last": losses[-1], "rollout": tok.decode(out)}


# ------------------------------------------------------------------------------------------- vision-language ---
def _tiny_llava(dev: str, seed: int, vocab: int = 50):
    from ..models import CLIPVisionConfig, CLIPVisionModel, Llama, LlamaConfig, LlamaVision
    cv = CLIPVisionModel(CLIPVisionConfig(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4,
                                          ffn_dim=64, device=dev, seed=seed))
    ll = Llama(LlamaConfig(vocab, 48, 32, 1, 4, 2, 64, device=dev, seed=seed + 1))
    return LlamaVision.build(cv, ll, seed=seed + 2)


def _captioned_images(n: int, seed: int, dev: str):
    """Image class c (brightness pattern) is captioned by the token sequence [1, 10+c, 20+c, 2]."""
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, 4, (n,), generator=g)
    patches = 0.1 * torch.randn(n, 4, 192, generator=g)
    for i, c in enumerate(labels.tolist()):
        patches[i, c] += 1.0
    caps = torch.stack([torch.tensor([1, 10 + c, 20 + c, 2]) for c in labels.tolist()])
    return patches.to(dev), caps.to(dev), labels


def demo_clip_smoke(args) -> Dict:
    """CLIP vision tower shapes: patch rows, a batch of images, CLS token first, no bias on the patch projection."""
    from ..models import CLIPVisionConfig, CLIPVisionModel
    dev = _dev(args)
    cfg = CLIPVisionConfig(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4, ffn_dim=64,
                           device=dev, seed=args.seed)
    cv = CLIPVisionModel(cfg)
    g = torch.Generator().manual_seed(args.seed)
    a = cv(torch.randn(4, 192, generator=g).to(dev))
    b = cv(torch.randn(2, 3, 16, 16, generator=g).to(dev))
    out = {"patch_rows": tuple(a.shape), "image_batch": tuple(b.shape), "num_patches": cfg.num_patches,
           "finite": bool(torch.isfinite(a).all() and torch.isfinite(b).all())}
    print(out)
    return out


def demo_train_llama_vision_demo(args) -> Dict:
    """End-to-end training of the vision tower + projector + Llama on captioned toy images."""
    dev = _dev(args)
    lv = _tiny_llava(dev, args.seed)
    patches, caps, _ = _captioned_images(8, args.seed, dev)

    def loss_fn(step):
        i = step % 8
        return lv.loss(patches[i], caps[i][:-1], caps[i][1:])
    losses = _train(lv, lv.parameters(), loss_fn, args.steps, lr=2e-3)
    out = lv.generate(patches[0], [1.0], 3, temperature=0.0)
    print(f"caption loss {losses[0]:.3f} -> {losses[-1]:.3f}; generated {out} (target {caps[0].tolist()})")
    return {"loss_first": losses[0], "loss_last": losses[-1], "generated": out}


def demo_train_llava_projector(args) -> Dict:
    """LLaVA stage 1: vision tower and language model frozen, only the projector trains."""
    dev = _dev(args)
    lv = _tiny_llava(dev, args.seed)
    patches, caps, _ = _captioned_images(8, args.seed, dev)
    frozen = [p.detach().clone() for p in lv.llama.parameters() + lv.vit.parameters()]
    params = lv.projector.parameters()

    def loss_fn(step):
        i = step % 8
        return lv.loss(patches[i], caps[i][:-1], caps[i][1:])
    losses = _train(lv, params, loss_fn, args.steps, lr=3e-3)
    same = all(torch.equal(a, b.detach()) for a, b in zip(frozen, lv.llama.parameters() + lv.vit.parameters()))
    n_proj = sum(p.numel() for p in params)
    n_all = sum(p.numel() for p in lv.parameters())
    print(f"projector-only: {n_proj} of {n_all} parameters train; loss {losses[0]:.3f} -> {losses[-1]:.3f}; "
          f"backbones untouched: {same}")
    return {"loss_first": losses[0], "loss_last": losses[-1], "frozen_untouched": bool(same),
            "trainable": n_proj, "total": n_all}


def demo_llama_llava_demo(args) -> Dict:
    """Image + prompt -> answer with the KV cache: image tokens are prefilled once, then text decodes greedily."""
    dev = _dev(args)
    lv = _tiny_llava(dev, args.seed)
    patches, _, _ = _captioned_images(1, args.seed, dev)
    t0 = time.perf_counter()
    a = lv.generate(patches[0], [1.0, 5.0], 6, temperature=0.0)
    dt = time.perf_counter() - t0
    b = lv.generate(patches[0], [1.0, 5.0], 6, temperature=0.8, top_k=5, rng=random.Random(args.seed))
    print(f"{lv.num_image_tokens} image tokens + 2 prompt tokens -> greedy {a[2:]} ({6 / dt:.1f} tok/s); sampled {b[2:]}")
    return {"image_tokens": lv.num_image_tokens, "greedy": a, "sampled": b}


def demo_llama_image_rag(args) -> Dict:
    """Image retrieval feeding a vision-language model: gallery images are embedded by the vision tower (CLS row),
    the query image's nearest neighbours come from an inner-product index, and the best hit is described."""
    from .. import vector_store as vs
    dev = _dev(args)
    lv = _tiny_llava(dev, args.seed)
    gallery, _, labels = _captioned_images(12, args.seed, dev)

    def embed(p) -> np.ndarray:
        with torch.no_grad():
            e = lv.vit(p)[0].float()
        return (e / e.norm().clamp_min(1e-9)).cpu().numpy()
    index = vs.IndexFlatIP(lv.vit.embed_dim)
    index.add(np.stack([embed(gallery[i]) for i in range(gallery.shape[0])]))
    query = gallery[3] + 0.01 * torch.randn(gallery[3].shape, generator=torch.Generator().manual_seed(7)).to(dev)
    res = index.search(embed(query)[None, :], 3)
    hits = [int(i) for i in res.ids[0]]
    answer = lv.generate(gallery[hits[0]], [1.0], 4, temperature=0.0)
    print(f"query is a noisy copy of image 3; retrieved {hits} (scores {[round(float(s), 3) for s in res.distances[0]]}); "
          f"description tokens {answer[1:]}")
    return {"hits": hits, "top_is_source": hits[0] == 3, "labels": [int(labels[i]) for i in hits], "answer": answer}


# ------------------------------------------------------------------------------------------------------ LC0 ---
def _random_lc0_weights(filters: int, blocks: int, seed: int):
    from ..models.lc0 import Lc0ConvBlock, Lc0Residual, Lc0SEUnit, Lc0Weights
    g = torch.Generator().manual_seed(seed)

    def block(cin, cout, k):
        return Lc0ConvBlock(weights=0.05 * torch.randn(cout * cin * k * k, generator=g), biases=torch.zeros(cout),
                            bn_means=torch.zeros(cout), bn_stddivs=torch.ones(cout), bn_gammas=torch.ones(cout),
                            bn_betas=torch.zeros(cout))

    def se(c, hidden):
        return Lc0SEUnit(w1=0.05 * torch.randn(c, hidden, generator=g), b1=torch.zeros(hidden),
                         w2=0.05 * torch.randn(hidden, 2 * c, generator=g), b2=torch.zeros(2 * c))
    res = [Lc0Residual(block(filters, filters, 3), block(filters, filters, 3), se(filters, max(4, filters // 4)))
           for _ in range(blocks)]
    return Lc0Weights(filters=filters, num_blocks=blocks, policy_output_planes=80, value_filters=32,
                      value_fc_units=128, input=block(112, filters, 3), residual=res,
                      policy1=block(filters, filters, 3), policy_out=block(filters, 80, 3),
                      value_conv=block(filters, 32, 1), ip1_val_w=0.05 * torch.randn(128, 32 * 64, generator=g),
                      ip1_val_b=torch.zeros(128), ip2_val_w=0.05 * torch.randn(3, 128, generator=g),
                      ip2_val_b=torch.zeros(3), wdl=3)


def demo_lc0_bench_batch(args) -> Dict:
    """ms/position of the LC0 network at batch sizes 1..32 (random weights of the 128x10 shape on a GPU, 16x2 on the
    CPU so that the command stays quick)."""
    from ..models.lc0 import START_FEN, Lc0Input, Lc0Net
    dev = _dev(args)
    filters, blocks = (128, 10) if dev == "cuda" else (16, 2)
    net = Lc0Net(_random_lc0_weights(filters, blocks, args.seed), device=dev)
    plane = Lc0Input.from_fen(START_FEN)
    out = {}
    for b in (1, 8, 32):
        batch = plane.repeat(b, 1, 1, 1)
        net.forward_planes(batch)
        t0 = time.perf_counter()
        for _ in range(max(1, args.steps)):
            pol, val = net.forward_planes(batch)
        if dev == "cuda":
            torch.cuda.synchronize()
        out[f"ms_per_position_b{b}"] = 1e3 * (time.perf_counter() - t0) / max(1, args.steps) / b
    out["policy_shape"], out["value_shape"] = tuple(pol.shape), tuple(val.shape)
    print(f"lc0 {filters}x{blocks}:", {k: (round(v, 4) if isinstance(v, float) else v) for k, v in out.items()})
    return out
