"""The reference's remaining demo programs as CLI commands (``python -m dart_pytorch_b200.apps <name>``).

Each function mirrors one ``bin/*.dart`` program: it builds the same kind of model on small synthetic data, trains or
runs it for ``--steps`` steps and prints what the original prints (losses, matches, retrieved passages ...).  They run
offline on the CPU in seconds and on a GPU when ``--device cuda`` is given.  Every function returns a small dict of
its results so that tests can check it.

Reference programs: bin/gpt_demo.dart, bin/lm_demo.dart, bin/aft_demo.dart, bin/seq2seq_optim_bench.dart,
bin/word2vec_demo.dart, bin/data_loaders_demo.dart, bin/tutorial.dart, bin/_aft_bench.dart, bin/vit_face_recognition_demo.dart,
bin/vit_object_detection_demo.dart, bin/vit_hungarian_matching_demo.dart, bin/vit_hungarian_batch_demo.dart,
bin/train_face_folder.dart, bin/multi_modal_demo.dart, bin/train_multimodal_demo.dart, bin/train_muzero_shakespeare.dart,
bin/train_llama_vision_demo.dart, bin/train_llava_projector.dart, bin/llama_llava_demo.dart, bin/llama_image_rag.dart,
bin/rag_learn.dart, bin/rag_demo.dart, bin/rag_gpu_demo.dart, bin/rag_qa_demo.dart, bin/qa.dart,
bin/vector_store_demo.dart, bin/gpt2_hf_demo.dart, bin/_lc0_bench_batch.dart, bin/_clip_smoke.dart.
"""
from __future__ import annotations

import math
import os
import random
import tempfile
import time
from typing import Dict, List

import torch

from .util import get_window, load_corpus


def _dev(args) -> str:
    name = getattr(args, "device", "cpu")
    if name == "auto":
        return "cuda" if torch.cuda.is_available() else "cpu"
    return name


def _train(model, params, loss_fn, steps: int, lr: float = 3e-3, clip: float = 1.0, log_every: int = 0) -> List[float]:
    """Adam + gradient clipping loop shared by the demos (reference recipe: bin/gpt_train.dart:111-131)."""
    from .. import Adam, clip_grad_norm
    opt = Adam(params, lr=lr)
    losses = []
    for step in range(steps):
        opt.zero_grad()
        loss = loss_fn(step)
        loss.backward()
        clip_grad_norm(params, clip)
        opt.step()
        losses.append(float(loss.detach()))
        if log_every and (step + 1) % log_every == 0:
            print(f"step {step + 1:4d}  loss {losses[-1]:.4f}")
    return losses


# ------------------------------------------------------------------------------------------ language models ---
def demo_gpt_demo(args) -> Dict:
    """Tiny GPT: forward shapes, a few training steps, greedy and sampled generation with and without the KV cache."""
    from .. import GPT, GPTConfig
    from ..nn.transformer import Activation
    dev = _dev(args)
    cfg = GPTConfig(vocab_size=64, max_ctx=32, embed_dim=32, num_layers=2, num_heads=4, activation=Activation.geluTanh,
                    seed=args.seed, device=dev)
    model = GPT(cfg)
    g = torch.Generator().manual_seed(args.seed)
    seq = torch.randint(0, 64, (33,), generator=g).to(dev)
    print("logits", tuple(model(seq[:-1]).shape))
    losses = _train(model, model.parameters(), lambda s: model.loss(seq[:-1], seq[1:]), args.steps)
    a = model.generate([1, 2, 3], 8, temperature=0.0, use_cache=True)
    b = model.generate([1, 2, 3], 8, temperature=0.0, use_cache=False)
    c = model.generate([1, 2, 3], 8, temperature=0.8, top_k=5, rng=random.Random(args.seed))
    print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}; greedy {a}; sampled {c}")
    return {"loss_first": losses[0], "loss_last": losses[-1], "cache_equal": a == b, "generated": a}


def demo_lm_demo(args) -> Dict:
    """TransformerLM (sinusoidal positions, untied head) on a character corpus."""
    from ..data.tokenizers import CharTokenizer
    from ..models import TransformerLM
    dev = _dev(args)
    text = load_corpus(4000)
    tok = CharTokenizer.from_text(text)
    ids = tok.encode(text)
    model = TransformerLM(tok.vocab_size, 32, 2, 4, 64, device=dev, seed=args.seed)
    rng = random.Random(args.seed)

    def loss_fn(_):
        x, y = get_window(ids, 32, rng, device=dev)
        return model.loss(x, y)
    losses = _train(model, model.parameters(), loss_fn, args.steps)
    print(f"TransformerLM loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return {"loss_first": losses[0], "loss_last": losses[-1], "vocab": tok.vocab_size}


def demo_aft_demo(args) -> Dict:
    """AFT language model (attention-free) on a character corpus."""
    from ..data.tokenizers import CharTokenizer
    from ..models import AFTLanguageModel
    dev = _dev(args)
    text = load_corpus(4000)
    tok = CharTokenizer.from_text(text)
    ids = tok.encode(text)
    model = AFTLanguageModel(tok.vocab_size, 32, 2, 32, device=dev, seed=args.seed)
    rng = random.Random(args.seed)

    def loss_fn(_):
        x, y = get_window(ids, 32, rng, device=dev)
        return model.loss(x, y)
    losses = _train(model, model.parameters(), loss_fn, args.steps)
    print(f"AFT-LM loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return {"loss_first": losses[0], "loss_last": losses[-1]}


def demo_aft_bench(args) -> Dict:
    """Step time of the AFT-LM against the attention LM of the same size (the reference's only published bench)."""
    from ..models import AFTLanguageModel, TransformerLM
    dev = _dev(args)
    out = {}
    for name, model in (("aft", AFTLanguageModel(65, 128, 2, 128, device=dev, seed=1)),
                        ("mha", TransformerLM(65, 128, 2, 4, 128, device=dev, seed=1))):
        g = torch.Generator().manual_seed(0)
        x = torch.randint(0, 65, (129,), generator=g).to(dev)
        for _ in range(3):
            _train(model, model.parameters(), lambda s: model.loss(x[:-1], x[1:]), 1)
        t0 = time.perf_counter()
        _train(model, model.parameters(), lambda s: model.loss(x[:-1], x[1:]), args.steps)
        if dev == "cuda":
            torch.cuda.synchronize()
        out[name + "_ms_per_step"] = 1e3 * (time.perf_counter() - t0) / max(1, args.steps)
    print(out)
    return out


def demo_seq2seq_optim_bench(args) -> Dict:
    """Encoder-decoder copy task trained once with SGD(momentum) and once with Adam: final losses side by side."""
    from .. import SGD, Adam, clip_grad_norm
    from ..models import EncoderDecoderTransformer
    dev = _dev(args)
    g = torch.Generator().manual_seed(args.seed)
    src = torch.randint(2, 20, (10,), generator=g).to(dev)
    tgt_in = torch.cat([torch.tensor([1], device=dev), src[:-1]])
    res = {}
    for name in ("sgd", "adam"):
        model = EncoderDecoderTransformer(20, 20, 32, 4, 1, 1, 16, 64, device=dev, seed=args.seed)
        params = model.parameters()
        opt = SGD(params, lr=0.05, momentum=0.9) if name == "sgd" else Adam(params, lr=3e-3)
        last = 0.0
        for _ in range(args.steps):
            opt.zero_grad()
            loss = model.loss(src, tgt_in, src)
            loss.backward()
            clip_grad_norm(params, 1.0)
            opt.step()
            last = float(loss.detach())
        res[name] = last
    print(f"copy task after {args.steps} steps: SGD {res['sgd']:.4f}  Adam {res['adam']:.4f}")
    return res


def demo_word2vec_demo(args) -> Dict:
    """Skip-gram with negative sampling on the toy corpus through ``Embedding`` + autograd; prints nearest words."""
    from ..nn import Embedding
    dev = _dev(args)
    words = load_corpus(6000).lower().split()
    vocab = sorted(set(words))
    index = {w: i for i, w in enumerate(vocab)}
    ids = [index[w] for w in words]
    emb_in = Embedding(len(vocab), 16, device=dev, seed=args.seed)
    emb_out = Embedding(len(vocab), 16, device=dev, seed=args.seed + 1)
    params = emb_in.parameters() + emb_out.parameters()
    rng = random.Random(args.seed)

    def loss_fn(_):
        centers, contexts, negs = [], [], []
        for _ in range(64):
            i = rng.randrange(2, len(ids) - 2)
            centers.append(ids[i])
            contexts.append(ids[i + rng.choice((-2, -1, 1, 2))])
            negs.append(rng.randrange(len(vocab)))
        c = emb_in(torch.tensor(centers, device=dev))
        pos = (c * emb_out(torch.tensor(contexts, device=dev))).sum(-1)
        neg = (c * emb_out(torch.tensor(negs, device=dev))).sum(-1)
        return -(torch.nn.functional.logsigmoid(pos) + torch.nn.functional.logsigmoid(-neg)).mean()
    losses = _train(None, params, loss_fn, args.steps, lr=0.05)
    w = emb_in.weight.detach().float()
    w = w / w.norm(dim=-1, keepdim=True).clamp_min(1e-9)
    probe = max(set(words), key=words.count)
    near = torch.topk(w @ w[index[probe]], min(4, len(vocab))).indices.tolist()
    print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}; nearest to '{probe}':", [vocab[i] for i in near])
    return {"loss_first": losses[0], "loss_last": losses[-1], "vocab": len(vocab)}


def demo_data_loaders_demo(args) -> Dict:
    """Every dataset / loader of the data package on in-memory samples (and a generated image folder)."""
    from ..data import CharTokenizer, CsvDataset, DataLoader, ListDataset, TextTokenDataset
    out = {}
    loader = DataLoader(ListDataset(list(range(10))), batch_size=4, shuffle=True, seed=args.seed)
    out["list_batches"] = [len(b) for b in loader.batches()]
    text = load_corpus(2000)
    tok = CharTokenizer.from_text(text)
    ds = TextTokenDataset.from_text(text, tok, 16)
    s = ds[0]
    out["lm_samples"] = len(ds)
    out["lm_shift_ok"] = bool(torch.equal(s.input[1:], s.target[:-1]))
    csv = CsvDataset.from_lines(["a,b,label", "1,2,0", "3,4,1", "5,6,0"], label_column=2)
    out["csv_rows"], out["csv_features"] = len(csv), int(csv[1].features.numel())
    try:
        from PIL import Image
        from ..data import ImageFolderDataset
        with tempfile.TemporaryDirectory() as root:
            g = random.Random(args.seed)
            for cls in ("alice", "bob"):
                os.makedirs(os.path.join(root, cls))
                for k in range(4):
                    px = bytes(g.randrange(256) for _ in range(16 * 16 * 3))
                    Image.frombytes("RGB", (16, 16), px).save(os.path.join(root, cls, f"{k}.png"))
            faces = ImageFolderDataset(root, 16, 8, val_split=0.25, seed=args.seed)
            out["image_classes"], out["image_train"], out["image_val"] = faces.num_classes, faces.num_train, faces.num_val
            out["patch_shape"] = tuple(faces[0].patches.shape)
    except ImportError:
        out["image_classes"] = None
    print(out)
    return out


def demo_tutorial(args) -> Dict:
    """The walk-through of the basics: tensors and autograd, a Linear regression fit, checkpoint save / load."""
    from .. import Adam, Checkpoint
    from ..nn import Linear
    dev = _dev(args)
    x = torch.tensor([[1.0, 2.0], [3.0, 4.0]], device=dev, requires_grad=True)
    y = (x * x).sum()
    y.backward()
    print("d(sum x^2)/dx =", x.grad.tolist())
    g = torch.Generator().manual_seed(args.seed)
    xs = torch.randn(64, 3, generator=g).to(dev)
    true_w = torch.tensor([[2.0, -1.0, 0.5]], device=dev)
    ys = xs @ true_w.t() + 0.3
    lin = Linear(3, 1, device=dev, seed=args.seed)
    opt = Adam(lin.parameters(), lr=0.05)
    for _ in range(max(args.steps, 1)):
        opt.zero_grad()
        loss = ((lin(xs) - ys) ** 2).mean()
        loss.backward()
        opt.step()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "lin.dptc")
        Checkpoint.save_file(lin, path)
        clone = Linear(3, 1, device=dev, seed=args.seed + 9)
        Checkpoint.load_into_file(clone, path)
    same = all(torch.equal(a.detach(), b.detach()) for a, b in zip(lin.parameters(), clone.parameters()))
    print(f"fit loss {float(loss.detach()):.5f}; weights {lin.weight.detach().flatten().tolist()}; reload identical: {same}")
    return {"grad": x.grad.tolist(), "fit_loss": float(loss.detach()), "reload_identical": bool(same)}


# ----------------------------------------------------------------------------------------------------- vision ---
def _toy_images(n: int, classes: int, size: int, seed: int, dev: str):
    """Class c = a bright square whose position depends on c, plus noise."""
    g = torch.Generator().manual_seed(seed)
    imgs = 0.1 * torch.randn(n, 3, size, size, generator=g)
    labels = torch.randint(0, classes, (n,), generator=g)
    q = size // 4
    for i, c in enumerate(labels.tolist()):
        r0, c0 = (c // 2) * 2 * q, (c % 2) * 2 * q
        imgs[i, :, r0:r0 + q, c0:c0 + q] += 1.0
    return imgs.to(dev), labels.to(dev)


def demo_vit_face_recognition_demo(args) -> Dict:
    """Triplet training of ``ViTFaceEmbedding``: same-identity pairs end closer than different-identity pairs."""
    from ..models import ViTFaceEmbedding
    dev = _dev(args)
    model = ViTFaceEmbedding(image_size=16, patch_size=8, embed_dim=32, num_layers=1, device=dev, seed=args.seed)
    imgs, labels = _toy_images(32, 4, 16, args.seed, dev)
    rng = random.Random(args.seed)
    by_class = {c: [i for i, l in enumerate(labels.tolist()) if l == c] for c in range(4)}
    ready = [c for c, idx in by_class.items() if len(idx) >= 2]

    def loss_fn(_):
        a_c = rng.choice(ready)
        n_c = rng.choice([c for c in by_class if c != a_c and by_class[c]])
        i, j = rng.sample(by_class[a_c], 2)
        k = rng.choice(by_class[n_c])
        e = model(imgs[[i, j, k]])
        return torch.relu((e[0] * e[2]).sum() - (e[0] * e[1]).sum() + 0.3)
    losses = _train(model, model.parameters(), loss_fn, args.steps, lr=1e-3)
    with torch.no_grad():
        e = model(imgs)
    sim = e @ e.t()
    same = labels[:, None] == labels[None, :]
    off = ~torch.eye(len(labels), dtype=torch.bool, device=sim.device)
    pos, neg = float(sim[same & off].mean()), float(sim[~same].mean())
    print(f"mean cosine same identity {pos:.3f}, different {neg:.3f}")
    return {"loss_last": losses[-1], "pos_sim": pos, "neg_sim": neg}


def _box_cost(pred_cls, pred_box, gt_cls, gt_box) -> List[List[int]]:
    """Integer matching cost (class probability + L1 box distance, scaled), as the detection demos build it."""
    prob = torch.softmax(pred_cls.float(), -1)
    cost = -prob[:, gt_cls] + torch.cdist(pred_box.float(), gt_box.float(), p=1)
    return (cost * 1000).round().to(torch.int64).tolist()


def demo_vit_hungarian_matching_demo(args) -> Dict:
    """Match the detector's queries to ground-truth boxes with the Hungarian algorithm (DETR-style set prediction)."""
    from ..models import ViTObjectDetector
    from ..utils import HungarianAlgorithm
    dev = _dev(args)
    det = ViTObjectDetector(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_queries=6, num_classes=3,
                            device=dev, seed=args.seed)
    img, _ = _toy_images(1, 4, 16, args.seed, dev)
    with torch.no_grad():
        cls, box = det(img[0:1])
    cls, box = cls.reshape(-1, cls.shape[-1]), box.reshape(-1, 4)
    gt_cls = torch.tensor([0, 2], device=dev)
    gt_box = torch.tensor([[0.25, 0.25, 0.2, 0.2], [0.7, 0.6, 0.3, 0.3]], device=dev)
    cost = _box_cost(cls, box, gt_cls, gt_box)                       # [queries, gts]
    square = [row + [0] * (len(cost) - len(row)) for row in cost]    # pad to square: unmatched queries cost 0
    assign = HungarianAlgorithm(square).get_assignment()
    matches = [(q, g) for q, g in enumerate(assign) if g < len(gt_cls)]
    print("query -> ground truth:", matches)
    return {"matches": matches, "num_queries": len(cost)}


def demo_vit_hungarian_batch_demo(args) -> Dict:
    """The same matching for a batch of images, then the set-prediction loss of the matched pairs."""
    from ..models import ViTObjectDetector
    from ..utils import HungarianAlgorithm
    dev = _dev(args)
    det = ViTObjectDetector(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_queries=6, num_classes=3,
                            device=dev, seed=args.seed)
    imgs, labels = _toy_images(4, 4, 16, args.seed, dev)
    total = 0.0
    counts = []
    for b in range(imgs.shape[0]):
        cls, box = det(imgs[b:b + 1])
        cls, box = cls.reshape(-1, cls.shape[-1]), box.reshape(-1, 4)
        gt_cls = torch.tensor([int(labels[b]) % 3], device=dev)
        gt_box = torch.tensor([[0.3, 0.3, 0.25, 0.25]], device=dev)
        cost = _box_cost(cls.detach(), box.detach(), gt_cls, gt_box)
        square = [row + [0] * (len(cost) - len(row)) for row in cost]
        assign = HungarianAlgorithm(square).get_assignment()
        target = torch.full((cls.shape[0],), det.num_classes, device=dev)          # default: "no object"
        l1 = torch.zeros((), device=dev)
        n = 0
        for q, g in enumerate(assign):
            if g < len(gt_cls):
                target[q] = gt_cls[g]
                l1 = l1 + (box[q] - gt_box[g]).abs().sum()
                n += 1
        total += float((torch.nn.functional.cross_entropy(cls.float(), target) + l1).detach())
        counts.append(n)
    print(f"set-prediction loss over the batch {total / imgs.shape[0]:.4f}; matched per image {counts}")
    return {"loss": total / imgs.shape[0], "matched": counts}


def demo_vit_object_detection_demo(args) -> Dict:
    """Train the detector on one-box toy images with Hungarian matching; the matched box error goes down."""
    from ..models import ViTObjectDetector
    from ..utils import HungarianAlgorithm
    dev = _dev(args)
    det = ViTObjectDetector(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_queries=4, num_classes=4,
                            device=dev, seed=args.seed)
    imgs, labels = _toy_images(16, 4, 16, args.seed, dev)
    q = 4.0 / 16.0

    def gt_of(c):
        return torch.tensor([[((c % 2) * 2 * 4 + 2) / 16.0, ((c // 2) * 2 * 4 + 2) / 16.0, q, q]], device=dev)
    errs = []

    def loss_fn(step):
        b = step % imgs.shape[0]
        cls, box = det(imgs[b:b + 1])
        cls, box = cls.reshape(-1, cls.shape[-1]), box.reshape(-1, 4)
        c = int(labels[b])
        gt_cls, gt_box = torch.tensor([c], device=dev), gt_of(c)
        cost = _box_cost(cls.detach(), box.detach(), gt_cls, gt_box)
        assign = HungarianAlgorithm([row + [0] * (len(cost) - 1) for row in cost]).get_assignment()
        qi = assign.index(0)
        target = torch.full((cls.shape[0],), det.num_classes, device=dev)
        target[qi] = c
        l1 = (box[qi] - gt_box[0]).abs().sum()
        errs.append(float(l1.detach()))
        return torch.nn.functional.cross_entropy(cls.float(), target) + 5.0 * l1
    _train(det, det.parameters(), loss_fn, args.steps, lr=2e-3)
    k = max(1, len(errs) // 4)
    first, last = sum(errs[:k]) / k, sum(errs[-k:]) / k
    print(f"matched box L1 error {first:.3f} -> {last:.3f}")
    return {"box_err_first": first, "box_err_last": last}


def demo_train_face_folder(args) -> Dict:
    """Triplet training from an image folder (``root/<identity>/*.png``); generates a toy folder when none is given."""
    from ..data import ImageFolderDataset
    from ..models import ViTFaceEmbedding
    from PIL import Image
    dev = _dev(args)
    tmp = None
    root = getattr(args, "root", "") or ""
    if not root:
        tmp = tempfile.TemporaryDirectory()
        root = tmp.name
        g = random.Random(args.seed)
        for ci, cls in enumerate(("ann", "ben", "cat")):
            os.makedirs(os.path.join(root, cls))
            base = [g.randrange(256) for _ in range(3)]
            for k in range(5):
                px = bytes(min(255, max(0, base[i % 3] + g.randrange(-30, 30))) for i in range(16 * 16 * 3))
                Image.frombytes("RGB", (16, 16), px).save(os.path.join(root, cls, f"{k}.png"))
    ds = ImageFolderDataset(root, 16, 8, val_split=0.2, device=dev, seed=args.seed)
    model = ViTFaceEmbedding(image_size=16, patch_size=8, embed_dim=32, num_layers=1, device=dev, seed=args.seed)

    def loss_fn(_):
        t = ds.sample_triplet()
        a, p, n = model(t.anchor), model(t.positive), model(t.negative)
        return torch.relu((a * n).sum() - (a * p).sum() + 0.3)
    losses = _train(model, model.parameters(), loss_fn, args.steps, lr=1e-3)
    if tmp is not None:
        tmp.cleanup()
    print(f"identities {ds.num_classes}, train {ds.num_train}, val {ds.num_val}; triplet loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return {"classes": ds.num_classes, "loss_first": losses[0], "loss_last": losses[-1]}
