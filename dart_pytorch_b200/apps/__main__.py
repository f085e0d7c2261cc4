"""Command-line entry points: ``python -m dart_pytorch_b200.apps <command> [options]``
(reference: the ``bin/`` programs — trainers ``gpt_train``, ``train_char_lm``, ``shakespeare_{gpt,gpt_big,
transformer_lm,aft,moe}``, ``vit_demo``, ``train_muzero_lm_demo``; runners ``gpt2`` / ``distilgpt2`` / ``pythia`` /
``gptj`` / ``llama_chat`` with ``--serve``; ``rag_chat_server``; ``lc0_demo``; cooperative training ``coop_train_phase0``,
``coop_coordinator``, ``coop_worker``, ``coop_peer``; vector tools ``demo_faiss``, ``bench_faiss``, ``faiss_describe``,
``faiss_strip``; and every remaining demo / debug program — ``gpt_demo``, ``lm_demo``, ``aft_demo``, ``aft_bench``,
``seq2seq_optim_bench``, ``word2vec_demo``, ``data_loaders_demo``, ``tutorial``, the ``vit_*`` demos,
``train_face_folder``, ``multi_modal_demo``, ``train_multimodal_demo``, ``train_muzero_shakespeare``,
``train_llama_vision_demo``, ``train_llava_projector``, ``llama_llava_demo``, ``llama_image_rag``, ``clip_smoke``,
``lc0_bench_batch``, ``rag_learn``, ``rag_demo``, ``rag_gpu_demo``, ``rag_qa_demo``, ``qa``, ``vector_store_demo``,
``gpt2_hf_demo``, the ``vector_*_demo`` programs, ``bug_repro``, ``gpt2_debug``, ``prep_coco_pairs``, ``hello`` —
from the ``demos*.py`` modules, registered by ``all_demos()``).
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time

import torch


def _device(name: str):
    if name == "auto":
        return "cuda" if torch.cuda.is_available() else "cpu"
    return name


def _lm_trainer(args, build):
    """Shared loop of the language-model demos: tokenizer -> model -> Adam + warmup/cosine + clip -> checkpoint ->
    sample (reference call stack: bin/gpt_train.dart:38-190)."""
    from .. import optim
    from ..data.tokenizers import BpeTokenizer, CharTokenizer
    from ..io.dptc import Checkpoint
    from .util import get_window, load_corpus, param_scalar_count
    dev = _device(args.device)
    text = load_corpus(args.max_chars, args.corpus)
    tok = BpeTokenizer.train(text, args.bpe_vocab) if args.bpe_vocab else CharTokenizer.from_text(text)
    ids = [int(i) for i in tok.encode(text)]
    vocab = tok.vocab_size
    model = build(vocab, dev)
    print(f"{args.command}: vocab {vocab}, {param_scalar_count(model.parameters())} parameters on {dev}")
    opt = optim.Adam(model.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    sched = optim.LinearWarmupCosineDecay(opt, warmup_steps=max(1, args.steps // 10), total_steps=args.steps,
                                          max_lr=args.lr, min_lr=args.lr * 0.1)
    rng = random.Random(args.seed)
    per_sample = False
    t0 = time.perf_counter()
    for step in range(1, args.steps + 1):
        xs, ys = zip(*(get_window(ids, args.block, rng, device=dev) for _ in range(args.batch)))
        x, y = torch.stack(xs), torch.stack(ys)
        if args.batch == 1:
            x, y = x[0], y[0]
        opt.zero_grad()
        if per_sample:
            loss = sum(model.loss(a, b).reshape(()) for a, b in zip(xs, ys)) / len(xs)
        else:
            try:
                loss = model.loss(x, y)
            except ValueError:              # families that keep the reference's one-sequence contract
                per_sample = True
                loss = sum(model.loss(a, b).reshape(()) for a, b in zip(xs, ys)) / len(xs)
        loss.backward()
        norm = optim.clip_grad_norm(model.parameters(), 1.0)
        opt.step()
        sched.step()
        if hasattr(model, "update_routing_bias"):
            model.update_routing_bias()
        if step == 1 or step % max(1, args.steps // 10) == 0:
            print(f"  step {step:5d}  loss {float(loss.detach()):.4f}  |g| {float(norm):.3f}  lr {opt.lr:.2e}")
    print(f"trained {args.steps} steps in {time.perf_counter() - t0:.1f}s")
    if args.save:
        Checkpoint.save_file(model, args.save)
        print(f"saved {args.save}")
    if hasattr(model, "generate") and args.sample > 0:
        prompt = [float(i) for i in tok.encode(args.prompt)] or [0.0]
        out = model.generate(prompt, args.sample, temperature=args.temperature, top_k=args.top_k,
                             rng=random.Random(args.seed))
        print(tok.decode([int(t) for t in out]))
    return model


def _add_lm_args(p, block=32, dim=64, layers=2, heads=4, steps=200, lr=3e-3):
    p.add_argument("--device", default="auto")
    p.add_argument("--corpus", default=None, help="text file (default: data/tiny_shakespeare.txt or the toy corpus)")
    p.add_argument("--max-chars", type=int, default=None)
    p.add_argument("--bpe-vocab", type=int, default=0, help="train a byte-level BPE of this size (0: characters)")
    p.add_argument("--block", type=int, default=block)
    p.add_argument("--dim", type=int, default=dim)
    p.add_argument("--layers", type=int, default=layers)
    p.add_argument("--heads", type=int, default=heads)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--steps", type=int, default=steps)
    p.add_argument("--lr", type=float, default=lr)
    p.add_argument("--weight-decay", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--save", default="")
    p.add_argument("--prompt", default="The ")
    p.add_argument("--sample", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-k", type=int, default=20)


def cmd_gpt_train(args):
    from ..models import GPT, GPTConfig
    return _lm_trainer(args, lambda v, dev: GPT(GPTConfig(vocab_size=v, max_ctx=args.block, embed_dim=args.dim,
                                                          num_layers=args.layers, num_heads=args.heads, device=dev,
                                                          seed=args.seed)))


def cmd_transformer_lm(args):
    from ..models import TransformerLM
    return _lm_trainer(args, lambda v, dev: TransformerLM(v, args.dim, args.layers, args.heads, args.block, device=dev,
                                                          seed=args.seed))


def cmd_aft(args):
    from ..models import AFTLanguageModel
    return _lm_trainer(args, lambda v, dev: AFTLanguageModel(v, args.dim, args.layers, args.block, device=dev,
                                                             seed=args.seed))


def cmd_moe(args):
    from ..models import MoELanguageModel
    return _lm_trainer(args, lambda v, dev: MoELanguageModel(v, args.dim, args.layers, args.heads, args.block,
                                                             device=dev, seed=args.seed))


def cmd_llama_train(args):
    from ..models.llama import Llama, LlamaConfig
    return _lm_trainer(args, lambda v, dev: Llama(LlamaConfig(v, args.block, args.dim, args.layers, args.heads,
                                                              max(1, args.heads // 2), args.dim * 3, device=dev,
                                                              seed=args.seed)))


def cmd_vit_demo(args):
    """Synthetic two-class image task through ``ViTClassifier`` (reference: bin/vit_demo.dart)."""
    from .. import ops as F
    from .. import optim
    from ..models import ViTClassifier
    dev = _device(args.device)
    model = ViTClassifier(image_size=16, patch_size=4, embed_dim=32, num_layers=2, num_heads=4, num_classes=2,
                          device=dev)
    opt = optim.Adam(model.parameters(), lr=3e-3)
    g = torch.Generator().manual_seed(0)
    for step in range(1, args.steps + 1):
        y = torch.randint(0, 2, (16,), generator=g)
        x = torch.randn(16, 3, 16, 16, generator=g) + y.view(-1, 1, 1, 1).float() * 0.8
        opt.zero_grad()
        loss = F.mean(F.cross_entropy(model(x.to(dev)), y.to(dev)))
        loss.backward()
        opt.step()
        if step % max(1, args.steps // 5) == 0:
            print(f"  step {step:4d}  loss {float(loss):.4f}")


def cmd_muzero(args):
    """Next-character MuZeroLM: the policy predicts the next token, the dynamics roll the latent forward
    (reference: bin/train_muzero_lm_demo.dart)."""
    from .. import ops as F
    from .. import optim
    from ..data.tokenizers import CharTokenizer
    from ..models import MuZeroLM
    from .util import load_corpus
    text = load_corpus(2000, None)
    tok = CharTokenizer.from_text(text)
    ids = [int(i) for i in tok.encode(text)]
    dev = _device(args.device)
    model = MuZeroLM(tok.vocab_size, 16, 32, tok.vocab_size, device=dev)
    opt = optim.Adam(model.parameters(), lr=3e-3)
    rng = random.Random(0)
    for step in range(1, args.steps + 1):
        s = rng.randrange(len(ids) - 20)
        obs, actions = ids[s:s + 16], ids[s + 16:s + 19]
        u = model.unroll(torch.tensor(obs, device=dev), actions[:-1])
        opt.zero_grad()
        loss = sum(F.mean(F.cross_entropy(p, torch.tensor([a], device=dev))) for p, a in zip(u.policies, actions))
        loss.backward()
        opt.step()
        if step % max(1, args.steps // 5) == 0:
            print(f"  step {step:4d}  loss {float(loss):.4f}")


def cmd_hf_runner(args):
    """``gpt2`` / ``distilgpt2`` / ``pythia`` / ``gptj`` / ``llama`` runner: one-shot generation or ``--serve``."""
    from .servers import GenerationService, load_hf_model
    dev = _device(args.device)
    dtype = torch.bfloat16 if (args.bf16 and dev == "cuda") else torch.float32
    t0 = time.perf_counter()
    model, tok, report = load_hf_model(args.family, args.model_dir, device=dev, dtype=dtype, preset=args.preset)
    print(f"loaded {report.consumed_count} tensors in {time.perf_counter() - t0:.1f}s "
          f"({len(report.unused_keys)} unused keys)")
    svc = GenerationService(model, tok, model_name=args.family, model_path=args.model_dir)
    if args.serve:
        h = svc.serve(args.host, args.port)
        print(f"{args.family} ({svc.device_label}) listening on {h.url}\n  GET  /health\n  GET  /info\n  POST /generate")
        try:
            while True:
                time.sleep(3600)
        except KeyboardInterrupt:
            h.close()
        return
    req = {"maxNewTokens": args.max_new_tokens, "temperature": args.temperature, "topK": args.top_k, "seed": args.seed,
           "useCache": not args.no_cache}
    if args.tokens:
        req["tokens"] = [int(t) for t in args.tokens.split(",")]
    else:
        req["text"] = args.prompt
    code, out = svc.run(req)
    print(json.dumps(out, indent=1))
    if out.get("elapsedMs"):
        print(f"{len(out['newTokens']) / (out['elapsedMs'] / 1000):.1f} tok/s")


def cmd_rag_chat_server(args):
    from ..coop.lm_factory import build_coop_lm
    from ..data.tokenizers import CharTokenizer
    from .servers import RagChatService, load_hf_model
    from .util import load_corpus
    dev = _device(args.device)
    if args.model_dir:
        model, tok, _ = load_hf_model(args.family, args.model_dir, device=dev)
        label = args.family
    else:                                   # self-contained demo backend: a small character GPT
        tok = CharTokenizer.from_text(load_corpus(None, None) + "".join(chr(c) for c in range(32, 127)))
        model = build_coop_lm("gpt", "small", tok.vocab_size, device=dev).module
        label = "char-gpt (untrained)"
    svc = RagChatService(model, tok, arch_label=args.family, preset_label=label)
    h = svc.serve(args.host, args.port)
    print(f"rag chat server on {h.url}  (GET /, /health, /status; POST /upload, /chat, /reset)")
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        h.close()


def cmd_llama_chat(args):
    from .servers import LlamaChat, load_hf_model
    model, tok, _ = load_hf_model("llama", args.model_dir, device=_device(args.device),
                                  dtype=torch.bfloat16 if args.bf16 else torch.float32, preset=args.preset)
    chat = LlamaChat(model, tok, system=args.system, max_new_tokens=args.max_new_tokens)
    print("llama chat — empty line to quit")
    while True:
        try:
            line = input("> ").strip()
        except EOFError:
            break
        if not line:
            break
        print(chat.ask(line))


def cmd_lc0_demo(args):
    from ..models.lc0 import START_FEN, Lc0Input, Lc0Net, Lc0Reader
    w = Lc0Reader.read_file(args.weights)
    net = Lc0Net(w, device=_device(args.device))
    print(f"lc0: {w.filters} filters x {w.num_blocks} blocks, policy planes {w.policy_output_planes}, wdl {w.wdl}")
    planes = [Lc0Input.from_fen(args.fen or START_FEN)] * args.batch
    net.call_batch(planes[:1])
    t0 = time.perf_counter()
    outs = net.call_batch(planes)
    dt = time.perf_counter() - t0
    print(f"value {outs[0].scalar_value:+.4f}; {dt * 1e3 / args.batch:.3f} ms/position at batch {args.batch}")


def cmd_coop(args):
    from ..coop import http_coop as C
    if args.command == "coop_train_phase0":
        hist = C.train_phase0(args.replicas, args.rounds, args.local_steps, arch=args.arch, model=args.model)
        print("round  coop    baseline")
        for i, (a, b) in enumerate(zip(hist["coop"], hist["baseline"])):
            print(f"{i:5d}  {a:.4f}  {b:.4f}")
    elif args.command == "coop_coordinator":
        co = C.Coordinator(arch=args.arch, model=args.model, target=args.target)
        h = co.serve(args.host, args.port)
        print(f"coordinator on {h.url} (GET /config /corpus /checkpoint /status; POST /submit)")
        try:
            while True:
                time.sleep(3600)
        except KeyboardInterrupt:
            h.close()
    elif args.command == "coop_worker":
        w = C.Worker(args.url, args.worker_id, args.shard_index, args.num_shards, local_steps=args.local_steps)
        for _ in range(args.rounds):
            print(w.run_round())
    else:
        p = C.Peer(args.peers.split(",") if args.peers else [], arch=args.arch, model=args.model,
                   gossip_every=args.gossip_every)
        h = p.serve(args.host, args.port)
        print(f"peer on {h.url}")
        time.sleep(args.warmup_secs)
        for _ in range(args.rounds):
            print(p.run_round())
        h.close()


def cmd_vector(args):
    import numpy as np
    from .. import vector_store as vs
    if args.command == "faiss_describe":
        # header-only probe (37 bytes of a plain file) as the reference tool does; --deep decodes and walks the index
        info = vs.probe_faiss_index_file(args.path)
        rec = {"path": args.path, "fourcc": info.fourcc_str, "kind": info.kind.value, "d": info.d,
               "ntotal": info.ntotal, "metric": None if info.metric is None else info.metric.name,
               "isTrained": info.is_trained, "codeSize": info.code_size}
        if info.tuning is not None:
            t = info.tuning
            rec["inner"] = info.inner.fourcc_str
            rec["tuning"] = {"createdAt": t.created_at.isoformat(), "metric": t.metric.name,
                             "chosen": t.chosen_param_value,
                             "points": [{"value": p.param_value, "label": p.param_label, "recall": p.recall,
                                         "meanUs": p.mean_us} for p in t.points]}
        print(json.dumps(rec) if args.json else "\n".join(f"{k}: {v}" for k, v in rec.items()))
        if args.deep:
            data = open(args.path, "rb").read()
            print(vs.faiss_describe(vs.strip_tuning_wrapper(data) if vs.is_tuned_faiss_blob(data) else data))
        return rec
    if args.command == "faiss_strip":
        data = open(args.path, "rb").read()
        out = args.out or (args.path[:-6] if args.path.endswith(".faiss") else args.path) + ".stripped.faiss"
        # default: remove the tuning-metadata wrapper so that upstream FAISS can read the file;
        # --vectors instead empties the stored vectors while keeping trained state
        open(out, "wb").write(vs.faiss_strip(data) if args.vectors else vs.strip_tuning_wrapper(data))
        print(f"wrote {out}")
        return out
    rng = np.random.default_rng(0)
    cent = rng.standard_normal((32, args.d)).astype(np.float32) * 3
    x = (cent[rng.integers(32, size=args.n)] + rng.standard_normal((args.n, args.d))).astype(np.float32)
    q = (cent[rng.integers(32, size=args.nq)] + rng.standard_normal((args.nq, args.d))).astype(np.float32)
    flat = vs.IndexFlat(args.d)
    flat.add(x)
    truth = flat.search(q, args.k)
    rows = [vs.bench_index(flat, q, args.k, truth, label="Flat")]
    for desc in args.indexes.split(";"):
        ix = vs.index_factory(args.d, desc)
        ix.train(x)
        ix.add(x)
        rows.append(vs.bench_index(ix, q, args.k, truth, label=desc))
    print(vs.format_bench_table(rows))
    if args.csv:
        open(args.csv, "w").write(vs.to_bench_csv(rows))


DEMO_OPTIONS = {      # per-demo extra flags with their defaults (every demo also takes --device --steps --seed --model-dir)
    "train_face_folder": {"root": ""},
    "qa": {"corpus": None, "out": None, "question": None, "chunk_words": 120, "overlap_words": 20},
    "gpt2_hf_demo": {"weights": None},
    "gpt2_debug": {"weights": None},
    "prep_coco_pairs": {"json": None, "images": None, "out": None, "n": 200},
    "vector_index_benchmark_demo": {"n": 2000},
    "vector_dedup_demo": {"threshold": None},
}


def all_demos():
    """``{command name: function}`` for every ``demo_*`` function of the demo modules."""
    from . import demos, demos_mm, demos_rag, demos_vector
    out = {}
    for mod in (demos, demos_mm, demos_rag, demos_vector):
        for attr in sorted(dir(mod)):
            if attr.startswith("demo_") and getattr(getattr(mod, attr), "__module__", None) == mod.__name__:
                out[attr[len("demo_"):]] = getattr(mod, attr)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m dart_pytorch_b200.apps")
    sub = ap.add_subparsers(dest="command", required=True)
    for name, fn, kw in (("gpt_train", cmd_gpt_train, {}), ("train_char_lm", cmd_gpt_train, {}),
                         ("shakespeare_gpt", cmd_gpt_train, dict(block=64, dim=128, layers=4, heads=8)),
                         ("shakespeare_gpt_big", cmd_gpt_train, dict(block=128, dim=256, layers=6, heads=8, lr=1e-3)),
                         ("shakespeare_transformer_lm", cmd_transformer_lm, dict(block=64, dim=128, layers=4, heads=8)),
                         ("shakespeare_aft", cmd_aft, dict(block=64, dim=128, layers=2)),
                         ("shakespeare_moe", cmd_moe, dict(block=64, dim=128, layers=2, heads=8)),
                         ("llama_train", cmd_llama_train, {})):
        p = sub.add_parser(name)
        _add_lm_args(p, **kw)
        p.set_defaults(fn=fn)
    for name, fn in (("vit_demo", cmd_vit_demo), ("train_muzero_lm_demo", cmd_muzero)):
        p = sub.add_parser(name)
        p.add_argument("--device", default="auto")
        p.add_argument("--steps", type=int, default=50)
        p.set_defaults(fn=fn)
    for fam in ("gpt2", "distilgpt2", "pythia", "gptj", "llama"):
        p = sub.add_parser(fam)
        p.add_argument("model_dir")
        p.add_argument("--device", default="auto")
        p.add_argument("--bf16", action="store_true")
        p.add_argument("--preset", default=None)
        p.add_argument("--prompt", default="Hello, my name is")
        p.add_argument("--tokens", default="")
        p.add_argument("--max-new-tokens", type=int, default=20)
        p.add_argument("--temperature", type=float, default=0.0)
        p.add_argument("--top-k", type=int, default=0)
        p.add_argument("--seed", type=int, default=None)
        p.add_argument("--no-cache", action="store_true")
        p.add_argument("--serve", action="store_true")
        p.add_argument("--host", default="127.0.0.1")
        p.add_argument("--port", type=int, default=8080)
        p.set_defaults(fn=cmd_hf_runner, family=fam)
    p = sub.add_parser("rag_chat_server")
    p.add_argument("--model-dir", default="")
    p.add_argument("--family", default="gpt2")
    p.add_argument("--device", default="auto")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8090)
    p.set_defaults(fn=cmd_rag_chat_server)
    p = sub.add_parser("llama_chat")
    p.add_argument("model_dir")
    p.add_argument("--device", default="auto")
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--preset", default=None)
    p.add_argument("--system", default=None)
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.set_defaults(fn=cmd_llama_chat)
    p = sub.add_parser("lc0_demo")
    p.add_argument("weights")
    p.add_argument("--fen", default="")
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--device", default="auto")
    p.set_defaults(fn=cmd_lc0_demo)
    for name in ("coop_train_phase0", "coop_coordinator", "coop_worker", "coop_peer"):
        p = sub.add_parser(name)
        p.add_argument("--arch", default="gpt")
        p.add_argument("--model", default="tiny")
        p.add_argument("--rounds", type=int, default=3)
        p.add_argument("--local-steps", type=int, default=30)
        p.add_argument("--replicas", type=int, default=2)
        p.add_argument("--target", type=int, default=2)
        p.add_argument("--host", default="127.0.0.1")
        p.add_argument("--port", type=int, default=0)
        p.add_argument("--url", default="http://127.0.0.1:8000")
        p.add_argument("--worker-id", default="w0")
        p.add_argument("--shard-index", type=int, default=0)
        p.add_argument("--num-shards", type=int, default=1)
        p.add_argument("--peers", default="")
        p.add_argument("--gossip-every", type=int, default=1)
        p.add_argument("--warmup-secs", type=float, default=0.0)
        p.set_defaults(fn=cmd_coop)
    for name in ("demo_faiss", "bench_faiss"):
        p = sub.add_parser(name)
        p.add_argument("--d", type=int, default=32)
        p.add_argument("--n", type=int, default=5000)
        p.add_argument("--nq", type=int, default=50)
        p.add_argument("--k", type=int, default=10)
        p.add_argument("--indexes", default="IVF32,Flat;HNSW16;PQ8;SQ8")
        p.add_argument("--csv", default="")
        p.set_defaults(fn=cmd_vector)
    p = sub.add_parser("faiss_describe")
    p.add_argument("path")
    p.add_argument("--json", action="store_true")
    p.add_argument("--deep", action="store_true")
    p.set_defaults(fn=cmd_vector)
    p = sub.add_parser("faiss_strip")
    p.add_argument("path")
    p.add_argument("out", nargs="?", default=None)
    p.add_argument("--vectors", action="store_true")
    p.set_defaults(fn=cmd_vector)
    for name, fn in all_demos().items():
        p = sub.add_parser(name, description=(fn.__doc__ or "").strip())
        p.add_argument("--device", default="auto")
        p.add_argument("--steps", type=int, default=60)
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--model-dir", dest="model_dir", default=None,
                       help="downloaded Hugging Face model directory for the demos that can use pretrained weights")
        for flag, default in DEMO_OPTIONS.get(name, {}).items():
            kind = float if flag == "threshold" else (type(default) if default is not None else str)
            p.add_argument("--" + flag.replace("_", "-"), dest=flag, default=default, type=kind)
        p.set_defaults(fn=fn)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    main()
