"""Inference runners and HTTP servers (reference: bin/_gpt2_hf_api_common.dart:1-461, bin/_pythia_hf_api_common.dart,
bin/_gptj_hf_api_common.dart, bin/rag_chat_server.dart:1-700, bin/llama_chat.dart).

``GenerationService`` wraps a loaded causal LM + optional tokenizer: ``run({...})`` answers the JSON contract of
``POST /generate`` (``text | tokens, maxNewTokens, temperature, topK, seed, useCache`` ->
``tokens, newTokens, text, elapsedMs``); ``serve()`` exposes ``GET /health``, ``GET /info``, ``POST /generate``.

``RagChatService`` is the chunked-RAG chat pipeline: uploaded documents are token-chunked (200 tokens, stride 100),
each chunk embedded with the LM's last-token hidden state, centred on the corpus mean and L2-normalised into an
inner-product index; a chat turn retrieves the top chunks, builds ``Context / Previous conversation / User`` prompts that
are trimmed to fit the context window, generates, and returns the answer with its sources.  Routes: ``GET /``,
``/health``, ``/status``; ``POST /upload``, ``/chat``, ``/reset``.
"""
from __future__ import annotations

import json
import os
import random
import threading
import time
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import vector_store as vs
from ..coop.http_coop import ServerHandle


# -------------------------------------------------------------------------------------------- model loading --
def load_hf_model(family: str, model_dir: str, device=None, dtype=torch.float32, preset: Optional[str] = None):
    """Build and load a causal LM from ``<model_dir>/model.safetensors`` (or a sharded index) and, when present,
    ``tokenizer.json``.  ``family``: ``gpt2``, ``distilgpt2``, ``pythia``, ``gptj`` or ``llama``; ``preset`` picks the size
    (e.g. ``medium``, ``160m``, ``8b``); without one the size is inferred from the checkpoint's tensor shapes."""
    from ..data.hf_tokenizers import HFBpeTokenizer
    from ..io.hf_loaders import GPT2HFLoader, LlamaHFLoader
    from ..io.hf_loaders_more import GPTJHFLoader, PythiaHFLoader
    from ..io.safetensors import SafeTensors
    from ..models import GPT, GPTJModel, Llama, PythiaModel
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    state = SafeTensors.load_sharded(idx) if os.path.exists(idx) else SafeTensors.load_file(
        os.path.join(model_dir, "model.safetensors"))
    kw = dict(device=device, dtype=dtype)
    fam = family.lower()
    if fam in ("gpt2", "distilgpt2"):
        layers = 1 + max(int(k.split("h.")[1].split(".")[0]) for k in state if ".h." in k or k.startswith("h."))
        d = state[next(k for k in state if k.endswith("wte.weight"))].shape[1]
        heads = {768: 12, 1024: 16, 1280: 20, 1600: 25}.get(d, max(1, d // 64))
        model = GPT(GPT2HFLoader._cfg(d, layers, heads, **kw))
        report = GPT2HFLoader.load_map(model, state)
    elif fam == "pythia":
        presets = {"14m": PythiaHFLoader.pythia_14m_config, "70m": PythiaHFLoader.pythia_70m_config,
                   "160m": PythiaHFLoader.pythia_160m_config, "410m": PythiaHFLoader.pythia_410m_config,
                   "1b": PythiaHFLoader.pythia_1b_config}
        if preset is None:
            d = state["gpt_neox.embed_in.weight"].shape[1]
            preset = {128: "14m", 512: "70m", 768: "160m", 1024: "410m", 2048: "1b"}[d]
        model = PythiaModel(presets[preset](**kw))
        report = PythiaHFLoader.load_map(model, state)
    elif fam == "gptj":
        model = GPTJModel(GPTJHFLoader.gpt_j_6b_config(**kw))
        report = GPTJHFLoader.load_map(model, state)
    elif fam == "llama":
        presets = {"1b": LlamaHFLoader.llama32_1b_config, "3b": LlamaHFLoader.llama32_3b_config,
                   "8b": LlamaHFLoader.llama31_8b_config}
        if preset is None:
            d = state["model.embed_tokens.weight"].shape[1]
            preset = {2048: "1b", 3072: "3b", 4096: "8b"}[d]
        model = Llama(presets[preset](**kw))
        report = LlamaHFLoader.load_map(model, state)
    else:
        raise ValueError(f"unknown model family {family!r}")
    tok_path = os.path.join(model_dir, "tokenizer.json")
    tok = HFBpeTokenizer.load_file(tok_path) if os.path.exists(tok_path) else None
    return model, tok, report


# --------------------------------------------------------------------------------------- generation service --
class _JsonHandler(BaseHTTPRequestHandler):
    routes: Dict[Tuple[str, str], Callable] = {}

    def log_message(self, *a):
        pass

    def _send(self, code: int, body, ctype="application/json"):
        data = body if isinstance(body, bytes) else (body if isinstance(body, str) else json.dumps(body)).encode()
        self.send_response(code)
        self.send_header("Content-Type", ctype)
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def _dispatch(self, method: str):
        path = self.path.split("?")[0]
        fn = self.routes.get((method, path))
        if fn is None:
            return self._send(404, {"error": f"not found: {method} {path}"})
        try:
            n = int(self.headers.get("Content-Length") or 0)
            code, body, *ctype = fn(self.rfile.read(n) if n else b"", self.headers)
            self._send(code, body, *(ctype or ["application/json"]))
        except Exception as e:  # handler errors become a 500 with the message, as in the reference
            self._send(500, {"error": str(e)})

    def do_GET(self):
        self._dispatch("GET")

    def do_POST(self):
        self._dispatch("POST")


def _serve(routes, host: str, port: int) -> ServerHandle:
    handler = type("Handler", (_JsonHandler,), {"routes": routes})
    httpd = ThreadingHTTPServer((host, port), handler)
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    return ServerHandle(httpd, th)


class GenerationService:
    def __init__(self, model, tokenizer=None, model_name: str = "model", model_path: str = ""):
        self.model, self.tok, self.model_name, self.model_path = model, tokenizer, model_name, model_path
        self._lock = threading.Lock()          # one generation at a time: the model holds per-call cache state

    @property
    def device_label(self) -> str:
        return str(self.model.device)

    def info(self) -> dict:
        c = self.model.config
        return {"model": self.model_name, "device": self.device_label, "embedDim": c.embed_dim,
                "numLayers": c.num_layers, "numHeads": c.num_heads, "vocabSize": c.vocab_size, "maxCtx": c.max_ctx}

    def health(self) -> dict:
        return {"status": "ok", "model": self.model_name, "device": self.device_label, "weights": self.model_path}

    def run(self, req: dict) -> Tuple[int, dict]:
        text, raw = req.get("text"), req.get("tokens") or []
        if text:
            if self.tok is None:
                return 400, {"error": 'field "text" supplied but no tokenizer.json loaded (vocab.json is decode-only)'}
            tokens = [float(i) for i in self.tok.encode(text)]
        elif raw:
            tokens = [float(t) for t in raw]
        else:
            return 400, {"error": 'either "text" or non-empty "tokens" is required'}
        max_new = int(req.get("maxNewTokens", 20))
        temperature = float(req.get("temperature", 0.0))
        top_k = int(req.get("topK", 0)) or None
        seed = req.get("seed")
        rng = random.Random(int(seed)) if seed is not None else random.Random()
        t0 = time.perf_counter()
        with self._lock:
            out = self.model.generate(tokens, max_new, temperature=temperature, top_k=top_k, rng=rng,
                                      use_cache=bool(req.get("useCache", True)))
        ids = [int(t) for t in out]
        new = ids[len(tokens):]
        return 200, {"tokens": ids, "newTokens": new, "text": self.tok.decode(ids) if self.tok else None,
                     "elapsedMs": int((time.perf_counter() - t0) * 1000)}

    def serve(self, host: str = "127.0.0.1", port: int = 0) -> ServerHandle:
        def generate(body, _h):
            try:
                req = json.loads(body.decode("utf-8") or "{}")
            except Exception:
                return 400, {"error": "request body is not valid JSON"}
            return self.run(req)
        return _serve({("GET", "/health"): lambda b, h: (200, self.health()),
                       ("GET", "/info"): lambda b, h: (200, self.info()),
                       ("POST", "/generate"): generate}, host, port)


# ------------------------------------------------------------------------------------------------ RAG chat --
CHUNK_TOKENS, CHUNK_STRIDE, TOP_K_CHUNKS = 200, 100, 4
MAX_NEW_TOKENS, HISTORY_TURNS, MAX_TOTAL_CHUNKS = 64, 3, 2000


def mean_vector(rows: Sequence[np.ndarray], d: int) -> np.ndarray:
    return np.mean(np.stack(rows), axis=0).astype(np.float32) if len(rows) else np.zeros(d, np.float32)


def center_and_normalize(v: np.ndarray, mean: np.ndarray) -> np.ndarray:
    c = np.asarray(v, dtype=np.float32) - mean
    n = float(np.linalg.norm(c))
    return c / n if n > 0 else c


def chunk_spans(n_tokens: int, size: int = CHUNK_TOKENS, stride: int = CHUNK_STRIDE) -> List[Tuple[int, int]]:
    if n_tokens <= size:
        return [(0, n_tokens)] if n_tokens else []
    spans = []
    for start in range(0, n_tokens, stride):
        end = min(start + size, n_tokens)
        spans.append((start, end))
        if end == n_tokens:
            break
    return spans


@dataclass
class _Chunk:
    id: int
    doc_id: int
    doc_title: str
    start_tok: int
    end_tok: int
    text: str
    raw_vec: np.ndarray


_INDEX_HTML = """<!doctype html><meta charset="utf-8"><title>RAG chat</title>
<body style="font-family:sans-serif;max-width:48rem;margin:2rem auto">
<h2>RAG chat</h2><input type=file id=f><button onclick="up()">Upload</button> <button onclick="rs()">Reset</button>
<pre id=log style="white-space:pre-wrap;border:1px solid #ccc;padding:1rem;min-height:12rem"></pre>
<input id=m style="width:80%"><button onclick="chat()">Send</button>
<script>
const log=t=>document.getElementById('log').textContent+=t+"\\n";
async function up(){const f=document.getElementById('f').files[0];if(!f)return;
 const r=await fetch('/upload',{method:'POST',headers:{'X-Filename':f.name},body:await f.arrayBuffer()});log(await r.text());}
async function rs(){log(await (await fetch('/reset',{method:'POST'})).text());}
async function chat(){const m=document.getElementById('m').value;log('You: '+m);
 const j=await (await fetch('/chat',{method:'POST',body:JSON.stringify({message:m})})).json();
 log('Bot: '+(j.answer||j.error));(j.sources||[]).forEach(s=>log('   ['+s.docTitle+' '+s.span+'] '+s.preview));}
</script>"""


class RagChatService:
    """``model`` needs ``hidden(tokens)`` (final hidden states), ``generate`` and ``config.{embed_dim, num_layers,
    max_ctx}``; ``tokenizer`` needs ``encode`` / ``decode``."""

    def __init__(self, model, tokenizer, arch_label: str = "gpt", preset_label: str = "custom",
                 temperature: float = 0.0, generator_top_k: Optional[int] = None, max_new_tokens: int = MAX_NEW_TOKENS):
        self.model, self.tok = model, tokenizer
        self.arch_label, self.preset_label = arch_label, preset_label
        self.temperature, self.generator_top_k, self.max_new_tokens = temperature, generator_top_k, max_new_tokens
        self.docs: List[dict] = []
        self.chunks: List[_Chunk] = []
        self.history: List[Tuple[str, str]] = []
        self.index = vs.IndexFlatIP(self.embed_dim)
        self.corpus_mean: Optional[np.ndarray] = None
        self._lock = threading.Lock()

    @property
    def embed_dim(self) -> int:
        return self.model.config.embed_dim

    def last_hidden(self, ids: Sequence[int]) -> np.ndarray:
        """Final hidden state of the last token: the chunk / query embedding."""
        ids = list(ids)[-self.model.config.max_ctx:]
        with torch.no_grad():
            was = self.model.training
            self.model.eval()
            h = self.model.hidden(torch.tensor(ids, dtype=torch.long, device=self.model.device))
            if was:
                self.model.train()
        return h.reshape(-1, h.shape[-1])[-1].float().cpu().numpy()

    def _rebuild_index(self) -> None:
        self.index = vs.IndexFlatIP(self.embed_dim)
        if not self.chunks:
            self.corpus_mean = None
            return
        raws = [c.raw_vec for c in self.chunks]
        self.corpus_mean = mean_vector(raws, self.embed_dim)
        self.index.add(np.stack([center_and_normalize(v, self.corpus_mean) for v in raws]))

    # ---- operations -------------------------------------------------------------------------------------
    def upload(self, filename: str, text: str) -> Tuple[int, dict]:
        text = text.strip()
        if not text:
            return 400, {"error": "empty document"}
        tokens = self.tok.encode(text)
        spans = chunk_spans(len(tokens))
        if len(self.chunks) + len(spans) > MAX_TOTAL_CHUNKS:
            return 400, {"error": f"index would exceed {MAX_TOTAL_CHUNKS} chunks — reset first"}
        with self._lock:
            doc_id = len(self.docs)
            for s, e in spans:
                ids = tokens[s:e]
                self.chunks.append(_Chunk(len(self.chunks), doc_id, filename, s, e, self.tok.decode(ids),
                                          self.last_hidden(ids)))
            self.docs.append({"id": doc_id, "title": filename, "numChunks": len(spans)})
            self._rebuild_index()
        return 200, {"ok": True, "docId": doc_id, "filename": filename, "chunks": len(spans),
                     "totalChunks": len(self.chunks)}

    def _prompt(self, ctx_lines: List[str], history: List[Tuple[str, str]], message: str) -> str:
        parts = []
        if ctx_lines:
            parts.append("Context:\n" + "\n".join(ctx_lines) + "\n")
        if history:
            recent = history[-HISTORY_TURNS * 2:]
            parts.append("Previous conversation:\n" + "\n".join(
                f"{'User' if role == 'user' else 'Assistant'}: {t}" for role, t in recent) + "\n")
        parts.append(f"User: {message}\nAssistant:")
        return "\n".join(parts)

    def chat(self, message: str) -> Tuple[int, dict]:
        message = (message or "").strip()
        if not message:
            return 400, {"error": "empty message"}
        t0 = time.perf_counter()
        with self._lock:
            retrieved, ctx_lines = [], []
            if self.chunks and self.corpus_mean is not None:
                q = center_and_normalize(self.last_hidden(self.tok.encode(message)), self.corpus_mean)
                res = self.index.search(q[None, :], min(TOP_K_CHUNKS, len(self.chunks)))
                for rank, (cid, score) in enumerate(zip(res.ids[0], res.distances[0])):
                    c = self.chunks[int(cid)]
                    ctx_lines.append(f"[{rank + 1}] {c.text.strip()}")
                    flat = c.text.replace("\n", " ")
                    retrieved.append({"docTitle": c.doc_title, "span": f"{c.start_tok}-{c.end_tok}",
                                      "score": float(score), "preview": flat[:140] + ("..." if len(c.text) > 140 else "")})
            max_ctx = self.model.config.max_ctx
            ids = self.tok.encode(self._prompt(ctx_lines, self.history, message))
            while len(ids) + self.max_new_tokens > max_ctx and self.history:       # drop oldest turns first
                self.history.pop(0)
                ids = self.tok.encode(self._prompt(ctx_lines, self.history, message))
            while len(ids) + self.max_new_tokens > max_ctx and len(ctx_lines) > 1:  # then the weakest sources
                ctx_lines.pop()
                retrieved.pop()
                ids = self.tok.encode(self._prompt(ctx_lines, [], message))
            ids = ids[-max(1, max_ctx - self.max_new_tokens):]
            full = self.model.generate([float(i) for i in ids], self.max_new_tokens, temperature=self.temperature,
                                       top_k=self.generator_top_k, rng=random.Random(0))
            answer = self.tok.decode([int(t) for t in full[len(ids):]])
            for stop in ("\nUser:", "\nAssistant:"):
                if stop in answer:
                    answer = answer.split(stop)[0]
            answer = answer.strip()
            self.history.append(("user", message))
            self.history.append(("assistant", answer))
        return 200, {"answer": answer, "sources": retrieved, "promptTokens": len(ids),
                     "elapsedMs": int((time.perf_counter() - t0) * 1000)}

    def reset(self) -> Tuple[int, dict]:
        with self._lock:
            self.docs.clear()
            self.chunks.clear()
            self.history.clear()
            self._rebuild_index()
        return 200, {"ok": True}

    def status(self) -> dict:
        return {"numDocs": len(self.docs), "numChunks": len(self.chunks), "historyLen": len(self.history),
                "docs": list(self.docs)}

    def health(self) -> dict:
        c = self.model.config
        return {"status": "ok", "arch": self.arch_label, "model": self.preset_label, "device": str(self.model.device),
                "embedDim": c.embed_dim, "numLayers": c.num_layers, "maxCtx": c.max_ctx}

    def serve(self, host: str = "127.0.0.1", port: int = 0) -> ServerHandle:
        def upload(body, headers):
            name = headers.get("X-Filename") or "upload.txt"
            return self.upload(name, body.decode("utf-8", errors="replace"))

        def chat(body, _h):
            try:
                msg = json.loads(body.decode("utf-8") or "{}").get("message")
            except Exception:
                return 400, {"error": "request body is not valid JSON"}
            return self.chat(msg)
        return _serve({("GET", "/"): lambda b, h: (200, _INDEX_HTML, "text/html; charset=utf-8"),
                       ("GET", "/index.html"): lambda b, h: (200, _INDEX_HTML, "text/html; charset=utf-8"),
                       ("GET", "/health"): lambda b, h: (200, self.health()),
                       ("GET", "/status"): lambda b, h: (200, self.status()),
                       ("POST", "/upload"): upload, ("POST", "/chat"): chat,
                       ("POST", "/reset"): lambda b, h: self.reset()}, host, port)


# ---------------------------------------------------------------------------------------------- llama chat --
def llama3_chat_prompt(turns: Sequence[Tuple[str, str]], system: Optional[str] = None) -> str:
    """Llama-3 chat template: ``<|begin_of_text|>`` then ``<|start_header_id|>role<|end_header_id|>\\n\\ntext<|eot_id|>``
    per turn, ending with an open assistant header."""
    out = "<|begin_of_text|>"
    if system:
        out += f"<|start_header_id|>system<|end_header_id|>\n\n{system}<|eot_id|>"
    for role, text in turns:
        out += f"<|start_header_id|>{role}<|end_header_id|>\n\n{text}<|eot_id|>"
    return out + "<|start_header_id|>assistant<|end_header_id|>\n\n"


class LlamaChat:
    """REPL-style chat over a Llama + HF tokenizer, with optional document retrieval prepended as system context."""

    def __init__(self, model, tokenizer, system: Optional[str] = None, max_new_tokens: int = 128,
                 temperature: float = 0.0, top_k: Optional[int] = None, rag: Optional[RagChatService] = None):
        self.model, self.tok, self.system = model, tokenizer, system
        self.max_new_tokens, self.temperature, self.top_k, self.rag = max_new_tokens, temperature, top_k, rag
        self.turns: List[Tuple[str, str]] = []

    def ask(self, message: str) -> str:
        system = self.system
        if self.rag is not None and self.rag.chunks:
            q = center_and_normalize(self.rag.last_hidden(self.tok.encode(message)), self.rag.corpus_mean)
            res = self.rag.index.search(q[None, :], min(TOP_K_CHUNKS, len(self.rag.chunks)))
            ctx = "\n".join(self.rag.chunks[int(i)].text.strip() for i in res.ids[0] if i >= 0)
            system = ((system + "\n\n") if system else "") + "Use this context when it helps:\n" + ctx
        self.turns.append(("user", message))
        ids = self.tok.encode(llama3_chat_prompt(self.turns, system))
        max_ctx = self.model.config.max_ctx
        while len(ids) + self.max_new_tokens > max_ctx and len(self.turns) > 1:
            self.turns.pop(0)
            ids = self.tok.encode(llama3_chat_prompt(self.turns, system))
        stop = getattr(self.tok, "llama_eot_id", None)
        out = self.model.generate([float(i) for i in ids], self.max_new_tokens, temperature=self.temperature,
                                  top_k=self.top_k, rng=random.Random(0))
        new = [int(t) for t in out[len(ids):]]
        if stop is not None and stop in new:
            new = new[:new.index(stop)]
        answer = self.tok.decode(new).strip()
        self.turns.append(("assistant", answer))
        return answer
