"""Cooperative training over HTTP: coordinator (star topology), worker and gossip peer
(reference: bin/coop_coordinator.dart:127-316, bin/coop_worker.dart:153-238, bin/coop_peer.dart:185-345).

Protocol of the coordinator (same routes, headers, status codes and JSON keys as the reference):
  GET  /config      {"version","arch","model","corpus","vocab","maxLen","seed","target"}
  GET  /corpus      the corpus text
  GET  /checkpoint  current global DPTC bytes, header ``X-Coop-Round``
  GET  /status      {"round","queueSize","target","workersSeen"}
  POST /submit      DPTC bytes with ``X-Coop-Worker-Id``, ``X-Coop-Round``, ``X-Coop-Local-Steps``
                    409 when the round is stale; 400 when the blob does not load into a scratch model; once ``target``
                    submissions are queued they are averaged, weighted by local steps, together with the current global
                    at the median weight, and the round advances.
Peers serve GET /health and GET /checkpoint and, every ``gossip_every`` rounds, average 50/50 with one random peer;
connect / read failures are logged and skipped.  Everything here is CPU-side control plane; the training steps a
worker runs use whatever device its model lives on.
"""
from __future__ import annotations

import json
import random
import threading
import time
import urllib.error
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..io.dptc import Checkpoint
from ..optim import Adam, clip_grad_norm
from .lm_factory import Arch, CoopLM, arch_to_string, build_coop_lm, parse_arch
from .param_avg import average_checkpoints
from .shard import CharVocab, K_TOY_CORPUS, sample_window, shard_slice


def _median(xs: Sequence[float]) -> float:
    if not xs:
        return 1.0
    s = sorted(xs)
    mid = len(s) // 2
    return s[mid] if len(s) % 2 else 0.5 * (s[mid - 1] + s[mid])


class Coordinator:
    """In-memory coordinator state + request handling; ``serve()`` wraps it in an HTTP server thread."""

    def __init__(self, arch="gpt", model: str = "tiny", corpus_name: str = "toy", text: Optional[str] = None,
                 seed: int = 0, target: int = 2, device=None):
        self.arch, self.model, self.corpus_name, self.seed, self.target, self.device = parse_arch(arch) if \
            isinstance(arch, str) else arch, model, corpus_name, seed, target, device
        self.text = K_TOY_CORPUS if text is None else text
        self.vocab = CharVocab.from_text(self.text)
        self.global_lm = self._build()
        self.global_bytes = Checkpoint.save_bytes(self.global_lm.module)
        self.round = 0
        self.workers_seen = set()
        self.queue: List[Tuple[str, int, bytes]] = []
        self.lock = threading.Lock()
        self.log: List[str] = []

    def _build(self) -> CoopLM:
        return build_coop_lm(self.arch, self.model, self.vocab.size, device=self.device, seed=self.seed)

    def config_json(self) -> str:
        return json.dumps({"version": 1, "arch": arch_to_string(self.arch), "model": self.model,
                           "corpus": self.corpus_name, "vocab": self.vocab.itos, "maxLen": self.global_lm.max_len,
                           "seed": self.seed, "target": self.target})

    def status(self) -> dict:
        return {"round": self.round, "queueSize": len(self.queue), "target": self.target,
                "workersSeen": sorted(self.workers_seen)}

    def submit(self, worker_id: str, sub_round: int, local_steps: int, body: bytes) -> Tuple[int, dict]:
        """Returns ``(http_status, json_body)``."""
        with self.lock:
            if sub_round != self.round:
                return 409, {"accepted": False, "reason": "stale round", "workerRound": sub_round,
                             "currentRound": self.round}
            try:
                Checkpoint.load_into_bytes(self._build().module, body)
            except Exception as e:  # any malformed / mismatched blob is the submitter's fault
                return 400, {"accepted": False, "reason": f"invalid checkpoint: {e}"}
            self.queue.append((worker_id, local_steps, body))
            self.workers_seen.add(worker_id)
            aggregated = False
            if len(self.queue) >= self.target:
                blobs = [b for _, _, b in self.queue]
                weights = [float(s) for _, s, _ in self.queue]
                blobs.append(self.global_bytes)
                weights.append(_median(weights))
                self.global_bytes = average_checkpoints(blobs, weights)
                self.round += 1
                self.log.append(f"round {self.round} aggregated {len(self.queue)} updates "
                                f"(workers: {sorted({w for w, _, _ in self.queue})})")
                self.queue.clear()
                aggregated = True
            return 200, {"accepted": True, "round": self.round, "queueSize": len(self.queue),
                         "aggregated": aggregated}

    def serve(self, host: str = "127.0.0.1", port: int = 0) -> "ServerHandle":
        coord = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):  # quiet
                pass

            def _send(self, code, body: bytes, ctype: str, extra: Optional[Dict[str, str]] = None):
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                for k, v in (extra or {}).items():
                    self.send_header(k, v)
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                try:
                    if self.path == "/config":
                        self._send(200, coord.config_json().encode(), "application/json")
                    elif self.path == "/corpus":
                        self._send(200, coord.text.encode("utf-8"), "text/plain; charset=utf-8")
                    elif self.path == "/checkpoint":
                        with coord.lock:
                            blob, rnd = coord.global_bytes, coord.round
                        self._send(200, blob, "application/octet-stream", {"X-Coop-Round": str(rnd)})
                    elif self.path == "/status":
                        self._send(200, json.dumps(coord.status()).encode(), "application/json")
                    else:
                        self._send(404, b"unknown route", "text/plain")
                except Exception:
                    self._send(500, b"", "text/plain")

            def do_POST(self):
                try:
                    if self.path != "/submit":
                        self._send(404, b"unknown route", "text/plain")
                        return
                    n = int(self.headers.get("Content-Length", "0"))
                    body = self.rfile.read(n)

                    def as_int(name, default):
                        try:
                            return int(self.headers.get(name, default))
                        except ValueError:
                            return int(default)
                    code, js = coord.submit(self.headers.get("X-Coop-Worker-Id", "?"), as_int("X-Coop-Round", "-1"),
                                            as_int("X-Coop-Local-Steps", "1"), body)
                    self._send(code, json.dumps(js).encode(), "application/json")
                except Exception:
                    self._send(500, b"", "text/plain")

        httpd = ThreadingHTTPServer((host, port), Handler)
        th = threading.Thread(target=httpd.serve_forever, daemon=True)
        th.start()
        return ServerHandle(httpd, th)


class ServerHandle:
    def __init__(self, httpd, thread):
        self.httpd, self.thread = httpd, thread

    @property
    def url(self) -> str:
        host, port = self.httpd.server_address[:2]
        return f"http://{host}:{port}"

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()


def _http(method: str, url: str, data: Optional[bytes] = None, headers: Optional[Dict[str, str]] = None,
          timeout: float = 30.0) -> Tuple[int, Dict[str, str], bytes]:
    req = urllib.request.Request(url, data=data, method=method, headers=headers or {})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, dict(r.headers), r.read()
    except urllib.error.HTTPError as e:
        return e.code, dict(e.headers), e.read()


def local_steps(lm: CoopLM, opt, ids: Sequence[float], block_size: int, steps: int, rng: random.Random,
                clip: float = 1.0) -> float:
    """K local steps: zeroGrad, sample a window, loss, backward, clipGradNorm, step.  Returns the last loss."""
    last = float("nan")
    for _ in range(steps):
        opt.zero_grad()
        x, y = sample_window(ids, block_size, rng, device=lm.module.device)
        loss = lm.loss(x, y)
        loss.backward()
        clip_grad_norm(lm.module.parameters(), clip)
        opt.step()
        last = float(loss.detach())
    return last


class Worker:
    """Pull the global checkpoint, train K local steps on this worker's corpus shard, submit.  Adam state persists across
    rounds and is never averaged, as in the reference."""

    def __init__(self, base_url: str, worker_id: str, shard_index: int = 0, num_shards: int = 1, local_steps: int = 30,
                 lr: float = 3e-3, seed: int = 0, device=None):
        self.base, self.worker_id, self.k, self.device = base_url.rstrip("/"), worker_id, local_steps, device
        code, _, body = _http("GET", self.base + "/config")
        if code != 200:
            raise RuntimeError(f"worker: GET /config -> {code}")
        self.config = json.loads(body)
        _, _, corpus = _http("GET", self.base + "/corpus")
        self.vocab = CharVocab.from_itos(self.config["vocab"])
        ids = self.vocab.encode(corpus.decode("utf-8"))
        self.ids = shard_slice(ids, shard_index, num_shards)
        self.lm = build_coop_lm(parse_arch(self.config["arch"]), self.config["model"], self.vocab.size, device=device,
                                seed=self.config["seed"])
        self.opt = Adam(self.lm.module.parameters(), lr=lr)
        self.rng = random.Random(seed)
        self.block = min(self.lm.max_len, max(2, len(self.ids) - 2))

    def run_round(self) -> dict:
        code, headers, blob = _http("GET", self.base + "/checkpoint")
        if code != 200:
            raise RuntimeError(f"worker: GET /checkpoint -> {code}")
        rnd = int(headers.get("X-Coop-Round", "0"))
        Checkpoint.load_into_bytes(self.lm.module, blob)
        loss = local_steps(self.lm, self.opt, self.ids, self.block, self.k, self.rng)
        code, _, body = _http("POST", self.base + "/submit", Checkpoint.save_bytes(self.lm.module),
                              {"X-Coop-Worker-Id": self.worker_id, "X-Coop-Round": str(rnd),
                               "X-Coop-Local-Steps": str(self.k), "Content-Type": "application/octet-stream"})
        out = json.loads(body) if body else {}
        out.update({"status": code, "loss": loss, "pulledRound": rnd})
        return out


class Peer:
    """Gossip peer: trains locally, serves its checkpoint, periodically averages 50/50 with one random peer."""

    def __init__(self, peer_urls: Sequence[str], arch="gpt", model: str = "tiny", text: Optional[str] = None,
                 shard_index: int = 0, num_shards: int = 1, local_steps: int = 30, gossip_every: int = 1,
                 lr: float = 3e-3, seed: int = 0, connect_timeout: float = 5.0, read_timeout: float = 30.0,
                 device=None):
        self.peers = [u.rstrip("/") for u in peer_urls]
        self.k, self.gossip_every = local_steps, gossip_every
        self.timeout = max(connect_timeout, read_timeout)
        text = K_TOY_CORPUS if text is None else text
        self.vocab = CharVocab.from_text(text)
        self.ids = shard_slice(self.vocab.encode(text), shard_index, num_shards)
        self.lm = build_coop_lm(parse_arch(arch) if isinstance(arch, str) else arch, model, self.vocab.size,
                                device=device, seed=seed)
        self.opt = Adam(self.lm.module.parameters(), lr=lr)
        self.rng = random.Random(seed + 1000 * shard_index)
        self.block = min(self.lm.max_len, max(2, len(self.ids) - 2))
        self.round = 0
        self.lock = threading.Lock()
        self.blob = Checkpoint.save_bytes(self.lm.module)
        self.log: List[str] = []

    def serve(self, host: str = "127.0.0.1", port: int = 0) -> ServerHandle:
        peer = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_GET(self):
                if self.path == "/health":
                    body = json.dumps({"ok": True, "round": peer.round}).encode()
                    ctype = "application/json"
                elif self.path == "/checkpoint":
                    with peer.lock:
                        body = peer.blob
                    ctype = "application/octet-stream"
                else:
                    self.send_response(404)
                    self.end_headers()
                    return
                self.send_response(200)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

        httpd = ThreadingHTTPServer((host, port), Handler)
        th = threading.Thread(target=httpd.serve_forever, daemon=True)
        th.start()
        return ServerHandle(httpd, th)

    def run_round(self) -> dict:
        loss = local_steps(self.lm, self.opt, self.ids, self.block, self.k, self.rng)
        self.round += 1
        gossiped = None
        if self.peers and self.round % self.gossip_every == 0:
            target = self.rng.choice(self.peers)
            try:
                code, _, other = _http("GET", target + "/checkpoint", timeout=self.timeout)
                if code != 200:
                    raise RuntimeError(f"status {code}")
                mine = Checkpoint.save_bytes(self.lm.module)
                Checkpoint.load_into_bytes(self.lm.module, average_checkpoints([mine, other], [0.5, 0.5]))
                gossiped = target
            except Exception as e:  # a vanished or slow peer must not stop training
                self.log.append(f"gossip with {target} failed: {e}")
        with self.lock:
            self.blob = Checkpoint.save_bytes(self.lm.module)
        return {"round": self.round, "loss": loss, "gossiped": gossiped}


def train_phase0(num_replicas: int = 2, rounds: int = 3, local_steps_per_round: int = 10, arch="gpt",
                 model: str = "tiny", text: Optional[str] = None, lr: float = 3e-3, seed: int = 0, device=None) -> dict:
    """In-process simulation (reference: bin/coop_train_phase0.dart:122-264): N replicas train K local steps each on
    their shard, are averaged and reloaded; a baseline model gets K*N steps per round on the full corpus.  Returns the
    per-round evaluation losses of both."""
    text = K_TOY_CORPUS if text is None else text
    vocab = CharVocab.from_text(text)
    ids = vocab.encode(text)
    a = parse_arch(arch) if isinstance(arch, str) else arch
    replicas = [build_coop_lm(a, model, vocab.size, device=device, seed=seed) for _ in range(num_replicas)]
    opts = [Adam(r.module.parameters(), lr=lr) for r in replicas]
    rngs = [random.Random(seed + 17 * i) for i in range(num_replicas)]
    shards = [shard_slice(ids, i, num_replicas) for i in range(num_replicas)]
    base = build_coop_lm(a, model, vocab.size, device=device, seed=seed)
    base_opt, base_rng = Adam(base.module.parameters(), lr=lr), random.Random(seed + 999)
    block = min(base.max_len, min(len(s) for s in shards) - 2)
    eval_rng_seed = seed + 4242

    def evaluate(lm: CoopLM) -> float:
        r = random.Random(eval_rng_seed)
        was = lm.module.training
        lm.module.eval()
        tot = 0.0
        with torch.no_grad():
            for _ in range(8):
                x, y = sample_window(ids, block, r, device=lm.module.device)
                tot += float(lm.loss(x, y))
        if was:
            lm.module.train()
        return tot / 8

    history = {"coop": [], "baseline": []}
    global_blob = Checkpoint.save_bytes(replicas[0].module)
    for _ in range(rounds):
        blobs = []
        for lm, opt, rng, shard in zip(replicas, opts, rngs, shards):
            Checkpoint.load_into_bytes(lm.module, global_blob)
            local_steps(lm, opt, shard, block, local_steps_per_round, rng)
            blobs.append(Checkpoint.save_bytes(lm.module))
        global_blob = average_checkpoints(blobs)
        Checkpoint.load_into_bytes(replicas[0].module, global_blob)
        history["coop"].append(evaluate(replicas[0]))
        local_steps(base, base_opt, ids, block, local_steps_per_round * num_replicas, base_rng)
        history["baseline"].append(evaluate(base))
    return history
