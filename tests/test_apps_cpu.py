"""Apps: demo trainers through the CLI, the /generate HTTP contract, the RAG chat service, helper functions."""
import json
import random
import urllib.error
import urllib.request

import numpy as np
import pytest
import torch

from dart_pytorch_b200.apps import (GenerationService, RagChatService, chunk_spans, generate_text, get_window,
                                    last_row_logits, llama3_chat_prompt, load_corpus, sample_from_logits)
from dart_pytorch_b200.apps.__main__ import main as cli
from dart_pytorch_b200.data.tokenizers import CharTokenizer
from dart_pytorch_b200.models import GPT, GPTConfig


def _http(method, url, body=None, headers=None):
    req = urllib.request.Request(url, data=body, method=method, headers=headers or {})
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, r.read()
    except urllib.error.HTTPError as e:
        return e.code, e.read()


def _tiny_gpt(vocab, ctx=48):
    return GPT(GPTConfig(vocab_size=vocab, max_ctx=ctx, embed_dim=32, num_layers=1, num_heads=4, seed=1))


def test_util_helpers():
    text = load_corpus(100)
    assert len(text) == 100
    ids = list(range(50))
    x, y = get_window(ids, 8, random.Random(0))
    assert x.shape == (8,) and torch.equal(y, x + 1)
    with pytest.raises(ValueError):
        get_window(ids[:8], 8, random.Random(0))
    assert sample_from_logits([0.1, 3.0, 0.2], temperature=0.0) == 1
    assert sample_from_logits([0.1, 3.0, 0.2], temperature=1.0, top_k=1) == 1
    draws = {sample_from_logits([0.0, 0.0, -50.0], 1.0, None, random.Random(s)) for s in range(20)}
    assert draws == {0, 1}
    out = generate_text([1, 2], 5, max_ctx=3, vocab_size=4, step_fn=lambda ctx: [0, 0, 0, 0, 9.0, 0, 0, 0][:8][-4:] if False
                        else [0.0] * 4 + [0.0, 5.0, 0.0, 0.0], temperature=0.0)
    assert out == [1, 2, 1, 1, 1, 1, 1]
    assert last_row_logits(torch.arange(12.0).reshape(3, 4), 3) == [8.0, 9.0, 10.0]


@pytest.mark.parametrize("cmd", ["gpt_train", "shakespeare_transformer_lm", "shakespeare_aft", "shakespeare_moe",
                                 "llama_train"])
def test_cli_trainers_run(cmd, tmp_path, capsys):
    save = tmp_path / "m.dptc"
    cli([cmd, "--device", "cpu", "--steps", "3", "--block", "16", "--dim", "16", "--layers", "1", "--heads", "2",
         "--batch", "2", "--max-chars", "400", "--sample", "4", "--save", str(save)])
    out = capsys.readouterr().out
    assert "trained 3 steps" in out and save.exists() and save.read_bytes()[:4] == b"DPTC"


def test_cli_misc_demos(capsys, tmp_path):
    cli(["vit_demo", "--device", "cpu", "--steps", "2"])
    cli(["train_muzero_lm_demo", "--device", "cpu", "--steps", "2"])
    cli(["coop_train_phase0", "--rounds", "1", "--local-steps", "2"])
    cli(["demo_faiss", "--n", "300", "--nq", "5", "--d", "8", "--indexes", "IVF4,Flat", "--csv", str(tmp_path / "b.csv")])
    out = capsys.readouterr().out
    assert "baseline" in out and "IVF4,Flat" in out and (tmp_path / "b.csv").read_text().startswith("label,")


def test_generation_service_http_contract():
    tok = CharTokenizer.from_text("abcdefgh ")
    svc = GenerationService(_tiny_gpt(tok.vocab_size), tok, model_name="tiny")
    h = svc.serve()
    try:
        code, body = _http("GET", h.url + "/health")
        assert code == 200 and json.loads(body)["status"] == "ok"
        info = json.loads(_http("GET", h.url + "/info")[1])
        assert info["embedDim"] == 32 and info["vocabSize"] == tok.vocab_size and info["maxCtx"] == 48
        code, body = _http("POST", h.url + "/generate", json.dumps({"text": "abc", "maxNewTokens": 5}).encode())
        out = json.loads(body)
        assert code == 200 and len(out["newTokens"]) == 5 and out["tokens"][:3] == tok.encode("abc")
        assert out["text"].startswith("abc") and out["elapsedMs"] >= 0
        again = json.loads(_http("POST", h.url + "/generate", json.dumps({"tokens": out["tokens"][:3],
                                                                          "maxNewTokens": 5, "useCache": False}).encode())[1])
        assert again["newTokens"] == out["newTokens"]          # greedy: cache and no-cache agree
        s1 = json.loads(_http("POST", h.url + "/generate", json.dumps({"text": "ab", "temperature": 1.0, "topK": 5,
                                                                       "seed": 7}).encode())[1])
        s2 = json.loads(_http("POST", h.url + "/generate", json.dumps({"text": "ab", "temperature": 1.0, "topK": 5,
                                                                       "seed": 7}).encode())[1])
        assert s1["tokens"] == s2["tokens"] and len(s1["newTokens"]) == 20
        assert _http("POST", h.url + "/generate", b"{}")[0] == 400
        assert _http("POST", h.url + "/generate", b"not json")[0] == 400
        assert _http("GET", h.url + "/nope")[0] == 404
        no_tok = GenerationService(_tiny_gpt(tok.vocab_size), None)
        assert no_tok.run({"text": "abc"})[0] == 400 and no_tok.run({"tokens": [1, 2]})[1]["text"] is None
    finally:
        h.close()


def test_rag_chat_service():
    corpus = "the cat sat on the mat. " * 30 + "quantum flux capacitors need plutonium. " * 30
    tok = CharTokenizer.from_text(corpus + "UserAssistant:Context[]0123456789\nPrevious conversation?")
    svc = RagChatService(_tiny_gpt(tok.vocab_size, ctx=512), tok, max_new_tokens=8)
    assert chunk_spans(150) == [(0, 150)] and chunk_spans(0) == []
    assert chunk_spans(450) == [(0, 200), (100, 300), (200, 400), (300, 450)]
    h = svc.serve()
    try:
        assert b"<title>RAG chat" in _http("GET", h.url + "/")[1]
        code, body = _http("POST", h.url + "/upload", ("the cat sat on the mat. " * 30).encode(),
                           {"X-Filename": "cats.txt"})
        up = json.loads(body)
        assert code == 200 and up["ok"] and up["filename"] == "cats.txt" and up["chunks"] == up["totalChunks"] >= 6
        _http("POST", h.url + "/upload", ("quantum flux capacitors need plutonium. " * 30).encode(),
              {"X-Filename": "flux.txt"})
        st = json.loads(_http("GET", h.url + "/status")[1])
        assert st["numDocs"] == 2 and [d["title"] for d in st["docs"]] == ["cats.txt", "flux.txt"]
        code, body = _http("POST", h.url + "/chat", json.dumps({"message": "quantum flux capacitors"}).encode())
        ans = json.loads(body)
        assert code == 200 and isinstance(ans["answer"], str) and 1 <= len(ans["sources"]) <= 4
        assert all(set(s) == {"docTitle", "span", "score", "preview"} for s in ans["sources"])
        assert ans["promptTokens"] + 8 <= 512
        assert json.loads(_http("GET", h.url + "/status")[1])["historyLen"] == 2
        assert _http("POST", h.url + "/chat", json.dumps({"message": "  "}).encode())[0] == 400
        assert _http("POST", h.url + "/upload", b"   ")[0] == 400
        assert json.loads(_http("POST", h.url + "/reset")[1])["ok"]
        assert json.loads(_http("GET", h.url + "/status")[1]) == {"numDocs": 0, "numChunks": 0, "historyLen": 0, "docs": []}
        assert json.loads(_http("GET", h.url + "/health")[1])["maxCtx"] == 512
    finally:
        h.close()
    # index rows are centred and unit-norm
    svc.upload("a.txt", "the cat sat on the mat. " * 30)
    assert np.allclose(np.linalg.norm(svc.index.storage, axis=1), 1.0, atol=1e-4)


def test_llama3_chat_template():
    p = llama3_chat_prompt([("user", "hi"), ("assistant", "hello"), ("user", "bye")], system="be brief")
    assert p.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nbe brief<|eot_id|>")
    assert p.count("<|eot_id|>") == 4 and p.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
