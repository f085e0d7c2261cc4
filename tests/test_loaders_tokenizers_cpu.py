"""CPU tests: HF GPT-2 / Llama loaders on synthetic state dicts, HF BPE and WordPiece tokenizers
(modelled on the reference's gpt2_hf_loader_test.dart, llama_hf_loader_test.dart, hf_bpe_tokenizer_test.dart,
wordpiece_tokenizer_test.dart; fixtures are synthesised in memory)."""
import json

import pytest
import torch

from dart_pytorch_b200.data.hf_tokenizers import HFBpeTokenizer, WordPieceTokenizer, bytes_to_unicode
from dart_pytorch_b200.io.hf_loaders import GPT2HFLoader, LlamaHFLoader
from dart_pytorch_b200.io.safetensors import SafeTensors
from dart_pytorch_b200.models.gpt import GPT, GPTConfig
from dart_pytorch_b200.models.llama import Llama, LlamaConfig
from dart_pytorch_b200.nn.transformer import Activation


def _gpt(seed):
    return GPT(GPTConfig(vocab_size=40, max_ctx=16, embed_dim=16, num_layers=2, num_heads=4, attn_bias=True,
                         activation=Activation.geluTanh, seed=seed))


def test_gpt2_loader_round_trip_prefix_and_rejections(tmp_path):
    src, dst = _gpt(1), _gpt(2)
    state = GPT2HFLoader.dump(src, prefix="transformer.")
    state["transformer.h.0.attn.bias"] = torch.ones(1, 1, 16, 16)       # ignorable HF buffer
    state["lm_head.weight"] = state["transformer.wte.weight"].clone()
    assert state["transformer.h.0.attn.c_attn.weight"].shape == (16, 48)    # Conv1D layout [in, out]
    rep = GPT2HFLoader.load_map(dst, state)
    assert rep.consumed_count == 2 + 12 * 2 + 2 and sorted(rep.unused_keys) == ["h.0.attn.bias", "lm_head.weight"]
    x = torch.randint(0, 40, (9,))
    with torch.no_grad():
        assert torch.allclose(src(x), dst(x), atol=1e-6)
    # per-head view of the fused projection equals the reference's slice of c_attn
    w = state["transformer.h.1.attn.c_attn.weight"].t()
    assert torch.equal(dst.encoder.blocks[1].mha.wk_weight(2), w[16 + 2 * 4:16 + 3 * 4])
    path = tmp_path / "model.safetensors"
    SafeTensors.save_file({k: v for k, v in state.items()}, str(path))
    third = _gpt(3)
    GPT2HFLoader.load_file(third, str(path))
    with torch.no_grad():
        assert torch.allclose(src(x), third(x), atol=1e-6)
    bad = dict(state)
    del bad["transformer.h.1.mlp.c_fc.bias"]
    with pytest.raises(ValueError, match="missing tensor"):
        GPT2HFLoader.load_map(_gpt(4), bad)
    bad = dict(state)
    bad["transformer.wpe.weight"] = torch.zeros(8, 16)
    with pytest.raises(ValueError, match="shape"):
        GPT2HFLoader.load_map(_gpt(4), bad)
    cfg = GPT2HFLoader.gpt2_medium_config()
    assert (cfg.embed_dim, cfg.num_layers, cfg.num_heads, cfg.attn_bias) == (1024, 24, 16, True)


def test_llama_loader_round_trip_tied_and_untied():
    def mk(seed, tie):
        return Llama(LlamaConfig(vocab_size=50, max_ctx=16, embed_dim=32, num_layers=2, num_heads=4, num_kv_heads=2,
                                 ffn_dim=24, tie_weights=tie, seed=seed, init_std=0.05))
    for tie in (True, False):
        src, dst = mk(1, tie), mk(2, tie)
        state = LlamaHFLoader.dump(src)
        state["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(4)
        rep = LlamaHFLoader.load_map(dst, state)
        assert rep.unused_keys == []
        x = torch.randint(0, 50, (2, 7))
        with torch.no_grad():
            assert torch.allclose(src(x), dst(x), atol=1e-6)
        assert state["model.layers.1.self_attn.k_proj.weight"].shape == (16, 32)
    bad = LlamaHFLoader.dump(mk(1, True))
    bad["model.layers.0.mlp.up_proj.weight"] = torch.zeros(25, 32)
    with pytest.raises(ValueError):
        LlamaHFLoader.load_map(mk(3, True), bad)
    c = LlamaHFLoader.llama31_8b_config(max_ctx=4096)
    assert (c.embed_dim, c.num_layers, c.num_kv_heads, c.ffn_dim, c.tie_weights, c.max_ctx) == \
        (4096, 32, 8, 14336, False, 4096)


def _tiny_bpe_json(pattern=None, merges_as_lists=False):
    b2u = bytes_to_unicode()
    sp = b2u[ord(" ")]
    vocab = {b2u[i]: i for i in range(256)}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (sp, "w")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    doc = {"model": {"type": "BPE", "vocab": vocab,
                     "merges": [[a, b] for a, b in merges] if merges_as_lists else [f"{a} {b}" for a, b in merges]},
           "added_tokens": [{"id": 300, "content": "<|endoftext|>"}, {"id": 301, "content": "<|eot_id|>"},
                            {"id": 302, "content": "<|eot|>"}]}
    if pattern:
        doc["pre_tokenizer"] = {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": pattern}, "behavior": "Isolated"}, {"type": "ByteLevel"}]}
    return json.dumps(doc)


def test_hf_bpe_tokenizer():
    tok = HFBpeTokenizer.from_json(_tiny_bpe_json())
    ids = tok.encode("hello world")
    assert ids[0] == tok.vocab["hello"] and ids[1] == tok.vocab[bytes_to_unicode()[32] + "w"]
    assert tok.decode(ids) == "hello world"
    text = "héllo <|endoftext|>wörld<|eot_id|>!"
    ids = tok.encode(text)
    assert 300 in ids and 301 in ids and tok.decode(ids) == text
    assert tok.decode(ids, skip_special=True) == "héllo wörld!"
    assert tok.decode([5000, tok.vocab["hello"]]) == "hello"       # unknown ids are skipped
    assert tok.end_of_text_id == 300 and tok.llama_eot_id == 301 and tok.llama_begin_of_text_id is None
    assert tok.vocab_size == 303
    lists = HFBpeTokenizer.from_json(_tiny_bpe_json(merges_as_lists=True))
    assert lists.encode("hello world") == tok.encode("hello world")
    llama_pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    l3 = HFBpeTokenizer.from_json(_tiny_bpe_json(pattern=llama_pat))
    assert l3.decode(l3.encode("Hello 12345 wORLD'S")) == "Hello 12345 wORLD'S"
    assert len(l3.encode("12345")) == 5 and len(l3._pre.findall("12345")) == 2     # digits split in groups of <= 3
    with pytest.raises(ValueError):
        HFBpeTokenizer.from_json('{"model": {"type": "Unigram", "vocab": {}}}')


def test_wordpiece_tokenizer(tmp_path):
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "hello", "world", "un", "##aff", "##able", ",", "cafe", "!"]
    p = tmp_path / "vocab.txt"
    p.write_text("\n".join(vocab) + "\n", encoding="utf-8")
    tok = WordPieceTokenizer.from_vocab_file(str(p))
    assert tok.tokenize("Hello, unaffable Café!") == ["hello", ",", "un", "##aff", "##able", "cafe", "!"]
    assert tok.tokenize("xyzzy hello") == ["[UNK]", "hello"]
    ids = tok.encode("hello world")
    assert ids == [2, 4, 5, 3] and tok.decode(ids) == "hello world"
    assert tok.encode("hello world hello world", max_length=4) == [2, 4, 5, 3]
    assert tok.encode("hello", add_special_tokens=False) == [4]
    assert tok.encode_pair("hello", "world") == [2, 4, 3, 5, 3]
    assert len(tok.encode_pair("hello world hello", "world world", max_length=6)) == 6
    assert tok.decode([2, 6, 7, 8, 3, 0]) == "unaffable"
    with pytest.raises(ValueError):
        WordPieceTokenizer(["a", "b"])
