"""Loader parity against the HuggingFace reference implementations (tiny random models built in-process, no
downloads): GPT-NeoX / Pythia, GPT-J (interleaved rotary), BERT, CLIP vision."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from dart_pytorch_b200.io.hf_loaders_more import BertHFLoader, ClipHFLoader, GPTJHFLoader, PythiaHFLoader
from dart_pytorch_b200.models import (BertConfig, BertModel, CLIPVisionConfig, CLIPVisionModel, GPTJConfig, GPTJModel,
                                      PythiaConfig, PythiaModel)


def _state(m):
    return {k: v.detach().clone() for k, v in m.state_dict().items()}


def test_pythia_matches_hf_gpt_neox():
    cfg = transformers.GPTNeoXConfig(vocab_size=97, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                     intermediate_size=128, rotary_pct=0.5, max_position_embeddings=64,
                                     hidden_act="gelu_pytorch_tanh", use_parallel_residual=True,
                                     attention_dropout=0.0, hidden_dropout=0.0)
    torch.manual_seed(0)
    hf = transformers.GPTNeoXForCausalLM(cfg).eval()
    ours = PythiaModel(PythiaConfig(97, 64, 32, 2, 4, rotary_pct=0.5))
    rep = PythiaHFLoader.load_map(ours, _state(hf))
    assert rep.consumed_count == 3 + 2 * 12 + 1 and all("rotary" in k or "bias" in k.split(".")[-1] or "masked" in k
                                                        for k in rep.unused_keys)
    x = torch.randint(0, 97, (1, 11))
    with torch.no_grad():
        want = hf(x).logits[0]
        got = ours(x[0])
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
    # dump -> load round trip reproduces the HF tensors
    back = PythiaHFLoader.dump(ours)
    st = _state(hf)
    for k, v in back.items():
        assert torch.allclose(v, st[k].float(), atol=1e-6), k
    bad = _state(hf)
    del bad["embed_out.weight"]
    with pytest.raises(ValueError):
        PythiaHFLoader.load_map(ours, bad)


def test_gptj_matches_hf_with_rotary_permutation():
    cfg = transformers.GPTJConfig(vocab_size=89, n_positions=64, n_embd=32, n_layer=2, n_head=4, rotary_dim=4,
                                  n_inner=128, activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0,
                                  attn_pdrop=0.0)
    torch.manual_seed(1)
    hf = transformers.GPTJForCausalLM(cfg).eval()
    with torch.no_grad():
        hf.lm_head.bias.normal_(0, 0.1)
    ours = GPTJModel(GPTJConfig(89, 64, 32, 2, 4, rotary_dim=4))
    GPTJHFLoader.load_map(ours, _state(hf))
    x = torch.randint(0, 89, (1, 9))
    with torch.no_grad():
        want = hf(x).logits[0]
        got = ours(x[0])
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
    # cached decode equals the full forward
    with torch.no_grad():
        cache = ours.new_cache()
        a = ours.logits(x[0, :5], 0, cache)
        b = ours.logits(x[0, 5:], 5, cache)
    assert torch.allclose(torch.cat([a, b]), got, atol=2e-4)
    back = GPTJHFLoader.dump(ours)
    st = _state(hf)
    for k, v in back.items():
        assert torch.allclose(v, st[k].float(), atol=1e-6), k
    idx = GPTJHFLoader.rotary_row_permutation(8, 4)
    assert idx.tolist() == [0, 2, 1, 3, 4, 5, 6, 7]
    hyb = GPTJHFLoader.gpt_j_6b_hybrid_config(4, gpu="cpu")
    assert hyb.num_layers == 28 and len(hyb.layer_devices) == 28
    with pytest.raises(ValueError):
        GPTJHFLoader.gpt_j_6b_hybrid_config(29)


def test_bert_matches_hf():
    cfg = transformers.BertConfig(vocab_size=101, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                  intermediate_size=64, max_position_embeddings=40, hidden_act="gelu_pytorch_tanh",
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    torch.manual_seed(2)
    hf = transformers.BertModel(cfg, add_pooling_layer=False).eval()
    ours = BertModel(BertConfig(101, 40, 32, 2, 4, 64))
    rep = BertHFLoader.load_map(ours, _state(hf))
    assert all("position_ids" in k or "pooler" in k for k in rep.unused_keys)
    x = torch.randint(0, 101, (1, 13))
    with torch.no_grad():
        want = hf(x).last_hidden_state[0]
        got = ours(x[0])
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
    st = _state(hf)
    for k, v in BertHFLoader.dump(ours).items():
        if "token_type" in k:
            assert torch.allclose(v[0], st[k][0], atol=1e-6)
        else:
            assert torch.allclose(v, st[k].float(), atol=1e-6), k
    assert BertHFLoader.mini_lm_l6_v2_config().embed_dim == 384


def test_clip_vision_matches_hf():
    cfg = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                        num_attention_heads=4, image_size=16, patch_size=8, hidden_act="quick_gelu",
                                        attention_dropout=0.0)
    torch.manual_seed(3)
    hf = transformers.CLIPVisionModel(cfg).eval()
    ours = CLIPVisionModel(CLIPVisionConfig(image_size=16, patch_size=8, embed_dim=32, num_layers=2, num_heads=4,
                                            ffn_dim=64))
    ClipHFLoader.load_map(ours, _state(hf))
    img = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        out = hf(pixel_values=img)
        got = ours(img)
    # HF applies post_layernorm to the pooled CLS row only; the encoder here ends with that norm on every row
    want_cls = out.pooler_output
    assert torch.allclose(got[:, 0], want_cls, atol=2e-4), float((got[:, 0] - want_cls).abs().max())
    ln = hf.vision_model.post_layernorm
    with torch.no_grad():
        assert torch.allclose(got, ln(out.last_hidden_state), atol=2e-4)
    st = _state(hf)
    for k, v in ClipHFLoader.dump(ours).items():
        assert torch.allclose(v, st[k].float(), atol=1e-6), k
    with pytest.raises(ValueError):
        ClipHFLoader.load_map(ours, {"text_model.x": torch.zeros(1)})
    assert ClipHFLoader.large14_config().num_patches == 256


def test_gpt2_matches_hf():
    from dart_pytorch_b200.io.hf_loaders import GPT2HFLoader
    from dart_pytorch_b200.models import GPT, GPTConfig
    from dart_pytorch_b200.nn.transformer import Activation
    cfg = transformers.GPT2Config(vocab_size=83, n_positions=32, n_embd=32, n_layer=2, n_head=4,
                                  activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(4)
    hf = transformers.GPT2LMHeadModel(cfg).eval()
    ours = GPT(GPTConfig(vocab_size=83, max_ctx=32, embed_dim=32, num_layers=2, num_heads=4, attn_bias=True,
                         activation=Activation.geluTanh))
    GPT2HFLoader.load_map(ours, _state(hf))
    x = torch.randint(0, 83, (1, 12))
    with torch.no_grad():
        want = hf(x).logits[0]
        got = ours(x[0])
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
    out = ours.generate(x[0, :4].tolist(), 5, temperature=0.0)
    with torch.no_grad():
        ref = hf.generate(x[:, :4], max_new_tokens=5, do_sample=False, pad_token_id=0)[0].tolist()
    assert [int(t) for t in out] == ref


def test_llama_matches_hf_with_gqa():
    from dart_pytorch_b200.io.hf_loaders import LlamaHFLoader
    from dart_pytorch_b200.models.llama import Llama, LlamaConfig
    cfg = transformers.LlamaConfig(vocab_size=79, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                   rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                   attention_bias=False, mlp_bias=False)
    torch.manual_seed(5)
    hf = transformers.LlamaForCausalLM(cfg).eval()
    ours = Llama(LlamaConfig(79, 64, 32, 2, 4, 2, 64, rope_base=10000.0, rms_norm_eps=1e-5, tie_weights=False))
    LlamaHFLoader.load_map(ours, _state(hf))
    x = torch.randint(0, 79, (2, 10))
    with torch.no_grad():
        want = hf(x).logits
        got = ours(x)
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
