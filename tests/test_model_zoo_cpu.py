"""CPU tests of the long-tail model families: GPT-J, Pythia, BERT, sentence encoders and losses, modality encoders and
the multimodal classifier / encoder / generator / LM, MuZeroLM, CLIP vision, LlamaVision."""
import math

import pytest
import torch

from dart_pytorch_b200.io.dptc import Checkpoint
from dart_pytorch_b200.models import (AudioTransformer, BertConfig, BertModel, CLIPVisionConfig, CLIPVisionModel,
                                      CrossEncoder, GPTJConfig, GPTJModel, LlamaVision, MultiModalClassifier,
                                      MultiModalEncoder, MultiModalGenerator, MultiModalLM, MuZeroLM, PoolingMode,
                                      PythiaConfig, PythiaModel, SentenceEncoder, SentenceLosses, Similarity,
                                      TextTransformer, VideoTransformer, compute_rotary_dim, l2_normalize_row,
                                      mean_rows, pool_tokens)
from dart_pytorch_b200.models.llama import Llama, LlamaConfig


def _tokens(n=7, v=50, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, v, (n,), generator=g)


@pytest.mark.parametrize("family", ["gptj", "pythia"])
def test_parallel_residual_decoders_cache_matches_no_cache(family):
    if family == "gptj":
        m = GPTJModel(GPTJConfig(50, 16, 32, 2, 4, rotary_dim=4))
    else:
        m = PythiaModel(PythiaConfig(50, 16, 32, 2, 4))
    x = _tokens()
    assert m(x).shape == (7, 50)
    assert m(torch.stack([x, x]))[1].allclose(m(x), atol=1e-5)
    a = m.generate([1, 2, 3], 6, temperature=0.0)
    b = m.generate([1, 2, 3], 6, temperature=0.0, use_cache=False)
    assert a == b and len(a) == 9 and a[:3] == [1.0, 2.0, 3.0]
    with pytest.raises(ValueError):
        m.generate([], 3)
    with pytest.raises(ValueError):
        m(torch.zeros(17, dtype=torch.long))
    # training signal flows
    loss = m.loss(x[:-1], x[1:])
    loss.backward()
    assert all(p.grad is not None for p in m.parameters())
    # checkpoint round trip in the reference parameter order
    blob = Checkpoint.save_bytes(m)
    m2 = type(m)(m.config)
    for p in m2.parameters():
        p.data.add_(1.0)
    Checkpoint.load_into_bytes(m2, blob)
    assert torch.equal(m2(x), m(x))


def test_gptj_block_is_parallel_residual_with_single_norm():
    m = GPTJModel(GPTJConfig(30, 8, 16, 1, 2, rotary_dim=8))
    blk = m.blocks[0]
    x = torch.randn(5, 16)
    h = blk.ln(x)
    want = x + blk.attn(h, causal=True) + blk.ffn2(torch.nn.functional.gelu(blk.ffn1(h), approximate="tanh"))
    assert torch.allclose(blk(x), want, atol=1e-5)
    assert m.lm_head.bias is not None and blk.attn.b_qkv is None


def test_gptj_layer_placement_api():
    c = GPTJConfig(30, 8, 16, 2, 2, rotary_dim=8, layer_devices=["cpu", "cpu"], embedding_device="cpu")
    assert not c.has_mixed_placement and c.device_for_layer(1) == "cpu"
    with pytest.raises(ValueError):
        GPTJConfig(30, 8, 16, 2, 2, rotary_dim=8, layer_devices=["cpu"])
    assert GPTJModel(c)(_tokens(5, 30)).shape == (5, 30)


def test_rotary_pct_rule():
    assert compute_rotary_dim(64, 0.25) == 16
    assert compute_rotary_dim(10, 0.5) == 4      # 5 -> made even
    assert compute_rotary_dim(8, 0.1) == 2       # clamped
    assert compute_rotary_dim(8, 1.0) == 8
    with pytest.raises(ValueError):
        compute_rotary_dim(8, 0.0)


def test_bert_post_ln_layer_and_parameter_order():
    m = BertModel(BertConfig(60, 32, 32, 2, 4, 64))
    x = _tokens(7, 60)
    out = m(x)
    assert out.shape == (7, 32)
    # every row is a LayerNorm output: zero mean, unit variance (gamma=1, beta=0 at init)
    assert torch.allclose(out.mean(-1), torch.zeros(7), atol=1e-5)
    assert torch.allclose(out.var(-1, unbiased=False), torch.ones(7), atol=1e-3)
    ref = m.reference_parameters()
    assert ref[0].shape == (60, 32) and ref[1].shape == (32, 32) and ref[2].shape == (1, 32)
    with pytest.raises(ValueError):
        m(torch.zeros(33, dtype=torch.long))
    assert torch.allclose(m(torch.stack([x, x]))[0], out, atol=1e-5)


def test_sentence_encoder_pooling_similarity_and_losses():
    bert = BertModel(BertConfig(60, 32, 32, 1, 4, 64))
    enc = SentenceEncoder.wrap(bert, pooling=PoolingMode.mean)
    x = _tokens(7, 60)
    e = enc(x)
    assert e.shape == (1, 32) and abs(float((e * e).sum()) - 1.0) < 1e-5
    feats = torch.randn(5, 8)
    assert torch.allclose(pool_tokens(feats, PoolingMode.mean), feats.mean(0, keepdim=True), atol=1e-6)
    assert torch.equal(pool_tokens(feats, PoolingMode.cls), feats[:1])
    assert torch.allclose(mean_rows(feats), feats.mean(0, keepdim=True), atol=1e-6)
    with pytest.raises(ValueError):
        l2_normalize_row(feats)
    own = SentenceEncoder(50, 16, 32, 2, 4)
    E = own.encode_batch([_tokens(5), _tokens(6, seed=1), _tokens(4, seed=2)])
    assert E.shape == (3, 32)
    hits = Similarity.semantic_search(E, E, top_k=2)
    assert [h[0].corpus_index for h in hits] == [0, 1, 2] and len(hits[0]) == 2
    assert abs(Similarity.cos_sim(E[:1], E[:1]) - 1.0) < 1e-5
    a, p, n = torch.randn(4, 8), torch.randn(4, 8), torch.randn(4, 8)
    mnrl = SentenceLosses.multiple_negatives_ranking_loss(a, p, scale=2.0)
    want = torch.nn.functional.cross_entropy(2.0 * a @ p.t(), torch.arange(4), reduction="none")
    assert torch.allclose(mnrl.reshape(-1), want, atol=1e-5)
    t = torch.tensor([1.0, 0.0, 0.5, -1.0])
    assert torch.allclose(SentenceLosses.cosine_similarity_loss(a, p, t).reshape(()),
                          (((a * p).sum(-1) - t) ** 2).mean(), atol=1e-5)
    assert torch.allclose(SentenceLosses.triplet_loss(a, p, n, margin=0.5).reshape(()),
                          torch.relu((a * n).sum(-1) - (a * p).sum(-1) + 0.5).mean(), atol=1e-5)
    ce = CrossEncoder(50, 16, 32, 1, 4, num_labels=1)
    assert ce(_tokens(6)).shape == (1, 1) and 0.0 < ce.score(_tokens(6)) < 1.0


def test_multimodal_family_shapes_and_guards():
    au = AudioTransformer(10, 20, 32, 1, 4)
    vi = VideoTransformer(32, 8, 32, 1, 4)
    tx = TextTransformer(50, 16, 32, 1, 4)
    assert vi.frame_projection is None
    a, v, t = torch.randn(6, 10), torch.randn(4, 32), _tokens(7)
    clf = MultiModalClassifier(au, vi, 5, text=tx)
    assert clf(a, v, t).shape == (1, 5)
    with pytest.raises(ValueError):
        clf(a, v)
    enc = MultiModalEncoder(au, vi, 32, text=tx)
    assert enc(a, v, t).shape == (17, 32)
    gen = MultiModalGenerator(50, 12, 32, audio=au, text=tx)
    assert gen(t[:4], audio_features=a, text_in=t).shape == (4, 50)
    out = gen.generate([1], 4, audio_features=a, text_in=t, eos_id=None)
    assert len(out) == 5 and out[0] == 1
    with pytest.raises(ValueError):
        gen.encode(audio_features=a)          # text encoder present but no text input
    lm = MultiModalLM(50, 32, 40, image_patch_pixels=12, audio_feature_dim=10)
    img = torch.randn(3, 12)
    logits, start, total = lm.forward_all(t[:4], image_patches=img, audio_features=a, text_prompt=t[:2])
    assert logits.shape == (15, 50) and start == 11 and total == 15
    assert lm(t[:4], image_patches=img, audio_features=a, text_prompt=t[:2]).shape == (4, 50)
    assert len(lm.generate([1], 3, image_patches=img, audio_features=a, text_prompt=t[:2])) == 4
    with pytest.raises(ValueError):
        lm(t[:4], image_patches=img, audio_features=a)      # prompt required
    # causality of the packed stream: changing the last target token leaves earlier target logits unchanged
    t2 = t[:4].clone()
    t2[-1] = (t2[-1] + 1) % 50
    l1 = lm(t[:4], image_patches=img, audio_features=a, text_prompt=t[:2])
    l2 = lm(t2, image_patches=img, audio_features=a, text_prompt=t[:2])
    assert torch.allclose(l1[:3], l2[:3], atol=1e-5)


def test_muzero_unroll_contract():
    mz = MuZeroLM(50, 16, 32, 6)
    u = mz.unroll(_tokens(7), [1, 2, 3])
    assert len(u.states) == 4 and len(u.policies) == 4 and len(u.values) == 4 and len(u.rewards) == 3
    assert u.states[0].shape == (1, 32) and u.policies[0].shape == (1, 6) and u.rewards[0].shape == (1, 1)
    r = mz.recurrent_inference(u.states[0], 1)
    assert torch.allclose(r.next_state, u.states[1], atol=1e-6)
    with pytest.raises(ValueError):
        mz.dynamics(u.states[0], 6)
    (u.values[-1].sum() + u.rewards[-1].sum()).backward()
    assert mz.representation.token_embed.weight.grad is not None


def test_clip_vision_and_llama_vision():
    cfg = CLIPVisionConfig(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4, ffn_dim=64)
    cv = CLIPVisionModel(cfg)
    patches = torch.randn(4, 192)
    assert cv(patches).shape == (5, 32) and cv(torch.randn(2, 3, 16, 16)).shape == (2, 5, 32)
    assert cv.patch_projection.bias is None
    with pytest.raises(ValueError):
        cv(torch.randn(3, 192))
    ll = Llama(LlamaConfig(50, 32, 32, 1, 4, 2, 64))
    lv = LlamaVision.build(cv, ll)
    x = _tokens(7)
    assert lv.num_image_tokens == 5 and lv(patches, x).shape == (12, 50)
    out = lv.generate(patches, [1, 2], 3, temperature=0.0)
    assert len(out) == 5 and out[:2] == [1.0, 2.0]
    loss = lv.loss(patches, x[:-1], x[1:])
    loss.backward()
    assert lv.projector.up.weight.grad is not None and math.isfinite(float(loss))
    with pytest.raises(ValueError):
        lv(patches, torch.zeros(40, dtype=torch.long))
