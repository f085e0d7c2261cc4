"""CPU behaviour of the Llama, ViT and MoE families (modelled on the reference's llama_test.dart, gqa_test.dart,
vit_test.dart, moe_test.dart)."""
import random

import pytest
import torch

from dart_pytorch_b200 import Checkpoint, Adam, clip_grad_norm
from dart_pytorch_b200.models.llama import Llama, LlamaConfig
from dart_pytorch_b200.models.moe_lm import MoELanguageModel
from dart_pytorch_b200.models.vit import (ViTBackbone, ViTClassifier, ViTFaceEmbedding, ViTObjectDetector, patchify,
                                          vit_cls_feature)
from dart_pytorch_b200.nn.moe import (BiasUpdateRule, Expert, ExpertVariant, GateFunction, MoEFeedForward)


def small_llama(seed=0, **kw):
    base = dict(vocab_size=97, max_ctx=48, embed_dim=32, num_layers=2, num_heads=4, num_kv_heads=2, ffn_dim=48,
                init_std=0.05, seed=seed)
    base.update(kw)
    return Llama(LlamaConfig(**base))


def test_llama_parameter_layout_matches_reference_order():
    m = small_llama()
    shapes = [tuple(p.shape) for p in m.reference_parameters()]
    # embedIn, per block {attnNorm, ffnNorm, wq x4, wk x2, wv x2, wo, gate, up, down}, finalNorm (tied head)
    blk = [(32,), (32,)] + [(8, 32)] * 8 + [(32, 32), (48, 32), (48, 32), (32, 48)]
    assert shapes == [(97, 32)] + blk + blk + [(32,)]
    assert len(small_llama(tie_weights=False).reference_parameters()) == len(shapes) + 1
    with pytest.raises(ValueError):
        LlamaConfig(vocab_size=10, max_ctx=8, embed_dim=32, num_layers=1, num_heads=4, num_kv_heads=3, ffn_dim=8)


def test_llama_cache_equals_no_cache_and_batch_equals_single():
    m = small_llama(seed=2)
    prompt = [3.0, 9.0, 27.0, 81.0]
    a = m.generate(prompt, 12, temperature=0.0)
    b = m.generate(prompt, 12, temperature=0.0, use_cache=False)
    assert a == b
    s1 = m.generate(prompt, 8, temperature=0.8, top_k=4, rng=random.Random(1))
    s2 = m.generate(prompt, 8, temperature=0.8, top_k=4, rng=random.Random(1), use_cache=False)
    assert s1 == s2
    gb = m.generate_batch(torch.tensor([[3, 9, 27, 81], [1, 2, 3, 4]]), 12)
    assert gb[0].tolist() == [int(t) for t in a]
    x = torch.randint(0, 97, (3, 11))
    with torch.no_grad():
        assert torch.allclose(m(x)[1], m(x[1]), atol=1e-5)
    with pytest.raises(ValueError):
        m(torch.zeros(49, dtype=torch.long))
    # forwardFromEmbeddings == logits of the embedded tokens
    with torch.no_grad():
        e = m.embed_in(x[0])
        assert torch.allclose(m.forward_from_embeddings(e), m(x[0]), atol=1e-5)


def test_llama_overfits_tiny_sequence_and_checkpoint_round_trip():
    torch.manual_seed(0)
    m = small_llama(seed=4)
    opt = Adam(m.parameters(), lr=5e-3)
    x = torch.randint(0, 97, (2, 16))
    y = torch.roll(x, -1, 1)
    first = None
    for _ in range(60):
        opt.zero_grad()
        loss = m.loss(x, y)
        loss.backward()
        clip_grad_norm(m.parameters(), 1.0)
        opt.step()
        first = first or float(loss)
    assert float(loss) < 0.5 * first
    other = small_llama(seed=77)
    Checkpoint.load_into_bytes(other, Checkpoint.save_bytes(m))
    assert other.generate([1.0, 2.0], 10, temperature=0.0) == m.generate([1.0, 2.0], 10, temperature=0.0)


def test_vit_inputs_agree_and_heads():
    m = ViTClassifier(image_size=32, patch_size=8, embed_dim=32, num_layers=2, num_heads=4, num_classes=5, seed=1)
    img = torch.randn(3, 3, 32, 32)
    p = patchify(img, 8)
    assert p.shape == (3, 16, 192)
    # (dy, dx, c) order inside a patch, row-major patches
    assert float(p[1, 5, (2 * 8 + 3) * 3 + 1]) == float(img[1, 1, 1 * 8 + 2, 1 * 8 + 3])
    with torch.no_grad():
        lo = m(img)
        assert torch.allclose(m(p), lo, atol=1e-5) and torch.allclose(m(p[0]), lo[:1], atol=1e-5)
        feats = m.backbone(p[0])
        assert feats.shape == (17, 32) and vit_cls_feature(feats).shape == (1, 32)
    with pytest.raises(ValueError):
        m(torch.randn(15, 192))
    with pytest.raises(ValueError):
        ViTBackbone(image_size=30, patch_size=8)
    shapes = [tuple(t.shape) for t in m.reference_parameters()]
    assert shapes[:4] == [(32, 192), (1, 32), (1, 32), (17, 32)] and shapes[-2:] == [(5, 32), (1, 5)]
    loss = m.loss(img, torch.tensor([0, 1, 2]))
    loss.backward()
    assert all(q.grad is not None for q in m.parameters())
    e = ViTFaceEmbedding(embed_dim=32, num_layers=1)(img)
    assert torch.allclose(e.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert abs(ViTFaceEmbedding.cosine_similarity(e[0], e[0]) - 1.0) < 1e-5
    cls, box = ViTObjectDetector(embed_dim=32, num_layers=1, num_queries=6, num_classes=3)(p[0])
    assert cls.shape == (6, 4) and box.shape == (6, 4) and float(box.min()) > 0 and float(box.max()) < 1


MOE_KW = dict(embed_dim=16, num_routed_experts=4, num_shared_experts=1, top_k=2, expert_hidden_dim=24, seed=3)


@pytest.mark.parametrize("variant", [ExpertVariant.mlp, ExpertVariant.swiGlu])
@pytest.mark.parametrize("gate", [GateFunction.softmax, GateFunction.sigmoid])
def test_moe_sparse_equals_dense_forward_and_backward(variant, gate):
    d = MoEFeedForward(expert_variant=variant, gate_function=gate, **MOE_KW)
    s = MoEFeedForward(expert_variant=variant, gate_function=gate, sparse_execution=True, **MOE_KW)
    x = torch.randn(10, 16, requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    yd, ys = d(x), s(x2)
    assert torch.allclose(yd, ys, atol=1e-6)
    yd.sum().backward()
    ys.sum().backward()
    assert torch.allclose(x.grad, x2.grad, atol=1e-6)
    for a, b in zip(d.parameters(), s.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-5)
    assert sum(d.expert_load) == 20  # exactly topK routed slots per token


def test_moe_routing_rules_bias_update_and_options():
    m = MoEFeedForward(16, 4, 0, 1, 8, seed=0)
    scores = torch.tensor([[0.4, 0.3, 0.2, 0.1], [0.1, 0.2, 0.3, 0.4]])
    assert m.route(scores).tolist() == [[1, 0, 0, 0], [0, 0, 0, 1]]
    m.routing_bias[:] = torch.tensor([0.0, 0.5, 0.0, 0.0])   # bias steers the choice only
    assert m.route(scores).tolist() == [[0, 1, 0, 0], [0, 1, 0, 0]]
    m._expert_load[:] = torch.tensor([4, 0, 2, 2])
    m.routing_bias.zero_()
    m.update_routing_bias()                                   # mean 2: under-loaded up, over-loaded down
    assert [round(v, 6) for v in m.routingBias] == [-0.001, 0.001, 0.0, 0.0] and m.expert_load == [0, 0, 0, 0]
    p = MoEFeedForward(16, 4, 0, 1, 8, bias_update_rule=BiasUpdateRule.proportional, bias_update_rate=0.1)
    p._expert_load[:] = torch.tensor([4, 0, 2, 2])
    p.update_routing_bias()
    assert [round(v, 6) for v in p.routingBias] == [-0.1, 0.1, 0.0, 0.0]
    g = MoEFeedForward(16, 8, 0, 2, 8, num_expert_groups=4, top_k_groups=1)
    mask = g.route(torch.rand(20, 8))
    for row in mask.view(20, 4, 2).sum(-1).tolist():          # both picks come from one group
        assert sorted(row) == [0, 0, 0, 2]
    for bad in (dict(top_k=0), dict(top_k=5), dict(num_expert_groups=3), dict(num_expert_groups=2, top_k_groups=3)):
        kw = dict(embed_dim=16, num_routed_experts=4, num_shared_experts=0, top_k=2, expert_hidden_dim=8)
        kw.update(bad)
        with pytest.raises(ValueError):
            MoEFeedForward(**kw)
    with pytest.raises(ValueError):
        m(torch.randn(2, 3, 16))
    c = MoEFeedForward(16, 4, 0, 2, 8, capacity_factor=1.0, aux_loss_coef=0.01)
    c(torch.randn(40, 16))
    assert max(c.expert_load) <= 20 and float(c.last_aux_loss) > 0
    assert [tuple(t.shape) for t in Expert(16, 8, variant=ExpertVariant.swiGlu).reference_parameters()] == \
        [(8, 16), (1, 8), (16, 8), (1, 16), (8, 16), (1, 8)]


def test_moe_language_model_reference_defaults_and_benchmark_options():
    m = MoELanguageModel(50, 32, 2, 4, 16, expert_hidden_dim=24, seed=1)
    assert m(torch.randint(0, 50, (12,))).shape == (12, 50)
    with pytest.raises(ValueError):
        m(torch.zeros(17, dtype=torch.long))
    b = MoELanguageModel(50, 32, 2, 4, 16, num_routed_experts=8, num_shared_experts=0, expert_hidden_dim=24,
                         expert_variant=ExpertVariant.swiGlu, norm="rms", rope_base=10000.0, capacity_factor=1.25,
                         aux_loss_coef=0.01, expert_bias=False, head_bias=False, sparse_execution=True, init_std=0.02)
    x = torch.randint(0, 50, (3, 16))
    opt = Adam(b.parameters(), lr=3e-3)
    first = None
    for _ in range(30):
        opt.zero_grad()
        loss = b.loss(x, torch.roll(x, -1, 1))
        loss.backward()
        opt.step()
        first = first or float(loss)
    assert float(loss) < first and float(b.aux_loss()) > 0
    b.update_routing_bias()


def test_tiny_char_gpt_recipe_end_to_end():
    """The smallest end-to-end workload (train with warm-up / cosine / clipping, DPTC round trip, cached greedy
    generation) runs and is self-consistent on the CPU."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from benchmarks.tiny_gpt_cpu import run_ours
    res = run_ours(24)
    assert res["checkpoint_round_trip"] and res["generate_matches_after_reload"] and res["cache_matches_no_cache"]
    assert res["checkpoint_bytes"] > 4 * 65 * 64
    # cached generation stops when the context (32 positions) is full
    assert 32 <= len(res["generated"]) <= 3 + 32 and all(0 <= t < 65 for t in res["generated"])
    assert abs(res["loss_first"] - 4.17) < 0.2          # ln(65) for random tokens
