"""CPU tests of sentence pooling, the sentence / cross encoders, similarity helpers and the three sentence losses,
case by case after the reference's test/sentence_encoder_test.dart and test/sentence_losses_test.dart."""
import pytest
import torch

from dart_pytorch_b200 import Adam
from dart_pytorch_b200.models import CrossEncoder, SentenceEncoder, SentenceLosses, Similarity, TextTransformer
from dart_pytorch_b200.models.sentence import PoolingMode, l2_normalize_row, pool_tokens


def _unit(rows):
    t = torch.tensor(rows, dtype=torch.float32)
    return t / t.norm(dim=1, keepdim=True)


def test_pooling_and_row_normalisation():
    feats = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 1.0]])
    assert pool_tokens(feats, PoolingMode.mean).tolist() == [[3.0, 3.0]]
    assert pool_tokens(feats, PoolingMode.cls).tolist() == [[1.0, 2.0]]
    with pytest.raises(ValueError):
        pool_tokens(torch.zeros(0, 2))
    with pytest.raises(ValueError):
        pool_tokens(torch.zeros(2, 3, 4))
    row = l2_normalize_row(torch.tensor([[3.0, 4.0]]))
    assert torch.allclose(row, torch.tensor([[0.6, 0.8]]), atol=1e-6)
    for bad in (torch.zeros(2, 3), torch.zeros(3)):
        with pytest.raises(ValueError):
            l2_normalize_row(bad)


def test_sentence_encoder_shapes_modes_batch_and_wrap():
    toks = torch.tensor([1, 5, 9, 3])
    enc = SentenceEncoder(20, 8, 16, 1, 4, seed=1)
    e = enc(toks)
    assert e.shape == (1, 16) and abs(float(e.detach().norm()) - 1.0) < 1e-5 and enc.embed_dim == 16
    raw = SentenceEncoder(20, 8, 16, 1, 4, seed=1, normalize=False)(toks)
    assert abs(float(raw.detach().norm()) - 1.0) > 1e-3
    assert torch.allclose(raw / raw.norm(), e, atol=1e-5)
    cls = SentenceEncoder(20, 8, 16, 1, 4, seed=1, pooling=PoolingMode.cls, normalize=False)
    assert torch.allclose(cls(toks), cls.backbone(toks)[0:1], atol=1e-6)
    batch = enc.encode_batch([[1, 5, 9, 3], [2, 2], [7]])
    assert batch.shape == (3, 16) and torch.allclose(batch[0:1], e, atol=1e-6)
    backbone = TextTransformer(20, 8, 16, 1, 4, seed=1)
    wrapped = SentenceEncoder.wrap(backbone)
    assert wrapped.backbone is backbone and torch.allclose(wrapped(toks), e, atol=1e-6)
    assert len(wrapped.parameters()) == len(backbone.parameters())


def test_sentence_encoder_trains_toward_a_target():
    enc = SentenceEncoder(20, 8, 16, 1, 4, seed=2)
    toks = torch.tensor([4, 8, 15, 16])
    target = _unit([[1.0] + [0.0] * 15])
    opt = Adam(enc.parameters(), lr=0.01)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = ((enc(toks) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.3 * losses[0]


def test_cross_encoder_logits_and_score():
    pair = torch.tensor([2, 5, 6, 3, 7, 8, 3])
    ce = CrossEncoder(20, 12, 16, 1, 4, seed=3)
    assert ce(pair).shape == (1, 1) and 0.0 < ce.score(pair) < 1.0 and ce.embed_dim == 16
    multi = CrossEncoder(20, 12, 16, 1, 4, num_labels=3, seed=3)
    assert multi(pair).shape == (1, 3)
    backbone = TextTransformer(20, 12, 16, 1, 4, seed=3)
    assert CrossEncoder.wrap(backbone, num_labels=2)(pair).shape == (1, 2)
    ce.score(pair)
    assert all(p.grad is None for p in ce.parameters())                       # scoring runs without a graph


def test_similarity_helpers():
    a = _unit([[1.0, 2.0, 2.0]])
    assert Similarity.cos_sim(a, a) == pytest.approx(1.0, abs=1e-6)
    assert Similarity.cos_sim(_unit([[1.0, 0.0]]), _unit([[0.0, 1.0]])) == 0.0
    with pytest.raises(ValueError):
        Similarity.cos_sim(a, _unit([[1.0, 0.0]]))
    A, B = torch.randn(3, 4, generator=torch.Generator().manual_seed(0)), torch.randn(5, 4, generator=torch.Generator().manual_seed(1))
    assert torch.allclose(Similarity.pairwise(A, B), A @ B.t(), atol=1e-6)
    corpus = _unit([[1.0, 0.0], [0.7, 0.7], [0.0, 1.0], [-1.0, 0.0]])
    hits = Similarity.semantic_search(_unit([[1.0, 0.1]]), corpus, top_k=3)
    assert [h.corpus_index for h in hits[0]] == [0, 1, 2]
    assert hits[0][0].score >= hits[0][1].score >= hits[0][2].score and hits[0][0].corpusIndex == 0
    assert len(Similarity.semantic_search(corpus[:1], corpus, top_k=10)[0]) == 4  # top_k is clamped to the corpus
    with pytest.raises(ValueError):
        Similarity.semantic_search(torch.zeros(1, 3), corpus)


def test_multiple_negatives_ranking_loss():
    e = _unit([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]])
    aligned = SentenceLosses.multiple_negatives_ranking_loss(e, e).mean()
    scrambled = SentenceLosses.multiple_negatives_ranking_loss(e, e[[1, 2, 0]]).mean()
    assert float(aligned) < 1e-6 and float(scrambled) > 10.0
    with pytest.raises(ValueError):
        SentenceLosses.multiple_negatives_ranking_loss(e, e[:2])
    with pytest.raises(ValueError):
        SentenceLosses.multiple_negatives_ranking_loss(e[0], e[0])
    enc = SentenceEncoder(20, 6, 16, 1, 4, seed=5)
    pairs = [([1, 2, 3], [4, 5, 6]), ([7, 8], [9, 10]), ([11, 12, 13], [14, 15])]
    opt = Adam(enc.parameters(), lr=0.01)

    def loss_now():
        a = torch.cat([enc(torch.tensor(p[0])) for p in pairs], 0)
        b = torch.cat([enc(torch.tensor(p[1])) for p in pairs], 0)
        return SentenceLosses.multiple_negatives_ranking_loss(a, b).mean()
    before = float(loss_now().detach())
    for _ in range(10):
        opt.zero_grad()
        loss_now().backward()
        opt.step()
    assert float(loss_now().detach()) < before


def test_cosine_similarity_and_triplet_losses():
    a = _unit([[1.0, 0.0], [0.0, 1.0]])
    assert float(SentenceLosses.cosine_similarity_loss(a, a, torch.ones(2))) == pytest.approx(0.0, abs=1e-9)
    assert float(SentenceLosses.cosine_similarity_loss(a, -a, torch.ones(2))) == pytest.approx(4.0, abs=1e-6)
    with pytest.raises(ValueError):
        SentenceLosses.cosine_similarity_loss(a, a, torch.ones(3))
    with pytest.raises(ValueError):
        SentenceLosses.cosine_similarity_loss(a, a[:1], torch.ones(2))
    anchor, near, far = _unit([[1.0, 0.0]]), _unit([[0.9, 0.1]]), _unit([[-1.0, 0.2]])
    assert float(SentenceLosses.triplet_loss(anchor, near, far, margin=0.5)) == 0.0
    assert float(SentenceLosses.triplet_loss(anchor, far, near, margin=0.5)) > 1.0
    same = SentenceLosses.triplet_loss(anchor, near, near, margin=0.25)
    assert float(same) == pytest.approx(0.25, abs=1e-6)                       # the margin is the floor for ties
    with pytest.raises(ValueError):
        SentenceLosses.triplet_loss(anchor, near, torch.cat([far, far], 0))
