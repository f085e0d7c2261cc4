"""CPU tests of the CLIP vision tower and its loader, the vision projector, ``LlamaVision``, the MuZero language model
and the ViT heads, case by case after the reference's test/clip_vision_test.dart, test/llama_vision_test.dart,
test/muzero_lm_test.dart, test/vit_test.dart and test/vit_object_detector_test.dart."""
import pytest
import torch

from dart_pytorch_b200 import Adam
from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.io import ClipHFLoader
from dart_pytorch_b200.models import (CLIPVisionConfig, CLIPVisionModel, Llama, LlamaConfig, LlamaVision, MuZeroLM,
                                      ViTClassifier, ViTFaceEmbedding, ViTObjectDetector)
from dart_pytorch_b200.models.vit import VisionEncoder, ViTBackbone
from dart_pytorch_b200.nn.layers import VisionProjector
from dart_pytorch_b200.utils import HungarianAlgorithm


def _x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def _clip(seed=0):
    return CLIPVisionModel(CLIPVisionConfig(image_size=16, patch_size=8, embed_dim=32, num_layers=2, num_heads=4,
                                            ffn_dim=64, seed=seed))


# ------------------------------------------------------------------------------------------------------ CLIP ---
def test_clip_vision_forward_and_protocol():
    cv = _clip()
    assert cv(_x(4, 192)).shape == (5, 32) and isinstance(cv, VisionEncoder)
    assert cv.num_patches == 4 and cv.embed_dim == 32
    for bad in (_x(3, 192), _x(4, 100), _x(2, 3, 8, 8)):
        with pytest.raises(ValueError):
            cv(bad)


def test_clip_loader_prefixes_unused_and_missing_keys():
    src, patches = _clip(seed=1), _x(4, 192)
    want = src(patches).detach()
    state = ClipHFLoader.dump(src)
    assert all(k.startswith("vision_model.") for k in state)
    extra = dict(state, **{"text_model.embeddings.token_embedding.weight": torch.zeros(3, 2), "logit_scale": torch.ones(1)})
    a = _clip(seed=2)
    rep = ClipHFLoader.load_map(a, extra)
    assert rep.consumed_count == len(state) and sorted(rep.unused_keys) == ["logit_scale",
                                                                            "text_model.embeddings.token_embedding.weight"]
    assert torch.allclose(a(patches), want, atol=1e-6)
    bare = {k[len("vision_model."):]: v for k, v in state.items()}
    b = _clip(seed=3)
    assert ClipHFLoader.load_map(b, bare).consumed_count == len(state) and torch.allclose(b(patches), want, atol=1e-6)
    broken = dict(state)
    del broken["vision_model.encoder.layers.1.mlp.fc2.bias"]
    with pytest.raises(ValueError, match="fc2.bias"):
        ClipHFLoader.load_map(_clip(), broken)
    with pytest.raises(ValueError, match="patch_embedding"):
        ClipHFLoader.load_map(_clip(), {"model.layers.0.weight": torch.zeros(1)})


def test_clip_conv_to_linear_matches_a_strided_convolution():
    conv = _x(6, 3, 4, 4)
    image = _x(1, 3, 8, 8, seed=1)
    want = torch.nn.functional.conv2d(image, conv, stride=4)                      # [1, 6, 2, 2]
    lin = ClipHFLoader.conv_to_linear(conv)
    assert lin.shape == (6, 48)
    patch = image[0, :, 4:8, 0:4].permute(1, 2, 0).reshape(-1)                    # patch (row 1, col 0) as (dy, dx, c)
    assert torch.allclose(lin @ patch, want[0, :, 1, 0], atol=1e-5)


def test_clip_presets():
    b32, b16, l14 = ClipHFLoader.base32_config(), ClipHFLoader.base16_config(), ClipHFLoader.large14_config()
    assert (b32.num_patches, b32.embed_dim, b32.num_layers, b32.num_heads, b32.ffn_dim) == (49, 768, 12, 12, 3072)
    assert b16.num_patches == 196 and b16.patch_pixels == 16 * 16 * 3
    assert (l14.num_patches, l14.embed_dim, l14.num_layers, l14.num_heads, l14.ffn_dim) == (256, 1024, 24, 16, 4096)


# ----------------------------------------------------------------------------------------------- LlamaVision ---
def test_vision_projector():
    proj = VisionProjector(12, 20, seed=1)
    assert proj(_x(5, 12)).shape == (5, 20) and len(proj.parameters()) == 4
    with pytest.raises((ValueError, RuntimeError)):
        proj(_x(5, 11))
    x = _x(3, 12)
    want = torch.nn.functional.silu(x @ proj.up.weight.t() + proj.up.bias) @ proj.down.weight.t() + proj.down.bias
    assert torch.allclose(proj(x), want, atol=1e-6)


def test_llama_forward_from_embeddings_matches_token_forward():
    ll = Llama(LlamaConfig(40, 16, 32, 1, 4, 2, 64, seed=2)).eval()
    toks = torch.tensor([1, 5, 9, 2])
    assert torch.allclose(ll.forward_from_embeddings(ll.embed_in(toks)), ll(toks), atol=1e-6)
    with pytest.raises(ValueError):
        ll.forward_from_embeddings(_x(4, 31))


def test_llama_vision_build_shapes_generation_and_parameters():
    cv, ll = _clip(), Llama(LlamaConfig(40, 24, 32, 1, 4, 2, 64, seed=2))
    lv = LlamaVision.build(cv, ll, seed=3)
    patches, toks = _x(4, 192), torch.tensor([1, 5, 9])
    assert lv.num_image_tokens == 5 and lv.encode_image(patches).shape == (5, 32)
    assert lv(patches, toks).shape == (5 + 3, 40)
    out = lv.generate(patches, [1.0, 5.0], 4, temperature=0.0)
    assert len(out) == 6 and out[:2] == [1.0, 5.0]
    stop = out[2]
    assert lv.generate(patches, [1.0, 5.0], 4, temperature=0.0, stop_id=int(stop)) == out[:3]   # stops at stopId
    assert len(lv.parameters()) == len(cv.parameters()) + len(lv.projector.parameters()) + len(ll.parameters())
    with pytest.raises(ValueError):
        LlamaVision(cv, VisionProjector(32, 16), ll)                              # projector width != llama width
    with pytest.raises(ValueError):
        lv.generate(patches, [], 2)


# ---------------------------------------------------------------------------------------------------- MuZero ---
def test_muzero_parts_shapes_and_guards():
    mz = MuZeroLM(30, 8, 16, 5, num_layers=1, seed=1)
    obs = torch.tensor([1, 2, 3, 4])
    s = mz.representation(obs)
    assert s.shape == (1, 16) and bool(torch.isfinite(s).all())
    with pytest.raises(ValueError):
        mz.representation(torch.zeros(9, dtype=torch.long))
    d = mz.dynamics(s, 3)
    assert d.next_state.shape == (1, 16) and d.reward.shape == (1, 1)
    for bad in (-1, 5):
        with pytest.raises(ValueError):
            mz.dynamics(s, bad)
    p = mz.prediction(s)
    assert p.policy.shape == (1, 5) and p.value.shape == (1, 1)
    init, rec = mz.initial_inference(obs), mz.recurrent_inference(s, 2)
    assert init.state.shape == rec.next_state.shape and init.policy.shape == rec.policy.shape
    n = lambda m: len(m.parameters())                                              # noqa: E731
    assert n(mz) == n(mz.representation) + n(mz.dynamics) + n(mz.prediction)


def test_muzero_k_step_loss_decreases():
    mz = MuZeroLM(30, 8, 16, 5, num_layers=1, seed=2)
    obs, actions = torch.tensor([1, 2, 3, 4]), [0, 3, 1]
    targets = torch.tensor([2, 0, 4, 1])
    opt = Adam(mz.parameters(), lr=0.01)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        u = mz.unroll(obs, actions)
        loss = sum(F.cross_entropy(u.policies[k], targets[k:k + 1]).mean() + ((u.values[k] - 0.5) ** 2).mean()
                   for k in range(4)) + sum(((r - 1.0) ** 2).mean() for r in u.rewards)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.5 * losses[0]


# ------------------------------------------------------------------------------------------------------- ViT ---
def test_vit_backbone_classifier_and_face_embedding():
    vit = ViTBackbone(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4, seed=1)
    img = _x(1, 3, 16, 16)
    assert vit(img).shape[-2:] == (5, 32)
    clf = ViTClassifier(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4, num_classes=3, seed=1)
    imgs, labels = _x(4, 3, 16, 16), torch.tensor([0, 1, 2, 1])
    assert clf(imgs).shape == (4, 3)
    opt = Adam(clf.parameters(), lr=0.01)
    first = last = None
    for _ in range(10):
        opt.zero_grad()
        loss = clf.loss(imgs, labels)
        loss.backward()
        opt.step()
        last = float(loss.detach())
        first = last if first is None else first
    assert last < first
    face = ViTFaceEmbedding(image_size=16, patch_size=8, embed_dim=32, num_layers=1, seed=2)
    e = face(imgs).detach()
    assert e.shape == (4, 32) and torch.allclose(e.norm(dim=1), torch.ones(4), atol=1e-5)
    assert ViTFaceEmbedding.cosine_similarity(e[0:1], e[0:1]) == pytest.approx(1.0, abs=1e-5)


def test_vit_object_detector_step_and_hungarian_assignment():
    det = ViTObjectDetector(image_size=16, patch_size=8, embed_dim=32, num_layers=1, num_heads=4, num_queries=3,
                            num_classes=2, seed=3)
    img = _x(1, 3, 16, 16)
    cls, box = det(img)
    cls, box = cls.reshape(-1, cls.shape[-1]), box.reshape(-1, 4)
    assert cls.shape == (3, 3) and box.shape == (3, 4) and float(box.min()) > 0 and float(box.max()) < 1
    target = torch.tensor([[0.2, 0.2, 0.1, 0.1], [0.5, 0.5, 0.3, 0.3], [0.8, 0.7, 0.2, 0.2]])
    opt = Adam(det.parameters(), lr=0.01)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = ((det(img)[1].reshape(-1, 4) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
    assert HungarianAlgorithm([[4, 1, 3], [2, 0, 5], [3, 2, 2]]).get_assignment() == [1, 0, 2]
    assert HungarianAlgorithm([[1, 9, 9], [9, 1, 9], [9, 9, 1]]).get_assignment() == [0, 1, 2]
