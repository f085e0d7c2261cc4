"""Decode attention and rope + cache append kernels against fp32 references."""
import pytest
import torch

from dart_pytorch_b200.ops import decode as D

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 4, 1), (64, 8, 2), (128, 8, 8), (64, 6, 2)])
@pytest.mark.parametrize("Sq,Sk,splits", [(1, 700, 0), (1, 33, 1), (3, 257, 4), (1, 2304, 0)])
def test_attn_decode_matches_reference(hd, Hq, Hkv, Sq, Sk, splits):
    torch.manual_seed(0)
    B, cap = 3, Sk + 5
    q = (torch.randn(B * Sq, Hq * hd, device="cuda")).bfloat16()
    kc = (torch.randn(B, cap, Hkv * hd, device="cuda")).bfloat16()
    vc = (torch.randn(B, cap, Hkv * hd, device="cuda")).bfloat16()
    q_off = Sk - Sq
    want = D.attn_decode_reference(q, kc, vc, B, Sq, Sk, Hq, Hkv, hd, q_off)
    got = D.attn_decode(q, kc, vc, B, Sq, Sk, Hq, Hkv, hd, q_off, splits=splits).float()
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), float((got - want).abs().max())
    pos = torch.tensor([q_off], dtype=torch.int32, device="cuda")
    got2 = D.attn_decode(q, kc, vc, B, Sq, cap, Hq, Hkv, hd, 0, splits=splits, pos=pos).float()
    assert torch.allclose(got2, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hd,rot", [(128, 128), (64, 64), (64, 16)])
def test_rope_kv_append_matches_reference(hd, rot):
    torch.manual_seed(1)
    B, S, Hq, Hkv, cap, pos0 = 2, 5, 4, 2, 40, 17
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda").bfloat16()
    kc = torch.zeros(B, cap, Hkv * hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_ref, k_ref, v_ref = qkv.clone().cpu(), kc.clone().cpu(), vc.clone().cpu()
    D.rope_kv_append(q_ref, k_ref, v_ref, B, S, Hq, Hkv, hd, pos0, rotary_dim=rot, base=10000.0)
    q2 = qkv.clone()
    D.rope_kv_append(q2, kc, vc, B, S, Hq, Hkv, hd, pos0, rotary_dim=rot, base=10000.0)
    assert torch.allclose(q2.float().cpu(), q_ref.float(), atol=2e-2)
    assert torch.allclose(kc.float().cpu(), k_ref.float(), atol=2e-2)
    assert torch.equal(vc.cpu(), v_ref)
    assert float(kc[:, :pos0].abs().max()) == 0 and float(kc[:, pos0 + S:].abs().max()) == 0
    kc2, vc2, q3 = torch.zeros_like(kc), torch.zeros_like(vc), qkv.clone()
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    D.rope_kv_append(q3, kc2, vc2, B, S, Hq, Hkv, hd, 0, rotary_dim=rot, base=10000.0, pos=pos)
    assert torch.equal(kc2, kc) and torch.equal(q3, q2)
    with pytest.raises(ValueError):
        D.rope_kv_append(qkv, kc, vc, B, S, Hq, Hkv, hd, cap - 2, rotary_dim=rot)
