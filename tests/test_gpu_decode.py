"""Decode attention over a KV cache against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Hq,Hkv,D,n,splits", [(4, 8, 2, 128, 300, None), (3, 4, 4, 64, 77, 1), (64, 8, 1, 128, 2100, 4)])
def test_attn_decode_matches_reference(B, Hq, Hkv, D, n, splits):
    from ghost_flow_b200.ops import raw

    torch.manual_seed(0)
    dev = "cuda"
    smax = n + 50
    q = torch.randn(B, Hq * D, device=dev, dtype=torch.bfloat16)
    kc = torch.randn(B, smax, Hkv * D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(B, smax, Hkv * D, device=dev, dtype=torch.bfloat16)
    got = raw.attn_decode(q, kc, vc, n, B, Hq, Hkv, D, splits=splits)
    ref = raw.attn_decode(q.cpu(), kc.cpu(), vc.cpu(), n, B, Hq, Hkv, D)
    assert ((got.cpu().float() - ref.float()).norm() / ref.float().norm()) < 1e-2
    lens = torch.randint(1, n, (B,), device=dev, dtype=torch.int32)
    got2 = raw.attn_decode(q, kc, vc, lens, B, Hq, Hkv, D, splits=splits)
    ref2 = raw.attn_decode(q.cpu(), kc.cpu(), vc.cpu(), lens.cpu(), B, Hq, Hkv, D)
    assert ((got2.cpu().float() - ref2.float()).norm() / ref2.float().norm()) < 1e-2
