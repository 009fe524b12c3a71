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


def test_llama_cached_generation_uses_the_decode_kernel_and_matches_full_forward(kernel_status):
    """``LLaMAForCausalLM.generate`` on a GPU: the prompt goes through FlashAttention, every new token through the
    decode-attention kernel over the KV cache. The logits of the cached path must agree with a full forward pass
    over the same tokens (no cache), for grouped-query heads too."""
    from ghost_flow_b200.models import LLaMAConfig, LLaMAForCausalLM
    from ghost_flow_b200.ops import _lib

    torch.manual_seed(0)
    cfg = LLaMAConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    model = LLaMAForCausalLM(cfg, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (3, 40), device="cuda")
    with torch.no_grad():
        n0 = _lib.launch_count()
        out = model.generate(ids, max_new_tokens=6)
        assert _lib.launch_count() > n0
        full = model(out[:, :-1])                       # logits of every position without a cache
        caches = model.new_caches(3, 64)
        step_logits = [model(out[:, :40], caches=caches, start_pos=0)[:, -1]]
        for t in range(40, 45):
            step_logits.append(model(out[:, t:t + 1], caches=caches, start_pos=t)[:, -1])
    cached = torch.stack(step_logits, 1).float()        # [3, 6, vocab]
    ref = full[:, 39:45].float()
    rel = ((cached - ref).norm() / ref.norm()).item()
    assert rel < 3e-2, rel
    assert out.shape == (3, 46)
