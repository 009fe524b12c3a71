"""Benchmark configuration 1: tiny GPT on CPU in fp32 (2 layers, d_model 128, 4 heads, MLP 512 GELU, LayerNorm,
learned positions, vocab 1000, seq 64, batch 8, AdamW lr 3e-4 wd 0.01, Xavier-uniform, seed 0, 20 steps).
The framework's model + optimizer must follow the same loss curve as an independent restatement of the same
formulas in plain PyTorch functional code with torch.optim.AdamW."""
import math

import torch
import torch.nn.functional as F

import ghost_flow_b200 as gf
from ghost_flow_b200.models import GPTConfig, GPTForCausalLM


def _oracle_forward(p, ids, cfg):
    B, S = ids.shape
    x = p["transformer.embeddings.wte.weight"][ids] + p["transformer.embeddings.wpe.weight"][torch.arange(S)]
    H, D = cfg.n_head, cfg.n_embd // cfg.n_head
    for i in range(cfg.n_layer):
        pre = f"transformer.h.{i}."
        h = F.layer_norm(x, (cfg.n_embd,), p[pre + "ln1.weight"], p[pre + "ln1.bias"], cfg.layer_norm_eps)
        qkv = h @ p[pre + "attn.qkv.weight"].t() + p[pre + "attn.qkv.bias"]
        qkv = qkv.view(B, S, 3 * H, D)
        q, k, v = (t.transpose(1, 2) for t in (qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:]))
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        a = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, cfg.n_embd)
        x = x + a @ p[pre + "attn.out_proj.weight"].t() + p[pre + "attn.out_proj.bias"]
        h = F.layer_norm(x, (cfg.n_embd,), p[pre + "ln2.weight"], p[pre + "ln2.bias"], cfg.layer_norm_eps)
        u = h @ p[pre + "mlp.fc1.weight"].t() + p[pre + "mlp.fc1.bias"]
        u = 0.5 * u * (1 + torch.tanh(math.sqrt(2 / math.pi) * (u + 0.044715 * u ** 3)))
        x = x + u @ p[pre + "mlp.fc2.weight"].t() + p[pre + "mlp.fc2.bias"]
    x = F.layer_norm(x, (cfg.n_embd,), p["transformer.ln_f.weight"], p["transformer.ln_f.bias"], cfg.layer_norm_eps)
    return x @ p["transformer.embeddings.wte.weight"].t()


def test_tiny_gpt_20_adamw_steps_match_oracle():
    gf.manual_seed(0)
    cfg = GPTConfig(vocab_size=1000, n_positions=64, n_embd=128, n_layer=2, n_head=4, n_inner=512, dropout=0.0,
                    initializer="xavier_uniform", tie_word_embeddings=True)
    model = GPTForCausalLM(cfg)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (8, 65), generator=g)
    x, y = ids[:, :-1], ids[:, 1:]
    params = {k: v.detach().clone().requires_grad_() for k, v in model.state_dict().items() if k != "lm_head.weight"}
    oracle_opt = torch.optim.AdamW(list(params.values()), lr=3e-4, weight_decay=0.01, betas=(0.9, 0.999), eps=1e-8)
    opt = gf.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01)
    ours, ref = [], []
    for _ in range(20):
        loss, _ = model(x, labels=y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        ours.append(loss.item())
        lo = F.cross_entropy(_oracle_forward(params, x, cfg).reshape(-1, 1000), y.reshape(-1))
        oracle_opt.zero_grad()
        lo.backward()
        oracle_opt.step()
        ref.append(lo.item())
    assert abs(ours[0] - math.log(1000)) < 0.5
    assert ours[-1] < ours[0]
    for a, b in zip(ours, ref):
        assert abs(a - b) < 2e-4, (ours, ref)


def test_timed_cpu_baseline_script_agrees_on_the_first_loss():
    """benchmarks/tiny_gpt_cpu_bench.py times this package's CPU training step against the C++ restatement of the
    reference's forward / loss / AdamW loops; both arms must start from the same loss."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "benchmarks", "tiny_gpt_cpu_bench.py"), "--steps", "3"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["first_loss_agreement"] < 1e-4
    assert d["ours"]["ms_per_step_median"] > 0 and d["reference_formulas"]["ms_per_step_median"] > 0
    assert d["ours"]["loss_last"] < d["ours"]["loss_first"]
