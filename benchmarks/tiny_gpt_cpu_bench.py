"""Benchmark configuration 1 on the CPU: the tiny GPT (2 layers, d_model 128, 4 heads, MLP 512 GELU, LayerNorm,
learned positions, vocab 1000, seq 64, batch 8, AdamW lr 3e-4 wd 0.01, Xavier-uniform, seed 0), 20 steps.

    python benchmarks/tiny_gpt_cpu_bench.py [--steps 20] [--threads N]

Two arms, both fp32, single process:

* ``ours``: this package's model and optimizer on CPU tensors: forward, backward and AdamW, i.e. a full training
  step (the loss curve of this arm is the one ``tests/test_tiny_gpt_cpu.py`` checks against an independent oracle).
* ``reference-formulas``: what the reference itself can execute for this model, restated in C++ with its own loop
  structure (``csrc/cpu_ref.cpp``: serial 64-blocked matmul as in ghostflow-core/src/ops/matmul.rs:91-119, per-row
  LayerNorm / softmax, tanh GELU, the element loop of ghostflow-optim/src/adam.rs:162-197): the forward pass, the
  loss, and one AdamW pass over every parameter. The reference has no backward pass
  (ghostflow-autograd/src/backward.rs:11-25), so this arm does LESS work per step than ``ours``; its time is a
  lower bound of what a training step would cost there.

Prints one JSON line with ms per step of both arms (median over the steps after the first).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import ghost_flow_b200 as gf  # noqa: E402
from ghost_flow_b200.models import GPTConfig, GPTForCausalLM  # noqa: E402
from ghost_flow_b200.ops import cpu_ref  # noqa: E402


def reference_formulas_step(p, cfg, x, y, moments, step):
    """Forward + loss + AdamW element loops through the C++ restatement of the reference's CPU code."""
    B, S = x.shape
    H, D = cfg.n_head, cfg.n_embd // cfg.n_head
    h = (p["transformer.embeddings.wte.weight"][x] + p["transformer.embeddings.wpe.weight"][torch.arange(S)])
    h = h.reshape(B * S, cfg.n_embd)
    for i in range(cfg.n_layer):
        pre = f"transformer.h.{i}."
        n1 = cpu_ref.layer_norm(h, p[pre + "ln1.weight"], p[pre + "ln1.bias"], cfg.layer_norm_eps)
        qkv = cpu_ref.linear(n1, p[pre + "attn.qkv.weight"], p[pre + "attn.qkv.bias"]).view(B, S, 3 * H, D)
        outs = []
        for b in range(B):
            q, k, v = (qkv[b, :, j * H:(j + 1) * H].transpose(0, 1).contiguous() for j in range(3))
            outs.append(cpu_ref.attention(q, k, v, causal=True).transpose(0, 1).reshape(S, cfg.n_embd))
        a = torch.cat(outs, 0)
        h = h + cpu_ref.linear(a, p[pre + "attn.out_proj.weight"], p[pre + "attn.out_proj.bias"])
        n2 = cpu_ref.layer_norm(h, p[pre + "ln2.weight"], p[pre + "ln2.bias"], cfg.layer_norm_eps)
        u = cpu_ref.gelu(cpu_ref.linear(n2, p[pre + "mlp.fc1.weight"], p[pre + "mlp.fc1.bias"]))
        h = h + cpu_ref.linear(u, p[pre + "mlp.fc2.weight"], p[pre + "mlp.fc2.bias"])
    h = cpu_ref.layer_norm(h, p["transformer.ln_f.weight"], p["transformer.ln_f.bias"], cfg.layer_norm_eps)
    logits = cpu_ref.linear(h, p["transformer.embeddings.wte.weight"])
    loss = cpu_ref.cross_entropy(logits, y.reshape(-1))
    for name, w in p.items():      # the optimizer's element loop, on stand-in gradients (there is no backward)
        m, v = moments[name]
        cpu_ref.adam_step(w, m, v, w, lr=3e-4, weight_decay=0.01, step=step)
    return loss


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--threads", type=int, default=0, help="torch CPU threads for the `ours` arm (0: leave as is)")
    args = ap.parse_args()
    if args.threads > 0:
        torch.set_num_threads(args.threads)
    gf.manual_seed(0)
    cfg = GPTConfig(vocab_size=1000, n_positions=64, n_embd=128, n_layer=2, n_head=4, n_inner=512, dropout=0.0,
                    initializer="xavier_uniform", tie_word_embeddings=True)
    model = GPTForCausalLM(cfg)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (8, 65), generator=g)
    x, y = ids[:, :-1], ids[:, 1:]
    params = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items() if k != "lm_head.weight"}
    moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in params.items()}

    opt = gf.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01)
    ours_ms, losses = [], []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        loss, _ = model(x, labels=y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
        ours_ms.append((time.perf_counter() - t0) * 1e3)

    ref_ms, ref_loss0 = [], None
    for s in range(args.steps):
        t0 = time.perf_counter()
        l = reference_formulas_step(params, cfg, x, y, moments, s + 1)
        ref_ms.append((time.perf_counter() - t0) * 1e3)
        ref_loss0 = l if ref_loss0 is None else ref_loss0

    print(json.dumps({
        "config": "tiny GPT, CPU fp32, batch 8 x 64 tokens, 20 AdamW steps",
        "threads": torch.get_num_threads(),
        "ours": {"what": "forward + backward + AdamW", "ms_per_step_median": statistics.median(ours_ms[1:]),
                 "ms_first_step": ours_ms[0], "total_ms": sum(ours_ms), "loss_first": losses[0],
                 "loss_last": losses[-1]},
        "reference_formulas": {"what": "forward + loss + AdamW element loops (no backward exists)",
                               "ms_per_step_median": statistics.median(ref_ms[1:]), "total_ms": sum(ref_ms),
                               "loss_first": float(ref_loss0)},
        "first_loss_agreement": abs(losses[0] - float(ref_loss0)),
        "ln_vocab": math.log(1000),
    }))


if __name__ == "__main__":
    main()
