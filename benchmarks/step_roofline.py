"""Budget of the LLaMA ZeRO-3 training step from first principles: what every part of the step would cost at the
measured peaks of this machine, next to what the step was measured at.

    python benchmarks/step_roofline.py [--gpus 8] [--measured-ms 188.8]

Peaks come from ``MEASURED_PEAKS.json`` at the repository root (the copy bandwidth and the sustained cuBLAS bf16 rate
measured on this pool; the documented fallbacks 6650 GB/s and 1400 TFLOP/s if the file is absent) and 770 GB/s per
direction for NVLink peer copies. Pure arithmetic: nothing runs on a GPU. The table separates what is bound by the
tensor cores (GEMMs, attention), by HBM (normalisation, activation, rotary, loss, optimizer) and by NVLink (parameter
all-gather, gradient reduce-scatter; these overlap the compute and only count if they exceed it).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p.get("bf16_tflops_sustained", p["bf16_tflops"]), "measured"
    return 6650.0, 1400.0, "fallback"


def budget(cfg: LLaMAConfig, tokens: int, world: int, persist: bool = True):
    hbm, tflops, src = peaks()
    d, f, L, V = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.vocab_size
    H, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    T = tokens
    qkv = (H + 2 * Hkv) * hd
    layer_params = d * qkv + H * hd * d + 3 * d * f + 2 * d
    params = L * layer_params + 2 * V * d + d
    rows = []

    def add(name, bound, ms, note=""):
        rows.append({"part": name, "bound": bound, "ideal_ms": round(ms, 2), "note": note})

    gemm_flops = 6.0 * (L * (layer_params - 2 * d) + V * d) * T           # forward + dgrad + wgrad; embedding lookup is no GEMM
    add("GEMMs (3 per weight: forward, input gradient, weight gradient)", "tensor", gemm_flops / (tflops * 1e12) * 1e3,
        f"{gemm_flops / 1e12:.0f} TFLOP")
    seq = 4096 if T % 4096 == 0 else T
    attn_fwd = 4.0 * (T // seq) * H * seq * seq * hd / 2                    # causal: half the square
    add("FlashAttention forward + backward (2.5x)", "tensor", L * attn_fwd * 3.5 / (tflops * 1e12) * 1e3,
        f"{L * attn_fwd * 3.5 / 1e12:.1f} TFLOP, at the GEMM rate (the kernels reach 0.55 / 0.38 of the burst rate)")
    bf = 2
    norm = L * 2 * (2 * T * d * bf) + L * 2 * (3 * T * d * bf)            # 2 RMSNorm per layer: fwd r+w, bwd 2r+w
    swiglu = L * (3 * T * f * bf + 5 * T * f * bf)                          # fwd: read 2f write f; bwd: read 3f write 2f
    rope = L * 2 * (2 * T * (H + Hkv) * hd * bf)
    xent = 2 * T * V * bf
    add("RMSNorm, SwiGLU, RoPE, cross-entropy (separate passes over activations)", "HBM",
        (norm + swiglu + rope + xent) / (hbm * 1e9) * 1e3, f"{(norm + swiglu + rope + xent) / 1e9:.1f} GB")
    opt_bytes = params / world * (3 * 4 * 2 + 2 + 2)                        # p, m, v fp32 read + write; bf16 grad in, bf16 weight out
    add("AdamW on this rank's shard (fp32 master and moments)", "HBM", opt_bytes / (hbm * 1e9) * 1e3,
        f"{params / world / 1e9:.2f} B parameters")
    if world > 1:
        frac = (world - 1) / world
        ag = params * bf * frac * (1 if persist else 2)
        rs = params * bf * frac
        add("parameter all-gather over NVLink" + ("" if persist else " (forward and backward)"), "NVLink",
            ag / 770e9 * 1e3, f"{ag / 1e9:.1f} GB in per rank; overlaps the compute")
        add("gradient reduce-scatter over NVLink", "NVLink", rs / 770e9 * 1e3, f"{rs / 1e9:.1f} GB in per rank; overlaps the backward pass")
    compute = sum(r["ideal_ms"] for r in rows if r["bound"] in ("tensor", "HBM"))
    link = sum(r["ideal_ms"] for r in rows if r["bound"] == "NVLink")
    return {"peaks": {"hbm_gbs": hbm, "bf16_tflops_sustained": tflops, "nvlink_gbs_per_direction": 770.0, "source": src},
            "model": {"params": params, "tokens_per_gpu": T, "gpus": world}, "parts": rows,
            "ideal_compute_ms": round(compute, 2), "ideal_link_ms": round(link, 2),
            "ideal_step_ms": round(max(compute, link), 2)}


def budget_mixtral(tokens: int, world: int, layers: int = 32):
    """Mixtral 8x7B shapes, expert parallelism = world, ZeRO-3 for the attention parameters."""
    from ghost_flow_b200.models.configs import MixtralConfig

    hbm, tflops, src = peaks()
    c = MixtralConfig.mixtral_8x7b()
    d, f, V, E, k = c.hidden_size, c.intermediate_size, c.vocab_size, c.num_local_experts, c.num_experts_per_tok
    H, Hkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    T, L, bf = tokens, layers, 2
    attn_params = d * (H + 2 * Hkv) * hd + H * hd * d
    active = L * (attn_params + k * 3 * d * f + E * d) + V * d
    expert_params_rank = L * (E // world if world <= E else 1) * 3 * d * f
    rows = []
    gemm = 6.0 * active * T
    rows.append({"part": "GEMMs on the active parameters (attention, router, two experts per token, head)", "bound": "tensor",
                 "ideal_ms": round(gemm / (tflops * 1e12) * 1e3, 2), "note": f"{gemm / 1e12:.0f} TFLOP"})
    attn = L * 3.5 * 4.0 * H * T * T * hd / 2
    rows.append({"part": "FlashAttention forward + backward", "bound": "tensor",
                 "ideal_ms": round(attn / (tflops * 1e12) * 1e3, 2), "note": f"{attn / 1e12:.1f} TFLOP"})
    passes = L * (2 * 5 * T * d * bf + 8 * T * k * f * bf + 2 * 2 * T * (H + Hkv) * hd * bf) + 2 * T * V * bf
    rows.append({"part": "norms, SwiGLU over the routed rows, RoPE, cross-entropy", "bound": "HBM",
                 "ideal_ms": round(passes / (hbm * 1e9) * 1e3, 2), "note": f"{passes / 1e9:.1f} GB"})
    opt = expert_params_rank * 26 + (L * attn_params + 2 * V * d) / world * 28
    rows.append({"part": "AdamW: this rank's experts (local) and its shard of the dense parameters", "bound": "HBM",
                 "ideal_ms": round(opt / (hbm * 1e9) * 1e3, 2), "note": f"{expert_params_rank / 1e9:.2f} B expert parameters"})
    if world > 1:
        a2a = L * 4 * T * k * d * bf * (world - 1) / world              # dispatch + combine, forward and backward
        rows.append({"part": "token dispatch / combine over NVLink (forward and backward)", "bound": "NVLink",
                     "ideal_ms": round(a2a / 770e9 * 1e3, 2), "note": f"{a2a / 1e9:.1f} GB out per rank"})
    compute = sum(r["ideal_ms"] for r in rows if r["bound"] != "NVLink")
    link = sum(r["ideal_ms"] for r in rows if r["bound"] == "NVLink")
    return {"peaks": {"hbm_gbs": hbm, "bf16_tflops_sustained": tflops, "nvlink_gbs_per_direction": 770.0, "source": src},
            "model": {"active_params": active, "tokens_per_gpu": T, "gpus": world, "layers": L}, "parts": rows,
            "ideal_compute_ms": round(compute, 2), "ideal_link_ms": round(link, 2),
            "ideal_step_ms": round(max(compute, link), 2)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-7b", choices=["llama-7b", "mixtral-8x7b"])
    ap.add_argument("--layers", type=int, default=32, help="mixtral only")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU and step")
    ap.add_argument("--measured-ms", type=float, default=None)
    a = ap.parse_args()
    b = (budget(LLaMAConfig.llama_7b(), a.tokens, a.gpus) if a.model == "llama-7b"
         else budget_mixtral(a.tokens, a.gpus, a.layers))
    print(f"peaks ({b['peaks']['source']}): {b['peaks']['hbm_gbs']:.0f} GB/s copy, "
          f"{b['peaks']['bf16_tflops_sustained']:.0f} TFLOP/s bf16 sustained, 770 GB/s NVLink per direction")
    print(f"{'part':<78}{'bound':>8}{'ideal ms':>10}")
    for r in b["parts"]:
        print(f"{r['part']:<78}{r['bound']:>8}{r['ideal_ms']:>10.2f}   {r['note']}")
    print(f"ideal step = max(compute {b['ideal_compute_ms']} ms, links {b['ideal_link_ms']} ms) = {b['ideal_step_ms']} ms")
    if a.measured_ms:
        b["measured_ms"] = a.measured_ms
        b["fraction_of_ideal"] = round(b["ideal_step_ms"] / a.measured_ms, 3)
        print(f"measured {a.measured_ms} ms -> {b['fraction_of_ideal']} of the ideal step")
    print(json.dumps(b))


if __name__ == "__main__":
    main()
