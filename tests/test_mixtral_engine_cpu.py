"""The Mixtral expert-parallel training engine on CPU (one rank, fp32) against a plain PyTorch autograd model of the
same network trained with torch.optim.AdamW: attention from the LLaMA module, experts through the dense
per-expert oracle, Switch load-balancing loss added with the configured coefficient."""
import torch

from ghost_flow_b200 import models as M
from ghost_flow_b200.models.configs import MixtralConfig
from ghost_flow_b200.parallel.ep import ExpertParallelMoE, MoEContext
from ghost_flow_b200.parallel.mixtral import MixtralEngine
from ghost_flow_b200.parallel.zero3 import OptimConfig


def _cfg():
    return MixtralConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                         num_local_experts=4, num_experts_per_tok=2, router_aux_loss_coef=0.05)


class _Oracle(torch.nn.Module):
    def __init__(self, cfg, eng):
        super().__init__()
        self.cfg = cfg
        lcfg = M.LLaMAConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=8,
                             num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                             num_key_value_heads=cfg.num_key_value_heads,
                             max_position_embeddings=cfg.max_position_embeddings, rms_norm_eps=cfg.rms_norm_eps,
                             rope_theta=cfg.rope_theta)
        self.lm = M.LLaMAForCausalLM(lcfg)
        sd = eng.state_dict()
        own = self.lm.state_dict()
        own["model.embed_tokens.weight"].copy_(sd["embed_tokens.weight"])
        own["model.norm.weight"].copy_(sd["norm.weight"])
        own["lm_head.weight"].copy_(sd["lm_head.weight"])
        for i in range(cfg.num_hidden_layers):
            pre = f"model.layers.{i}."
            for a, b in (("attn_norm.weight", "attn_norm"), ("attn.wqkv.weight", "wqkv"), ("attn.wo.weight", "wo"),
                         ("ffn_norm.weight", "ffn_norm")):
                own[pre + a].copy_(sd[f"layers.{i}.{b}"])
        P = torch.nn.Parameter
        self.gate = torch.nn.ParameterList([P(e.master["gate"].clone()) for e in eng.experts])
        self.w13 = torch.nn.ParameterList([P(e.master["w13"].clone()) for e in eng.experts])
        self.w2 = torch.nn.ParameterList([P(e.master["w2"].clone()) for e in eng.experts])
        self.moe = eng.moe

    def trained(self):
        mlp = {id(p) for layer in self.lm.model.layers for p in layer.mlp.parameters()}
        return [p for p in self.parameters() if id(p) not in mlp]

    def forward(self, ids, tgt):
        c, m = self.cfg, self.lm.model
        B, S = ids.shape
        cos, sin = m.rope(S, ids.device)
        x = m.embed_tokens(ids)
        aux = 0.0
        for i, layer in enumerate(m.layers):
            x = layer.attn(layer.attn_norm(x), cos, sin, residual=x)
            h = layer.ffn_norm(x).reshape(B * S, -1)
            y = self.moe.dense_reference(h, self.w13[i], self.w2[i], residual=x.reshape(B * S, -1), gate=self.gate[i])
            probs = torch.softmax(h @ self.gate[i].t(), -1)
            idx = probs.topk(c.num_experts_per_tok, -1).indices
            frac = torch.bincount(idx.flatten(), minlength=c.num_local_experts).float() / idx.numel()
            aux = aux + c.num_local_experts * (frac * probs.mean(0)).sum()
            x = y.view(B, S, -1)
        logits = self.lm.lm_head(m.norm(x))
        ce = torch.nn.functional.cross_entropy(logits.view(B * S, -1), tgt.reshape(-1))
        return ce, ce + c.router_aux_loss_coef * aux, aux / len(m.layers)


def test_mixtral_engine_matches_autograd_model_on_cpu():
    cfg = _cfg()
    opt = OptimConfig(lr=3e-3, weight_decay=0.0)
    eng = MixtralEngine(cfg, "cpu", tokens_per_rank=2 * 32, optim=opt, dtype=torch.float32, seed=3)
    ref = _Oracle(cfg, eng)
    tor = torch.optim.AdamW(ref.trained(), lr=opt.lr, betas=(opt.beta1, opt.beta2), eps=opt.eps, weight_decay=0.0)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    ids, tgt = tok[:, :-1], tok[:, 1:]
    ours, theirs = [], []
    for _ in range(5):
        ours.append(float(eng.step(ids, tgt)))
        ce, total, aux = ref(ids, tgt)
        assert abs(float(eng.last_stats["aux_loss"]) - float(aux.detach())) < 3e-3   # a token changing expert moves it
        tor.zero_grad()
        total.backward()
        tor.step()
        theirs.append(float(ce.detach()))
    assert ours[-1] < ours[0] - 0.5
    for a, b in zip(ours, theirs):
        assert abs(a - b) < 2e-3, (ours, theirs)
    for i, e in enumerate(eng.experts):
        for name, p in (("gate", ref.gate[i]), ("w13", ref.w13[i]), ("w2", ref.w2[i])):
            rel = ((e.master[name] - p.detach()).norm() / p.detach().norm()).item()
            assert rel < 5e-3, (i, name, rel)
    wq = eng.gather_unit(eng.layers[1], master=True)["wqkv"]
    wr = ref.lm.model.layers[1].attn.wqkv.weight.detach()
    assert ((wq - wr).norm() / wr.norm()).item() < 5e-3


def test_router_backward_with_auxiliary_loss_matches_autograd():
    """The closed-form router gradient (routing weights and load-balancing loss -> logits) against autograd."""
    torch.manual_seed(0)
    T, E, k, coef = 24, 8, 2, 0.3
    logits = torch.randn(T, E, requires_grad=True)
    dw = torch.randn(T, k)
    probs = torch.softmax(logits, -1)
    top, idx = probs.topk(k, -1)
    w = top / top.sum(-1, keepdim=True)
    frac = torch.bincount(idx.flatten(), minlength=E).float() / idx.numel()
    aux = E * (frac * probs.mean(0)).sum()
    (w * dw).sum().add(coef * aux).backward()
    ctx = MoEContext(None, idx.int(), w.detach(), probs.detach(), None, None, None, None, None)
    got = ExpertParallelMoE._router_backward(ctx, dw, coef, E)
    assert torch.allclose(got, logits.grad, atol=1e-6), (got - logits.grad).abs().max()


def test_mixtral_engine_state_round_trip():
    cfg = _cfg()
    opt = OptimConfig(lr=3e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    a = MixtralEngine(cfg, "cpu", tokens_per_rank=64, optim=opt, dtype=torch.float32, seed=3)
    for _ in range(2):
        a.step(tok[:, :-1], tok[:, 1:])
    b = MixtralEngine(cfg, "cpu", tokens_per_rank=64, optim=opt, dtype=torch.float32, seed=11)
    b.load_shard_state({k: (v.clone() if torch.is_tensor(v) else v) for k, v in a.shard_state().items()})
    la, lb = float(a.step(tok[:, :-1], tok[:, 1:])), float(b.step(tok[:, :-1], tok[:, 1:]))
    assert abs(la - lb) < 1e-6
    sd = a.state_dict()
    assert sd["layers.1.moe.w13"].shape == (4, 256, 64) and sd["layers.0.moe.gate"].shape == (4, 64)
    assert torch.equal(sd["layers.1.moe.w2"], b.state_dict()["layers.1.moe.w2"])


def test_mixtral_engine_on_two_cpu_ranks_matches_one_rank(tmp_path):
    """Expert parallelism = 2 over gloo (tokens gathered, each rank runs its two experts, partial outputs summed
    back; attention units under ZeRO-3) against one rank holding all four experts and the whole batch."""
    import os
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    import _mixtral_cpu_worker as w

    for aux, tol in ((0.0, 2e-5), (0.05, 2e-3)):
        out = str(tmp_path / f"mx{aux}.pt")
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                            "--master-addr", "127.0.0.1", "--master-port", "29691" if aux == 0 else "29693",
                            os.path.join(here, "_mixtral_cpu_worker.py"), out, str(aux)],
                           env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-3000:]
        two = torch.load(out)
        one = w.run(1, 0, aux)
        assert one["losses"][-1] < one["losses"][0]
        # with the auxiliary loss every rank balances its own tokens, one rank the whole batch: close, not equal
        for a, b in zip(two["losses"], one["losses"]):
            assert abs(a - b) < tol, (aux, two["losses"], one["losses"])
        if aux == 0:        # (Adam turns the small difference of the balancing gradients into percents of the weights)
            for k in ("w13", "gate", "wqkv"):
                rel = ((two[k] - one[k]).norm() / one[k].norm()).item()
                assert rel < 1e-4, (k, rel)
