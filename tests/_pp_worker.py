"""Worker for the GPU pipeline test: a LLaMA stack cut into one stage per GPU, 1F1B over NCCL point-to-point, against the
whole model on one GPU (same weights, same micro-batches, gradients accumulated)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import models as M  # noqa: E402
from ghost_flow_b200.parallel.distributed import PipelineParallel  # noqa: E402


class Stage(torch.nn.Module):
    """Layers [lo, hi) of a LLaMAForCausalLM; the first stage embeds token ids, the last applies norm and head."""

    def __init__(self, lm, lo, hi, first, last):
        super().__init__()
        self.model, self.first, self.last = lm.model, first, last
        self.layers = torch.nn.ModuleList(list(lm.model.layers)[lo:hi])
        self.embed = lm.model.embed_tokens if first else None
        self.norm = lm.model.norm if last else None
        self.head = lm.lm_head if last else None

    def forward(self, x):
        if self.first:
            x = self.embed(x)
        cos, sin = self.model.rope(x.shape[1], x.device)
        for layer in self.layers:
            x = layer(x, cos, sin)
        return self.head(self.norm(x)) if self.last else x


def loss_fn(logits, tgt):
    return torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), tgt.reshape(-1))


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = M.LLaMAConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=4,
                        num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=128)
    torch.manual_seed(0)
    full = M.LLaMAForCausalLM(cfg).to(dev, torch.bfloat16)
    torch.manual_seed(0)
    mine = M.LLaMAForCausalLM(cfg).to(dev, torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (8, 129), generator=g).to(dev)
    x, y = ids[:, :-1], ids[:, 1:]
    m = 4
    # reference: every micro-batch through the whole model on this GPU
    ref_losses = []
    for xi, yi in zip(x.chunk(m), y.chunk(m)):
        l = loss_fn(full(xi), yi)
        (l / m).backward()
        ref_losses.append(l.detach())
    ref_loss = torch.stack(ref_losses).mean()
    per = cfg.num_hidden_layers // world
    stage = Stage(mine, rank * per, (rank + 1) * per, rank == 0, rank == world - 1)
    pp = PipelineParallel(stage, num_micro_batches=m, dtype=torch.bfloat16, device=dev,
                          activation_shape=lambda rows: (rows, 128, cfg.hidden_size))
    loss = pp.run(list(x.chunk(m)), loss_fn, list(y.chunk(m)), rows=x.shape[0] // m)
    torch.cuda.synchronize()
    res = {}
    names = dict(mine.named_parameters())
    refs = dict(full.named_parameters())
    worst = 0.0
    for n, p in names.items():
        if p.grad is None:
            continue
        gr = refs[n].grad.float()
        worst = max(worst, ((p.grad.float() - gr).norm() / (gr.norm() + 1e-12)).item())
    res["grad_rel"] = worst
    res["n_grads"] = sum(p.grad is not None for p in names.values())
    if pp.is_last:
        res["loss_err"] = abs(float(loss) - float(ref_loss))
    res["batches"] = pp.p2p_batches
    torch.save(res, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
