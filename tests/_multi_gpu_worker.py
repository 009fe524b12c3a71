"""Worker for the multi-GPU tests (launched with torch.distributed.run, one rank per GPU): runs the ZeRO-3
engine with the requested collective path and writes rank 0's loss curve and one gathered weight."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.comm import make_comm  # noqa: E402
from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine  # noqa: E402


def main():
    kind, out, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LLaMAConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512)
    base = kind.split("_")[0]
    persist = None if "nopersist" not in kind else False
    comm = make_comm(base, dev)
    clip = 0.5 if "clip" in kind else None      # well under the first steps' gradient norm: the bound bites
    eng = Zero3LlamaEngine(cfg, dev, optim=OptimConfig(lr=2e-3, max_grad_norm=clip), comm=comm, seed=5,
                           persist_gathered=persist)
    g = torch.Generator().manual_seed(99)
    tok = torch.randint(0, cfg.vocab_size, (world, 257), generator=g)
    mine = tok[rank:rank + 1].to(dev)
    if "resume" in kind:
        # half of the steps, a sharded checkpoint, then a NEW communicator and engine in the same job (fresh signal
        # pads and counters, as in a restarted process) that loads it and continues: the step counter starts
        # at steps / 2 while every flag of the new pads is zero
        from ghost_flow_b200 import io as gio

        ckdir = out + ".ck"
        losses = [float(eng.step(mine[:, :-1], mine[:, 1:])) for _ in range(steps // 2)]
        gio.save_sharded(eng, ckdir)
        torch.cuda.synchronize()
        dist.barrier()
        del eng
        comm = make_comm(base, dev)
        eng = Zero3LlamaEngine(cfg, dev, optim=OptimConfig(lr=2e-3), comm=comm, seed=1234, persist_gathered=persist)
        gio.load_sharded(eng, ckdir)
        assert eng.step_count == steps // 2
        losses += [float(eng.step(mine[:, :-1], mine[:, 1:])) for _ in range(steps - steps // 2)]
    else:
        losses = [float(eng.step(mine[:, :-1], mine[:, 1:])) for _ in range(steps)]
    torch.cuda.synchronize()
    _lib.check_status(dev)
    w = eng.gather_unit(eng.layers[2], master=True)["w_gate_up"].cpu()
    if rank == 0:
        torch.save({"losses": losses, "w": w, "fused": bool(getattr(comm, "fused", False)),
                    "stats": dict(eng.last_stats), "multimem": bool(getattr(comm, "arena_mc", 0))}, out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
