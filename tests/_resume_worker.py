"""Worker of tests/test_checkpoint_resume_cpu.py: ZeRO-3 engine on CPU ranks (gloo) that can stop, save its sharded
state, be started again (with the same or another world size) and continue; one rank can be made to fail between
steps. Started by torch.distributed.run."""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import io as gio  # noqa: E402
from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402
from ghost_flow_b200.optim.schedulers import ExponentialLR  # noqa: E402
from ghost_flow_b200.parallel import fault  # noqa: E402
from ghost_flow_b200.parallel.zero3 import Comm, OptimConfig, Zero3LlamaEngine  # noqa: E402

GLOBAL_BATCH = 4


def batch(cfg, step, rank, world):
    """The global batch of a step depends on the step only, so a run continues on the same data at any world size."""
    g = torch.Generator().manual_seed(1000 + step)
    tok = torch.randint(0, cfg.vocab_size, (GLOBAL_BATCH, 33), generator=g)
    per = GLOBAL_BATCH // world
    return tok[rank * per:(rank + 1) * per]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--load", default="")
    ap.add_argument("--save", default="")
    ap.add_argument("--save-at", type=int, default=-1, help="also save after this many steps of this run")
    ap.add_argument("--out", default="")
    ap.add_argument("--die-rank", type=int, default=-1)
    ap.add_argument("--die-step", type=int, default=-1)
    ap.add_argument("--marker-dir", default="")
    args = ap.parse_args()

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=7, comm=Comm())
    sched = ExponentialLR(eng, gamma=0.9)
    position = 0
    if args.load:
        ck = gio.load_sharded(eng, args.load)
        position = gio.restore_training_state(ck.extra, scheduler=sched)["data_position"]
    guard = None
    if args.die_rank >= 0:
        store = dist.distributed_c10d._get_default_store()
        hb = fault.Heartbeat(store, rank, world, interval=0.1).start()
        guard = fault.StepGuard(hb, timeout=1.5)
    losses, lrs = [], []
    exit_code = 0
    for s in range(args.steps):
        if guard is not None:
            if rank == args.die_rank and s == args.die_step:
                guard.report_failure("injected")      # the host-side fault: this rank leaves between two steps
                hb.stop()
                exit_code = 1
                break
            try:
                time.sleep(0.3)                        # lets the failure note of a peer arrive before the launch
                guard.check()
            except fault.PeerFailure as e:
                if args.marker_dir:
                    fault.write_restart_marker(args.marker_dir, args.save, e.ranks, world, eng.step_count, str(e))
                exit_code = fault.EXIT_RESTART
                break
        mine = batch(cfg, position, rank, world)
        losses.append(float(eng.step(mine[:, :-1], mine[:, 1:])))
        position += 1
        lrs.append(sched.step())
        if args.save and s + 1 == args.save_at:
            gio.save_sharded(eng, args.save, extra=gio.training_state_extra(scheduler=sched, data_position=position))
    if exit_code == 0:
        if args.save and args.save_at < 0:
            gio.save_sharded(eng, args.save, extra=gio.training_state_extra(scheduler=sched, data_position=position))
        w = eng.gather_unit(eng.layers[1], master=True)["w_down"]
        m = eng.gather_unit(eng.layers[0], which="m")["wqkv"]
        if rank == 0 and args.out:
            torch.save({"losses": losses, "lrs": lrs, "w": w, "m": m, "step": eng.step_count}, args.out)
        dist.barrier()
        dist.destroy_process_group()
    else:
        if rank == 0 and args.out:
            with open(args.out + ".partial.json", "w") as f:
                json.dump({"losses": losses, "exit": exit_code}, f)
    sys.exit(exit_code)


if __name__ == "__main__":
    main()
