"""CPU (gloo) worker for the distributed wrapper tests. argv: <case> <out-file>."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(12, 24), torch.nn.Tanh(), torch.nn.Linear(24, 24), torch.nn.Tanh(),
                               torch.nn.Linear(24, 4))


def data(n=16):
    g = torch.Generator().manual_seed(7)
    return torch.randn(n, 12, generator=g), torch.randn(n, 4, generator=g)


def case_ddp(rank, world, out):
    from ghost_flow_b200.parallel.distributed import DistributedDataParallel
    x, y = data()
    ref = model()
    torch.nn.functional.mse_loss(ref(x), y).backward()
    m = DistributedDataParallel(model(), bucket_mb=0.001)
    xs, ys = x.chunk(world), y.chunk(world)
    loss = torch.nn.functional.mse_loss(m(xs[rank]), ys[rank])
    loss.backward()
    m.finish()
    err = max((p.grad - q.grad).abs().max().item() for p, q in zip(m.module.parameters(), ref.parameters()))
    # accumulation: two micro-steps, sync only on the second
    m.zero_grad()
    m2 = DistributedDataParallel(model(), bucket_mb=0.001, accumulation_steps=2)
    halves_x, halves_y = xs[rank].chunk(2), ys[rank].chunk(2)
    due = [m2.backward(torch.nn.functional.mse_loss(m2(a), b)) for a, b in zip(halves_x, halves_y)]
    err2 = max((p.grad - q.grad).abs().max().item() for p, q in zip(m2.module.parameters(), ref.parameters()))
    # a parameter that takes no part in the forward pass on ANY rank, and one used only on rank 0: their hooks
    # never fire (everywhere / on rank 1), yet after finish() every rank must hold the same averaged gradients
    class Branchy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(3)
            self.a = torch.nn.Linear(12, 4)
            self.unused = torch.nn.Linear(12, 4)
            self.sometimes = torch.nn.Linear(12, 4)

        def forward(self, x, use_branch):
            y = self.a(x)
            return y + self.sometimes(x) if use_branch else y

    ref3 = Branchy()
    l_ref = sum(torch.nn.functional.mse_loss(ref3(xs[r], r == 0), ys[r]) for r in range(world)) / world
    l_ref.backward()
    m3 = DistributedDataParallel(Branchy(), bucket_mb=0.0001)
    torch.nn.functional.mse_loss(m3(xs[rank], rank == 0), ys[rank]).backward()
    m3.finish()
    err3 = 0.0
    for (n, p_), (_, q) in zip(m3.module.named_parameters(), ref3.named_parameters()):
        want = q.grad if q.grad is not None else torch.zeros_like(q)
        err3 = max(err3, (p_.grad - want).abs().max().item())
    # two backward passes after one forward each, without an intervening reset by hand
    m3.zero_grad()
    for _ in range(2):
        torch.nn.functional.mse_loss(m3(xs[rank], rank == 0), ys[rank]).backward()
        m3.finish()
    return {"ddp_grad_err": err, "ddp_accum_err": err2, "due": due, "ddp_unused_err": err3}


def case_zero(rank, world, out):
    from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer, ZeRoStage
    x, y = data()
    ref = model()
    opt_ref = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    res = {}
    for stage in (ZeRoStage.Stage1, ZeRoStage.Stage2, ZeRoStage.Stage3):
        m = model()
        ref.load_state_dict(model().state_dict())
        opt_ref = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        cfg = ZeRoConfig(stage=stage, world_size=world, rank=rank, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1,
                         bucket_size=500, cpu_offload=(stage == ZeRoStage.Stage3))
        opt = ZeRoOptimizer(m.parameters(), cfg)
        xs, ys = x.chunk(world), y.chunk(world)
        for _ in range(4):
            opt_ref.zero_grad()
            torch.nn.functional.mse_loss(ref(x), y).backward()
            opt_ref.step()
            opt.zero_grad()
            torch.nn.functional.mse_loss(m(xs[rank]), ys[rank]).backward()
            opt.step()
        res[f"zero{int(stage)}_param_err"] = max((p - q).abs().max().item() for p, q in zip(m.parameters(), ref.parameters()))
        st = opt.get_stats()
        res[f"zero{int(stage)}_savings"] = st.memory_savings_ratio()
        res[f"zero{int(stage)}_owned"] = st.owned_params
    return res


def case_zero_hooks(rank, world, out):
    """The hook-driven schedule of the generic ZeRO optimizer on CPU ranks: buckets launched from gradient hooks as
    their last gradient arrives, a parameter without a gradient (its bucket is launched by step()), gradient
    accumulation over two backward passes with no_sync()."""
    from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer, ZeRoStage
    x, y = data()
    xs, ys = x.chunk(world), y.chunk(world)

    class WithUnused(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.net = model()
            self.extra = torch.nn.Linear(3, 3)     # never used in the forward pass: no gradient, hook never fires

        def forward(self, t):
            return self.net(t)

    build = WithUnused

    ref = build()
    opt_ref = torch.optim.AdamW([p for p in ref.parameters()], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = build()
    m.load_state_dict(ref.state_dict())
    cfg = ZeRoConfig(stage=ZeRoStage.Stage2, world_size=world, rank=rank, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1,
                     bucket_size=300)
    opt = ZeRoOptimizer(m.parameters(), cfg, overlap=True)
    launched_in_backward = []
    res = {}
    for step in range(4):
        opt_ref.zero_grad()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        for p in ref.extra.parameters():
            p.grad = torch.zeros_like(p)           # the flat optimizer decays every parameter of its buckets
        opt_ref.step()
        opt.zero_grad()
        if step % 2 == 0:
            torch.nn.functional.mse_loss(m(xs[rank]), ys[rank]).backward()
        else:                                       # the same gradient from two half-weighted backward passes
            with opt.no_sync():
                (0.5 * torch.nn.functional.mse_loss(m(xs[rank]), ys[rank])).backward()
                assert not opt._launched
            (0.5 * torch.nn.functional.mse_loss(m(xs[rank]), ys[rank])).backward()
        launched_in_backward.append(len(opt._launched))
        opt.step()
        assert not opt._launched and not opt._open
    res["hooks_param_err"] = max((p - q).abs().max().item() for p, q in zip(m.parameters(), ref.parameters()))
    # a second backward pass without no_sync() would add to gradients that were already consumed: refused
    opt.zero_grad()
    torch.nn.functional.mse_loss(m(xs[rank]), ys[rank]).backward()
    try:
        torch.nn.functional.mse_loss(m(xs[rank]), ys[rank]).backward()
        res["hooks_second_backward_refused"] = False
    except RuntimeError as e:
        res["hooks_second_backward_refused"] = "no_sync" in str(e)
    opt.step()
    res["hooks_buckets"] = len(opt.buckets)
    res["hooks_launched_in_backward"] = launched_in_backward
    return res


def case_pipeline(rank, world, out):
    from ghost_flow_b200.parallel.distributed import PipelineParallel
    x, y = data(16)
    full = model()
    layers = list(full)
    loss_ref = torch.nn.functional.mse_loss(full(x), y)
    loss_ref.backward()
    cut = [0, 2, 5] if world == 2 else [0, 2, 4, 5]
    stage = torch.nn.Sequential(*[l for l in list(model())[cut[rank]:cut[rank + 1]]])
    pp = PipelineParallel(stage, num_micro_batches=4, activation_shape=lambda rows: (rows, 24))
    micro_x = pp.create_micro_batches(x)
    micro_y = pp.create_micro_batches(y)
    loss = pp.run(micro_x, lambda o, t: torch.nn.functional.mse_loss(o, t), micro_y, rows=micro_x[0].shape[0])
    ref_params = [p for l in layers[cut[rank]:cut[rank + 1]] for p in l.parameters()]
    err = max((p.grad - q.grad).abs().max().item() for p, q in zip(stage.parameters(), ref_params))
    res = {"pp_grad_err": err}
    if pp.is_last:
        res["pp_loss_err"] = abs(loss.item() - loss_ref.item())
    return res


def case_context(rank, world, out):
    from ghost_flow_b200.ops import raw
    from ghost_flow_b200.parallel.context import ContextParallelAttention, UlyssesAttention
    B, S, H, Hkv, D = 1, 32, 4, 2, 16
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B * S * world, H * D, generator=g)
    k = torch.randn(B * S * world, Hkv * D, generator=g)
    v = torch.randn(B * S * world, Hkv * D, generator=g)
    do = torch.randn(B * S * world, H * D, generator=g)
    o_ref, lse_ref = raw.attn_fwd(q, k, v, B, S * world, H, Hkv, D, True)
    dq_r, dk_r, dv_r = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    raw.attn_bwd(q, k, v, o_ref, do, lse_ref, dq_r, dk_r, dv_r, B, S * world, H, Hkv, D, True)
    sl = slice(rank * S, (rank + 1) * S)
    res = {}
    cp = ContextParallelAttention(B, S, H, Hkv, D, causal=True)
    o, lse = cp.forward(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous())
    dq, dk, dv = cp.backward(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), o, lse, do[sl].contiguous())
    res["ring_o"] = (o - o_ref[sl]).abs().max().item()
    res["ring_dq"] = (dq - dq_r[sl]).abs().max().item()
    res["ring_dk"] = (dk - dk_r[sl]).abs().max().item()
    res["ring_dv"] = (dv - dv_r[sl]).abs().max().item()
    ul = UlyssesAttention(B, S, H, Hkv, D, causal=True)
    o2, ctx = ul.forward(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous())
    dq2, dk2, dv2 = ul.backward(ctx, do[sl].contiguous())
    res["ulysses_o"] = (o2 - o_ref[sl]).abs().max().item()
    res["ulysses_dq"] = (dq2 - dq_r[sl]).abs().max().item()
    res["ulysses_dk"] = (dk2 - dk_r[sl]).abs().max().item()
    # zig-zag assignment: rank r holds chunks r and 2 * world - 1 - r of the sequence
    from ghost_flow_b200.parallel.context import ZigZagContextParallelAttention, causal_work_per_rank, zigzag_rows
    rows = zigzag_rows(S * world, world, rank)
    zz = ZigZagContextParallelAttention(B, S, H, Hkv, D)
    qz, kz, vz, doz = (t[rows].contiguous() for t in (q, k, v, do))
    oz, lz = zz.forward(qz, kz, vz)
    dqz, dkz, dvz = zz.backward(qz, kz, vz, oz, lz, doz)
    res["zigzag_o"] = (oz - o_ref[rows]).abs().max().item()
    res["zigzag_dq"] = (dqz - dq_r[rows]).abs().max().item()
    res["zigzag_dk"] = (dkz - dk_r[rows]).abs().max().item()
    res["zigzag_dv"] = (dvz - dv_r[rows]).abs().max().item()
    res["balance_contiguous"] = max(causal_work_per_rank(world, False)) * world
    res["balance_zigzag"] = max(causal_work_per_rank(world, True)) * world
    return res


def case_fault(rank, world, out):
    """Rank 1 fails on the host at step 3 and leaves between steps; rank 0 must learn of it before its next
    collective (heartbeat / failure note in the store) and must not hang."""
    from ghost_flow_b200.parallel.fault import FaultInjector, Heartbeat, PeerFailure, StepGuard, Watchdog
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.05).start()
    guard = StepGuard(hb, timeout=1.0)
    inj = FaultInjector(raise_at=3 if rank == 1 else None)
    steps_done, detected, t0 = 0, None, time.monotonic()
    t = torch.ones(4)
    try:
        for step in range(1, 8):
            try:
                inj.before_step(hb)
            except RuntimeError as e:
                guard.report_failure(str(e))
                hb.stop()
                raise
            if rank == 0 and step >= 3:
                guard.wait_healthy(1.5)        # gives the failing rank time to publish, then checks before launching
            else:
                guard.check()
            dist.all_reduce(t)
            steps_done += 1
    except PeerFailure as e:
        detected = e.ranks
    except RuntimeError:
        detected = "self"
    with Watchdog(0.05) as wd:
        time.sleep(0.2)
    hb.stop()
    return {"steps_done": steps_done, "detected": detected, "seconds": time.monotonic() - t0, "watchdog": wd.fired}


def case_syncbn(rank, world, out):
    """SyncBatchNorm over two ranks against plain batch norm over the concatenated batch."""
    from ghost_flow_b200 import nn
    torch.manual_seed(3)
    x = torch.randn(8, 5, 4, 4)
    w = torch.randn(8, 5, 4, 4)
    ref = torch.nn.BatchNorm2d(5)
    ref.weight.data.uniform_(0.5, 1.5)
    ref.bias.data.normal_()
    xr = x.clone().requires_grad_()
    (ref(xr) * w).sum().backward()
    net = nn.Sequential([nn.BatchNorm2d(5)])
    net[0].load_state_dict(ref.state_dict())
    net[0].running_mean.zero_()
    net[0].running_var.fill_(1.0)
    net = nn.SyncBatchNorm.convert(net)
    assert isinstance(net[0], nn.SyncBatchNorm)
    xs = x.chunk(world)[rank].clone().requires_grad_()
    y = net(xs)
    (y * w.chunk(world)[rank]).sum().backward()
    wg = net[0].weight.grad.clone()
    dist.all_reduce(wg)
    with torch.no_grad():
        y_ref = ref(x)  # second call only to compare outputs; running stats of `ref` advance twice
    return {"y_err": (y - y_ref.chunk(world)[rank]).abs().max().item(),
            "dx_err": (xs.grad - xr.grad.chunk(world)[rank]).abs().max().item(),
            "dw_err": (wg - ref.weight.grad).abs().max().item(),
            "rv_err": (net[0].running_var - (0.9 + 0.1 * x.var((0, 2, 3), unbiased=True))).abs().max().item(),
            "rm_err": (net[0].running_mean - 0.1 * x.mean((0, 2, 3))).abs().max().item()}


def main():
    case, out = sys.argv[1], sys.argv[2]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    res = globals()[f"case_{case}"](rank, world, out)
    torch.save(res, f"{out}.{rank}")
    if case != "fault":
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
