"""A whole training step (zero_grad, forward, backward, sharded AdamW) recorded once in a CUDA graph and replayed,
against the same steps launched one by one."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(graph: bool, steps: int = 6):
    from ghost_flow_b200.models.configs import GPTConfig
    from ghost_flow_b200.models.gpt import GPTForCausalLM
    from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer, ZeRoStage
    from ghost_flow_b200.utils import GraphedStep

    cfg = GPTConfig(vocab_size=512, n_positions=128, n_embd=128, n_layer=2, n_head=4, n_inner=512)
    cfg.dropout = 0.0
    torch.manual_seed(0)
    model = GPTForCausalLM(cfg).to("cuda", torch.bfloat16)
    opt = ZeRoOptimizer(model.parameters(), ZeRoConfig(stage=ZeRoStage.Stage2, lr=1e-3, betas=(0.9, 0.95),
                                                       weight_decay=0.1, bucket_size=150_000), capturable=graph)
    g = torch.Generator().manual_seed(7)
    batches = [torch.randint(0, cfg.vocab_size, (2, 129), generator=g).cuda() for _ in range(steps)]

    def train(x, y):
        opt.zero_grad()
        res = model(x, labels=y)
        loss = res[0] if isinstance(res, tuple) else res
        loss.backward()
        opt.step()
        return loss.detach()

    if not graph:
        losses = [float(train(b[:, :-1].contiguous(), b[:, 1:].contiguous())) for b in batches]
    else:
        # the warm-up steps are real steps on the first batch's buffers: feed them batch by batch instead
        losses = [float(train(b[:, :-1].contiguous(), b[:, 1:].contiguous())) for b in batches[:2]]
        gs = GraphedStep(train, (batches[2][:, :-1].contiguous(), batches[2][:, 1:].contiguous()), warmup=0)
        for b in batches[2:]:
            losses.append(float(gs(b[:, :-1].contiguous(), b[:, 1:].contiguous())))
        assert gs.replays == steps - 2
    torch.cuda.synchronize()
    return losses, [p.detach().float().clone() for p in model.parameters()], opt


def test_graph_replay_of_a_training_step_matches_eager(kernel_status):
    eager, pe, _ = _run(False)
    graphed, pg, opt = _run(True)
    assert int(opt._step_dev) == 6 and opt.step_count == 3       # host count stops at the recording, device goes on
    assert eager[-1] < eager[0]
    for a, b in zip(eager, graphed):
        assert abs(a - b) < 2e-2, (eager, graphed)
    worst = max(((a - b).norm() / (a.norm() + 1e-12)).item() for a, b in zip(pe, pg))
    assert worst < 2e-2, worst
