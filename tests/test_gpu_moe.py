"""Mixture-of-experts kernels on one GPU: router, dispatch, grouped GEMMs (forward, input and weight gradients),
combine, against a dense fp32 PyTorch restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("T,d,f,E,k", [(512, 256, 384, 8, 2), (1024, 512, 256, 16, 4), (300, 128, 128, 4, 1)])
def test_moe_forward_backward_matches_dense_reference(T, d, f, E, k):
    from ghost_flow_b200.ops import _lib
    from ghost_flow_b200.parallel.ep import ExpertParallelMoE

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    moe = ExpertParallelMoE(d, f, E, k, T, dev, seed=3)
    moe.gate_pad[:E] = (torch.randn(E, d, device=dev) * 0.5).to(torch.bfloat16)    # spread the routing
    x = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(T, d, device=dev, dtype=torch.bfloat16) * 0.1
    y, ctx = moe.forward(x)
    dx = moe.backward(ctx, dy)
    torch.cuda.synchronize()
    _lib.check_status(dev)

    xr = x.float().requires_grad_(True)
    gate = moe.gate.float().requires_grad_(True)
    w13 = moe.w13.float().requires_grad_(True)
    w2 = moe.w2.float().requires_grad_(True)
    moe_gate_saved = moe.gate
    moe.gate = gate
    ref = moe.dense_reference(xr, w13, w2)
    moe.gate = moe_gate_saved
    ref.backward(dy.float())
    assert int(moe.expert_counts().sum()) == T * k
    assert _rel(y, ref) < 2e-2
    assert _rel(dx, xr.grad) < 3e-2
    assert _rel(moe.grads["w2"], w2.grad) < 3e-2
    assert _rel(moe.grads["w13"], w13.grad) < 3e-2
    # with k = 1 the renormalised weight is identically 1 and the router gradient vanishes: compare absolutely
    assert (moe.grads["gate"].float() - gate.grad).norm() < 5e-2 * gate.grad.norm() + 1e-5


def test_router_matches_torch_topk():
    from ghost_flow_b200.parallel import ep

    dev = torch.device("cuda", 0)
    lib = ep._bind()
    from ghost_flow_b200.ops import _lib
    T, E, k = 777, 64, 6
    logits = torch.randn(T, E, device=dev)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    w = torch.empty(T, k, device=dev)
    probs = torch.empty(T, E, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    _lib.check_rc(lib.gf_moe_route(logits.data_ptr(), 1, T, E, k, 1, idx.data_ptr(), w.data_ptr(), probs.data_ptr(),
                                   counts.data_ptr(), _lib.stream_ptr()), "route")
    p = torch.softmax(logits, -1)
    top, ti = p.topk(k, -1)
    assert torch.equal(idx.long(), ti)
    assert torch.allclose(w, top / top.sum(-1, keepdim=True), atol=1e-5)
    assert torch.allclose(probs, p, atol=1e-6)
    assert torch.equal(counts.long(), torch.bincount(ti.flatten(), minlength=E))
