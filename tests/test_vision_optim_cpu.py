"""Vision models, Conv+BN+ReLU folding and the RMSprop / AdaGrad / Adadelta optimizers on CPU."""
import pytest
import torch
import torch.nn.functional as F

from ghost_flow_b200 import nn, optim
from ghost_flow_b200.models import MobileNetV2, resnet18, resnet50, vgg11


def _randomise_bn(m):
    for mod in m.modules():
        if hasattr(mod, "running_mean"):
            mod.running_mean.normal_(0, 0.1)
            mod.running_var.uniform_(0.5, 1.5)
            mod.weight.data.uniform_(0.5, 1.5)
            mod.bias.data.normal_(0, 0.1)


def test_fold_batch_norm_is_exact():
    torch.manual_seed(0)
    conv, bn = nn.Conv2d(5, 8, 3, 2, 1), nn.BatchNorm2d(8)
    _randomise_bn(bn)
    bn.eval()
    x = torch.randn(2, 5, 9, 9)
    want = torch.relu(bn(conv(x)))
    fused = nn.ConvBNReLU(conv, bn)
    assert torch.allclose(fused(x), want, atol=1e-5)
    assert torch.allclose(nn.ConvBNReLU(conv, bn, relu=False)(x), bn(conv(x)), atol=1e-5)
    w, b = nn.fold_batch_norm(conv.weight, conv.bias, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.eps)
    assert torch.allclose(F.conv2d(x, w, b, 2, 1), bn(conv(x)), atol=1e-5)


@pytest.mark.parametrize("make", [lambda: resnet18(10, small_input=True), lambda: resnet50(10, width=16),
                                  lambda: vgg11(10, hidden=32, pool_size=1)])
def test_fused_model_matches_unfused(make):
    torch.manual_seed(0)
    m = make()
    _randomise_bn(m)
    m.eval()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        want = m(x)
        assert nn.fuse_conv_bn_relu(m) > 0
        assert not any(isinstance(mod, nn.BatchNorm2d) for mod in m.modules())
        got = m(x)
    assert torch.allclose(got, want, atol=1e-3, rtol=1e-3)


def test_channels_last_engine_on_cpu_matches_model():
    torch.manual_seed(0)
    m = resnet18(10, small_input=True)
    _randomise_bn(m)
    m.eval()
    x = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        want, got = m(x), m.compile_inference()(x)
    assert (got - want).abs().max() <= 0.03 * want.abs().max() + 0.03


def test_resnet_trains_and_mobilenet_runs():
    torch.manual_seed(0)
    m = resnet18(4, small_input=True, width=8)
    opt = optim.SGD(m.parameters(), lr=0.05, momentum=0.9)
    x, y = torch.randn(8, 3, 16, 16), torch.randint(0, 4, (8,))
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = F.cross_entropy(m(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0]
    assert m.bn1.num_batches_tracked.item() == 8
    assert MobileNetV2(7, 0.5).eval()(torch.randn(1, 3, 64, 64)).shape == (1, 7)


@pytest.mark.parametrize("ours,theirs,kw", [
    (optim.RMSprop, torch.optim.RMSprop, dict(lr=0.01, momentum=0.9, centered=True, weight_decay=0.01)),
    (optim.RMSprop, torch.optim.RMSprop, dict(lr=0.01, alpha=0.9)),
    (optim.AdaGrad, torch.optim.Adagrad, dict(lr=0.1, lr_decay=0.1, weight_decay=0.01)),
    (optim.Adadelta, torch.optim.Adadelta, dict(lr=1.0, rho=0.9, weight_decay=0.01)),
])
def test_extra_optimizers_follow_the_textbook_updates(ours, theirs, kw):
    torch.manual_seed(0)
    a = [torch.randn(5, 3, requires_grad=True), torch.randn(7, requires_grad=True)]
    b = [t.detach().clone().requires_grad_() for t in a]
    oa, ob = ours(a, **kw), theirs(b, **kw)
    for _ in range(6):
        for ps, o in ((a, oa), (b, ob)):
            o.zero_grad()
            sum(((p * p).sum() + p.sin().sum()) for p in ps).backward()
            o.step()
    for p, q in zip(a, b):
        assert torch.allclose(p, q, atol=1e-6)
    assert oa.get_lr() == kw["lr"]


def test_inference_session_falls_back_without_cuda_and_maps_outputs():
    from ghost_flow_b200.models.encoders import BertOutput
    from ghost_flow_b200.nn.inference import _map_tensors

    sess = nn.InferenceSession(nn.Sequential([nn.Linear(4, 3), nn.ReLU()]), nn.InferenceConfig(use_cuda_graph=True))
    x = torch.randn(5, 4)
    assert torch.equal(sess.run(x), sess.model(x))           # CPU input: plain execution, no graph
    out = _map_tensors(BertOutput(torch.ones(2), torch.zeros(1)), lambda t: t + 1)
    assert isinstance(out, BertOutput) and float(out.last_hidden_state.sum()) == 4.0
    nested = _map_tensors({"a": [torch.zeros(1), (torch.ones(1),)], "n": 3}, lambda t: t + 2)
    assert float(nested["a"][1][0]) == 3.0 and nested["n"] == 3


def test_zero_optimizer_fused_arm_refuses_what_it_cannot_run():
    from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer

    p = [torch.nn.Parameter(torch.randn(4, 4))]
    with pytest.raises(RuntimeError, match="bf16 CUDA parameters"):
        ZeRoOptimizer(p, ZeRoConfig.stage2(), comm="fused")        # CPU fp32 parameters, one rank
    with pytest.raises(ValueError):
        ZeRoOptimizer(p, ZeRoConfig.stage2(), comm="carrier-pigeon")
    opt = ZeRoOptimizer(p, ZeRoConfig.stage3(1, 0).with_offload(False))
    assert opt._fc is None and opt.config.stage == 3


def test_fused_ops_skip_the_graph_node_only_when_no_gradient_is_wanted():
    from ghost_flow_b200.ops.fused import _call

    class Double(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, k):
            ctx.save_for_backward(x)
            ctx.k = k
            return x * k

        @staticmethod
        def backward(ctx, dy):
            return dy * ctx.k, None

    x = torch.randn(3, requires_grad=True)
    y = _call(Double, x, 2.0)
    assert y.grad_fn is not None
    y.sum().backward()
    assert torch.allclose(x.grad, torch.full((3,), 2.0))
    with torch.no_grad():
        assert _call(Double, x, 2.0).grad_fn is None
    z = _call(Double, x.detach(), 3.0)
    assert z.grad_fn is None and torch.allclose(z, x.detach() * 3.0)
