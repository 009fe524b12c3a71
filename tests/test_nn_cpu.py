"""Value-level checks of the framework layer on CPU against closed forms or plain PyTorch."""
import math

import pytest
import torch
import torch.nn.functional as F

import ghost_flow_b200 as gf
from ghost_flow_b200 import nn, optim


def test_reference_python_surface():
    # ghost-flow-py/examples/basic_usage.py shape of usage
    x = gf.Tensor.randn([2, 3]); y = gf.Tensor.ones([2, 3])
    assert (x + y).shape == [2, 3] and x.ndim == 2 and x.size == 6
    a = gf.Tensor([1.0, 2.0, 3.0, 4.0], [2, 2]); b = gf.Tensor([5.0, 6.0, 7.0, 8.0], [2, 2])
    assert (a @ b).tolist() == [19.0, 22.0, 43.0, 50.0]
    assert a.transpose(0, 1).tolist() == [1.0, 3.0, 2.0, 4.0]
    assert a.reshape([4]).shape == [4] and abs(a.softmax(1).sum().item() - 2.0) < 1e-6
    assert a.relu().tolist() == [1, 2, 3, 4] and a.sum().item() == 10 and a.mean().item() == 2.5
    lin = nn.Linear(10, 5)
    assert lin(gf.randn(4, 10)).shape == [4, 5]
    assert (a * 2 + 1000 - a / 2).shape == [2, 2] and ((a - 1) ** 2).mean().item() == 3.5
    assert a.argmax().item() == 3.0 and a.argmax().data.dtype == torch.float32


def test_linear_init_bounds_and_forward():
    lin = nn.Linear(64, 32)
    assert lin.weight.abs().max() <= math.sqrt(6 / 64) + 1e-6
    assert lin.bias.abs().max() <= 1 / math.sqrt(64) + 1e-6
    x = torch.randn(5, 64)
    assert torch.allclose(lin(x), x @ lin.weight.t() + lin.bias, atol=1e-6)


def test_norms_match_formulas():
    x = torch.randn(4, 7, 16)
    ln = nn.LayerNorm(16)
    ref = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-5)
    assert torch.allclose(ln(x), ref, atol=1e-5)
    rn = nn.RMSNorm(16)
    assert torch.allclose(rn(x), x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    bn = nn.BatchNorm1d(16)
    bn(torch.randn(32, 16) * 3 + 1)
    assert bn.running_mean.abs().sum() > 0  # running statistics are updated in training


def test_losses():
    logits = torch.randn(6, 5); tgt = torch.tensor([0, 1, 2, 3, 4, 0])
    assert torch.allclose(nn.cross_entropy(logits, tgt.float()), F.cross_entropy(logits, tgt))
    assert torch.allclose(nn.mse_loss(logits, logits + 1), torch.tensor(1.0))
    p = torch.sigmoid(torch.randn(8)); t = torch.randint(0, 2, (8,)).float()
    assert torch.allclose(nn.binary_cross_entropy(p, t), F.binary_cross_entropy(p, t), atol=1e-5)


def test_flash_and_ring_attention_match_full_attention():
    q, k, v = (torch.randn(2, 96, 32) for _ in range(3))
    for causal in (False, True):
        ref = nn.scaled_dot_product_attention(q, k, v, causal=causal)
        fa = nn.FlashAttention(nn.FlashAttentionConfig(32, 32, causal))(q, k, v)
        assert torch.allclose(fa, ref, atol=1e-5)
        ra = nn.RingAttention(nn.RingAttentionConfig(4, 24, causal)).forward(q, k, v)
        assert torch.allclose(ra, ref, atol=1e-5)
        sa = nn.StripedRingAttention(nn.RingAttentionConfig(4, 24, causal)).forward(q, k, v)
        assert torch.allclose(sa, ref, atol=1e-5)
    assert nn.StripedRingAttention(nn.RingAttentionConfig(4, 64, True)).load_balance_factor() > 0.9


def test_mha_cache_matches_full_forward():
    torch.manual_seed(0)
    mha = nn.MultiHeadAttention(32, 4, causal=True)
    x = torch.randn(1, 6, 32)
    full = mha(x)
    kc = vc = None
    outs = []
    for t in range(6):
        o, _, kc, vc = mha.forward_with_cache(x[:, t:t + 1], kc, vc)
        outs.append(o)
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-5)


def test_moe_matches_per_token_loop_and_trains():
    torch.manual_seed(0)
    cfg = nn.MoEConfig(num_experts=4, top_k=2, d_model=16, d_ff=32)
    moe = nn.MixtureOfExperts(cfg)
    x = torch.randn(10, 16)
    y = moe(x)
    probs = torch.softmax(moe.router.gate(x), -1)
    w, idx = probs.topk(2, -1)
    ref = torch.zeros_like(x)
    for t in range(10):
        for j in range(2):
            ref[t] += w[t, j] * moe.experts[int(idx[t, j])](x[t:t + 1])[0]
        ref[t] /= w[t].sum()
    assert torch.allclose(y, ref, atol=1e-5)
    (y.sum() + moe.get_aux_loss()).backward()
    assert moe.router.gate.weight.grad is not None and sum(moe.get_expert_usage()) == 20
    assert moe.get_stats().aux_loss > 0


def test_lora_merge_is_equivalent():
    l = nn.LoRALinear(8, 6, nn.LoRAConfig(rank=2, alpha=4))
    with torch.no_grad():
        l.lora_b.normal_()
    x = torch.randn(3, 8)
    y = l(x)
    l.merge_weights()
    assert torch.allclose(l(x), y, atol=1e-5)
    l.unmerge_weights()
    assert torch.allclose(l(x), y, atol=1e-5)
    q = nn.QLoRALinear(64, 16)
    assert q(torch.randn(2, 64)).shape == (2, 16) and q.codes.max() < 16


def test_quantization_error_and_ratio():
    w = torch.randn(16, 64)
    for pc in (False, True):
        for sym in (True, False):
            qt = nn.QuantizedTensor.from_tensor(w, nn.QuantizationConfig(per_channel=pc, symmetric=sym))
            assert (qt.dequantize() - w).abs().max() < 0.05 and qt.compression_ratio() == 4.0
    f = nn.QuantizationAwareTraining().fake_quantize(w.requires_grad_())
    f.sum().backward()
    assert torch.equal(w.grad, torch.ones_like(w))
    q8, s = nn.quantize_fp8_blockwise(w.detach())
    assert (nn.dequantize_fp8_blockwise(q8, s) - w.detach()).abs().max() < 0.3


def test_grad_scaler_state_machine():
    sc = nn.GradScaler(nn.MixedPrecisionConfig(nn.PrecisionMode.FP16, 1024.0, growth_interval=2))
    p = torch.nn.Parameter(torch.ones(2))
    opt = optim.SGD([p], lr=0.1)
    p.grad = torch.tensor([float("inf"), 1.0])
    assert not sc.unscale_gradients([p]) and not sc.step(opt) and sc.get_scale() == 512.0
    for _ in range(2):
        p.grad = torch.ones(2) * sc.get_scale()
        assert sc.unscale_gradients([p]) and sc.step(opt)
    assert sc.get_scale() == 1024.0 and torch.allclose(p.data, torch.tensor([0.8, 0.8]))


def test_gradient_checkpointing_same_grads():
    torch.manual_seed(0)
    layers = [nn.Linear(8, 8) for _ in range(4)]
    x = torch.randn(3, 8, requires_grad=True)
    seq = nn.CheckpointedSequential(layers, nn.CheckpointConfig(nn.CheckpointStrategy.All))
    seq(x).sum().backward()
    g1 = [l.weight.grad.clone() for l in layers]
    for l in layers:
        l.weight.grad = None
    nn.Sequential(layers)(x).sum().backward()
    for a, l in zip(g1, layers):
        assert torch.allclose(a, l.weight.grad, atol=1e-6)
    assert seq.manager.get_stats().num_recomputations == 4


def test_optimizers_match_reference_formulas():
    p = torch.nn.Parameter(torch.tensor([1.0]))
    o = optim.SGD([p], lr=0.01)
    p.grad = torch.tensor([1.0]); o.step()
    assert abs(p.item() - 0.99) < 1e-7        # ghostflow-optim/src/sgd.rs test value
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    o = optim.AdamW([p], lr=0.1, weight_decay=0.01)
    m = v = torch.zeros(2); ref = p.detach().clone()
    for t in (1, 2, 3):
        g = ref * 2
        p.grad = p.detach() * 2
        o.step()
        m = 0.9 * m + 0.1 * g; v = 0.999 * v + 0.001 * g * g
        ref = ref * (1 - 0.1 * 0.01) - 0.1 * (m / (1 - 0.9 ** t)) / ((v / (1 - 0.999 ** t)).sqrt() + 1e-8)
    assert torch.allclose(p.detach(), ref, atol=1e-6)


def test_schedulers():
    p = torch.nn.Parameter(torch.zeros(1))
    s = optim.StepLR(optim.SGD([p], lr=1.0), 2, 0.5)
    assert [round(s.step(), 3) for _ in range(4)] == [1.0, 0.5, 0.5, 0.25]
    c = optim.CosineAnnealingLR(optim.SGD([p], lr=1.0), 4)
    lrs = [c.step() for _ in range(4)]
    assert abs(lrs[1] - 0.5) < 1e-9 and abs(lrs[3] - 1.0) < 1e-9      # restarts: t = step % t_max
    w = optim.LinearWarmup(optim.SGD([p], lr=2.0), 4)
    assert [w.step() for _ in range(5)] == [0.5, 1.0, 1.5, 2.0, 2.0]
    r = optim.ReduceLROnPlateau(optim.SGD([p], lr=1.0), factor=0.1, patience=1)
    for loss in (1.0, 1.0, 1.0):
        lr = r.step_with_loss(loss)
    assert abs(lr - 0.1) < 1e-12 and r.optimizer().get_lr() == lr


def test_distillation_prompt_curriculum_privacy():
    kd = nn.KnowledgeDistillation(nn.DistillationConfig.standard(2.0, 0.5))
    s, t = torch.randn(4, 5), torch.randn(4, 5)
    assert kd.compute_loss(s, t, torch.tensor([0, 1, 2, 3])) > 0
    pt = nn.PromptTuning(nn.PromptTuningConfig.short(16))
    assert pt.prepend_prompts(torch.randn(2, 5, 16)).shape == (2, 15, 16)
    pk, pv = nn.PrefixTuning(nn.PrefixTuningConfig(4, 2, 16, 4)).prepend_to_kv(1, torch.randn(2, 5, 4, 4), torch.randn(2, 5, 4, 4))
    assert pk.shape == (2, 9, 4, 4)
    cl = nn.CurriculumLearning(nn.CurriculumConfig(warmup_epochs=2, min_samples_per_batch=2))
    cl.initialize_samples(list(range(10)))
    n0 = cl.select_samples().numel(); cl.next_epoch(); cl.next_epoch()
    assert cl.select_samples().numel() == 10 > n0
    acc = nn.PrivacyAccountant(nn.DPConfig())
    for _ in range(100):
        acc.step()
    assert 0 < acc.get_epsilon() and not acc.is_budget_exhausted()
    dp = nn.DPSGDOptimizer(optim.SGD([torch.nn.Parameter(torch.zeros(3))], lr=0.1), nn.DPConfig(max_grad_norm=1.0))
    clipped = dp.clip_gradients([torch.ones(4, 3) * 10])
    assert torch.allclose(clipped[0].flatten(1).norm(dim=1), torch.ones(4), atol=1e-4)
    sec = nn.SecureAggregation(3)
    ups = [{"w": torch.ones(2) * i} for i in range(3)]
    masked = [sec.mask(i, u) for i, u in enumerate(ups)]
    assert torch.allclose(sum(m["w"] for m in masked), torch.tensor([3.0, 3.0]), atol=1e-5)
    assert not torch.allclose(masked[0]["w"], ups[0]["w"])


def test_adversarial_and_federated():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(4, 3))
    x, y = torch.rand(5, 4), torch.tensor([0, 1, 2, 0, 1])
    atk = nn.AdversarialAttack(nn.AttackConfig(epsilon=0.1, num_iterations=3, step_size=0.05))
    for fn in (atk.fgsm, atk.pgd):
        adv = fn(model, x, y)
        assert (adv - x).abs().max() <= 0.1 + 1e-6
        assert F.cross_entropy(model(adv), y) >= F.cross_entropy(model(x), y) - 1e-6
    server = nn.FederatedServer(torch.nn.Linear(2, 1))
    clients = [nn.FederatedClient(i, torch.nn.Linear(2, 1), num_samples=4, lr=0.1) for i in range(3)]
    data = [(torch.randn(4, 2), torch.randn(4, 1))]
    before = server.model.weight.detach().clone()
    server.run_round(clients, lambda c: data, F.mse_loss)
    assert not torch.equal(before, server.model.weight)


def test_onnx_container_and_inference_session(tmp_path):
    net = nn.Sequential([nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2)])
    m = nn.ONNXModel.from_sequential(net)
    m.save(tmp_path / "m.onnx")
    back = nn.ONNXModel.load(tmp_path / "m.onnx")
    assert [n.op_type for n in back.graph.nodes] == ["Gemm", "ReLU", "Gemm"]
    assert torch.allclose(back.graph.initializers[0].to_tensor(), net[0].weight)
    sess = nn.InferenceSession(net)
    outs = sess.run_batch([torch.randn(4) for _ in range(5)])
    assert len(outs) == 5 and outs[0].shape == (2,)
    seq = torch.nn.Sequential(nn.Conv2d(3, 4, 3, 1, 1), nn.BatchNorm2d(4), nn.ReLU())
    seq[1].running_mean.normal_(); seq[1].running_var.uniform_(0.5, 2)
    seq.eval()
    x = torch.randn(2, 3, 8, 8); ref = seq(x)
    opt = nn.InferenceOptimizer()
    fused = opt.optimize(seq)
    assert torch.allclose(fused(x), ref, atol=1e-5) and opt.get_fusions()


def test_rnn_shapes_and_examples():
    lstm = nn.LSTM(50, 32, 2, False, 0.1)
    out, st = lstm(torch.randn(4, 7, 50))
    assert out.shape == (4, 7, 32) and len(st) == 2
    bi = nn.GRU(50, 16, 1, True, 0.0)
    assert bi(torch.randn(2, 5, 50))[0].shape == (2, 5, 32)
    enc = nn.TransformerEncoder(64, 4, 128, 2, 0.0)
    assert enc(torch.randn(2, 9, 64)).shape == (2, 9, 64)
