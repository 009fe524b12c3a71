"""The C++ CPU oracle against PyTorch's CPU kernels (independent implementations of the same formulas)."""
import torch

from ghost_flow_b200.ops import cpu_ref


def test_oracle_agrees_with_torch():
    torch.manual_seed(0)
    x = torch.randn(13, 40)
    w = torch.randn(24, 40)
    b = torch.randn(24)
    assert torch.allclose(cpu_ref.linear(x, w, b), x @ w.t() + b, atol=1e-4)
    assert torch.allclose(cpu_ref.matmul(x, w.t().contiguous()), x @ w.t(), atol=1e-4)
    assert torch.allclose(cpu_ref.gelu(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-6)
    assert (cpu_ref.gelu(x, fast_tanh=True) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max() < 0.03
    assert torch.allclose(cpu_ref.silu(x), torch.nn.functional.silu(x), atol=1e-6)
    assert torch.allclose(cpu_ref.softmax(x), torch.softmax(x, -1), atol=1e-6)
    g, bb = torch.randn(40), torch.randn(40)
    assert torch.allclose(cpu_ref.layer_norm(x, g, bb), torch.nn.functional.layer_norm(x, (40,), g, bb, 1e-5), atol=1e-5)
    rms = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * g
    assert torch.allclose(cpu_ref.rms_norm(x, g), rms, atol=1e-5)
    t = torch.randint(0, 40, (13,))
    xl = x.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xl, t)
    ref.backward()
    loss, grad = cpu_ref.cross_entropy(x, t, with_grad=True)
    assert abs(loss - ref.item()) < 1e-5 and torch.allclose(grad, xl.grad, atol=1e-6)
    assert torch.equal(cpu_ref.argmax(x), x.argmax(1).float())


def test_oracle_adamw_attention_conv():
    torch.manual_seed(1)
    p = torch.randn(100)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(100), torch.zeros(100)
    for step in range(1, 4):
        g = torch.randn(100)
        ref.grad = g.clone()
        opt.step()
        cpu_ref.adam_step(p, m, v, g, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(p, ref.detach(), atol=1e-6)
    q, k, vv = torch.randn(2, 9, 8), torch.randn(2, 9, 8), torch.randn(2, 9, 8)
    sd = torch.nn.functional.scaled_dot_product_attention(q, k, vv, is_causal=True)
    assert torch.allclose(cpu_ref.attention(q, k, vv, causal=True), sd, atol=1e-5)
    x, w, b = torch.randn(2, 3, 9, 8), torch.randn(5, 3, 3, 3), torch.randn(5)
    assert torch.allclose(cpu_ref.conv2d(x, w, b, stride=2, padding=1), torch.nn.functional.conv2d(x, w, b, 2, 1), atol=1e-4)
