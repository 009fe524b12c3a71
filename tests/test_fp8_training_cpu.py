"""The e4m3 training linear (forward, input gradient and weight gradient all quantised along their contraction axis)
on the CPU emulation path: close to the fp32 layer, and a small network still trains."""
import torch

from ghost_flow_b200.ops import fp8


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_fp8_linear_forward_and_both_gradients_are_close_to_fp32():
    torch.manual_seed(0)
    T, K, N = 64, 128, 96
    x = torch.randn(T, K, requires_grad=True)
    w = (0.1 * torch.randn(N, K)).requires_grad_()
    b = torch.randn(N, requires_grad=True)
    g = torch.randn(T, N)
    y = fp8.fp8_linear(x, w, b)
    y.backward(g)
    xr, wr, br = (t.detach().clone().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g)
    # e4m3 has 3 mantissa bits: relative error of a dot product of random terms is a few percent
    assert _rel(y, yr) < 0.05 and _rel(x.grad, xr.grad) < 0.06 and _rel(w.grad, wr.grad) < 0.06
    assert _rel(b.grad, br.grad) < 1e-2


def test_small_network_trains_with_fp8_linears():
    torch.manual_seed(1)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.GELU(), torch.nn.Linear(64, 64), torch.nn.GELU(),
                              torch.nn.Linear(64, 16))
    assert fp8.convert_linears_to_fp8(net) == 3 and isinstance(net[0], fp8.Fp8TrainLinear)
    x = torch.randn(256, 32)
    target = torch.tanh(x @ torch.randn(32, 16) * 0.3)
    opt = torch.optim.Adam(net.parameters(), lr=3e-3)
    first = last = None
    for _ in range(150):
        loss = torch.nn.functional.mse_loss(net(x), target)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    assert last < 0.35 * first, (first, last)


def test_mxfp8_format_round_trip_and_oracle():
    """Blocks of 32 share an E8M0 power-of-two scale: scales are exact powers of two, the largest element of a block
    lands in e4m3's top binade, the round trip error is e4m3's (3 mantissa bits), and the block-scaled product is
    closer to fp32 than one scale per row when the row mixes magnitudes."""
    torch.manual_seed(0)
    M, N, K = 48, 40, 256
    a = torch.randn(M, K) * torch.logspace(-3, 3, K // 32).repeat_interleave(32)      # magnitudes vary along K
    b = torch.randn(N, K)
    aq, sa = fp8.quantize_mxfp8(a)
    bq, sb = fp8.quantize_mxfp8(b)
    assert aq.dtype == torch.uint8 and sa.shape == (M, K // 32) and sa.dtype == torch.uint8
    top = fp8.dequantize_mxfp8(aq, sa).reshape(M, K // 32, 32).abs().amax(-1) / torch.exp2(sa.float() - 127)
    assert float(top.min()) >= 256 * 0.9 and float(top.max()) <= 448          # the block maximum sits in [2^8, 448]
    assert _rel(fp8.dequantize_mxfp8(aq, sa), a) < 0.04
    ref = a @ b.t()
    mx = fp8.gemm_mxfp8(aq, sa, bq, sb, out_dtype=torch.float32)
    assert _rel(mx, ref) < 0.06
    # what the block scales buy: every block keeps e4m3's relative accuracy, while one scale per row flushes the
    # small-magnitude blocks of the row to zero
    aq0, s0 = fp8.quantize_rows(a, 0)
    blocks = lambda t: t.reshape(M, K // 32, 32)                                  # noqa: E731
    err = lambda d: ((blocks(d) - blocks(a)).norm(dim=(0, 2)) / blocks(a).norm(dim=(0, 2)))   # noqa: E731
    e_mx, e_row = err(fp8.dequantize_mxfp8(aq, sa)), err(fp8.dequantize(aq0, s0, 0))
    assert float(e_mx.max()) < 0.05 and float(e_row[0]) > 0.5 and float(e_row[-1]) < 0.05, (e_mx, e_row)
