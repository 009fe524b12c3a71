"""fp8 quantisation kernels and the scaled tcgen05 fp8 GEMM against fp32 PyTorch on the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("mode", [0, 1])
def test_quantise_rows_matches_torch(mode):
    from ghost_flow_b200.ops import fp8

    x = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16) * 3
    q, s = fp8.quantize_rows(x, mode)
    qc, sc = fp8.quantize_rows(x.cpu(), mode)
    assert torch.allclose(s.cpu(), sc, rtol=1e-6)
    # bytes may differ by one code where x / scale sits on a rounding boundary; the values must agree closely
    d = fp8.dequantize(q.cpu(), s.cpu(), mode)
    assert _rel(d, fp8.dequantize(qc, sc, mode)) < 8e-3
    assert _rel(d, x.cpu()) < 4e-2


def test_quantise_block128_matches_torch():
    from ghost_flow_b200.ops import fp8

    w = torch.randn(320, 256, device="cuda", dtype=torch.bfloat16)
    q, s = fp8.quantize_block128(w)
    qc, sc = fp8.quantize_block128(w.cpu())
    assert torch.allclose(s.cpu(), sc, rtol=1e-6)
    assert _rel(fp8.dequantize(q.cpu(), s.cpu(), 1, weight=True), fp8.dequantize(qc, sc, 1, weight=True)) < 8e-3


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 777 // 8 * 8, 1024), (4096, 4096, 4096)])
def test_fp8_gemm_matches_dequantised_reference(mode, M, N, K):
    from ghost_flow_b200.ops import _lib, fp8

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    aq, sa = fp8.quantize_rows(a, mode)
    bq, sb = fp8.quantize_rows(b, 0) if mode == 0 else fp8.quantize_block128(b)
    y = fp8.gemm_fp8(aq, sa, bq, sb, mode, bias)
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    ref = fp8.dequantize(aq, sa, mode) @ fp8.dequantize(bq, sb, mode, weight=True).t() + bias.float()
    assert _rel(y, ref) < 6e-3
    # and the quantised product is close to the bf16 one
    assert _rel(y, a.float() @ b.float().t() + bias.float()) < 6e-2


@pytest.mark.parametrize("M,N,K", [(64, 5120, 8192), (16, 1280, 8192)])
def test_fp8_skinny_gemm_split_k(M, N, K):
    from ghost_flow_b200.ops import _lib, fp8

    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    aq, sa = fp8.quantize_rows(a, 0)
    bq, sb = fp8.quantize_rows(b, 0)
    y = fp8.gemm_fp8(aq, sa, bq, sb, 0, bias)
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    ref = fp8.dequantize(aq, sa, 0) @ fp8.dequantize(bq, sb, 0, weight=True).t() + bias.float()
    assert _rel(y, ref) < 6e-3


def test_fp8_training_linear_matches_the_emulation_and_fp32(kernel_status):
    """Forward, input gradient and weight gradient of the e4m3 training linear on the tcgen05 fp8 kernel against the
    same quantisation emulated in fp32 on the CPU, and against the unquantised layer."""
    from ghost_flow_b200.ops import fp8

    torch.manual_seed(0)
    T, K, N = 512, 256, 384
    x = torch.randn(T, K)
    w = 0.1 * torch.randn(N, K)
    b = torch.randn(N)
    g = torch.randn(T, N)
    outs = {}
    for dev in ("cpu", "cuda"):
        xd = x.to(dev, torch.bfloat16).requires_grad_()
        wd = w.to(dev, torch.bfloat16).requires_grad_()
        bd = b.to(dev, torch.bfloat16).requires_grad_()
        y = fp8.fp8_linear(xd, wd, bd)
        y.backward(g.to(dev, torch.bfloat16))
        outs[dev] = [t.detach().float().cpu() for t in (y, xd.grad, wd.grad, bd.grad)]
    xr, wr, br = x.clone().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g)
    rel = lambda a, c: ((a - c).norm() / c.norm()).item()  # noqa: E731
    for got, emu, ref in zip(outs["cuda"], outs["cpu"], (yr.detach(), xr.grad, wr.grad, br.grad)):
        assert rel(got, emu) < 2e-2, rel(got, emu)          # same quantisation, different summation order
        assert rel(got, ref) < 7e-2, rel(got, ref)          # e4m3 against fp32
