"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _ops():
    from ghost_flow_b200 import ops

    return ops


def _assert_gemm_elementwise(out, ref, K, what=""):
    """A norm ratio hides a wrong tail row or column (one row of a 4096-row product moves it by 1e-4). Element by
    element: inputs are exact bf16 values accumulated in fp32, so an entry is off by its bf16 rounding (2^-9
    relative) plus noise far below sqrt(K) * 2^-7; an entry that was never written, or written from the wrong
    tile, is off by about sqrt(K)."""
    err = (out.float() - ref.float()).abs()
    bound = ref.float().abs() * 2.0 ** -7 + math.sqrt(K) * 2.0 ** -7
    bad = err > bound
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} entries off, worst {float((err - bound).max()):.3g} " \
                                f"at {tuple(torch.nonzero(bad)[0].tolist())}"


# ----------------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 256, 192), (200, 136, 72),
                                   (1024, 4096, 1024), (4096, 1024, 512)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn", "tt"])
def test_gemm_layouts(M, N, K, layout, kernel_status):
    ops = _ops()
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float()
    if layout == "nt":
        out = ops.matmul_nt(a, b.t().contiguous())
    elif layout == "nn":
        out = ops.matmul_nn(a, b)
    elif layout == "tn":
        out = ops.matmul_tn(a.t().contiguous(), b)
    else:
        out = ops.matmul_tt(a.t().contiguous(), b.t().contiguous())
    torch.cuda.synchronize()
    assert out.shape == (M, N)
    assert _rel_err(out, ref) < 1e-2, f"{layout} {M}x{N}x{K}"
    _assert_gemm_elementwise(out, ref, K, f"{layout} {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K,layout", [(768, 2304, 8192, "tn"), (768, 768, 4096, "tn"), (3072, 768, 8192, "tn"),
                                          (200, 760, 2056, "nt"), (64, 4096, 4096, "nt")])
def test_gemm_split_k_when_tiles_are_few(M, N, K, layout, kernel_status):
    """Weight-gradient shapes of narrow layers (few output tiles, K = tokens): K is split over the idle SMs and the
    slices meet in an fp32 workspace that the caller's allocator provides."""
    ops = _ops()
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float()
    out = ops.matmul_tn(a.t().contiguous(), b) if layout == "tn" else ops.matmul_nt(a, b.t().contiguous())
    torch.cuda.synchronize()
    assert _rel_err(out, ref) < 1e-2
    _assert_gemm_elementwise(out, ref, K, f"split-k {layout} {M}x{N}x{K}")


@pytest.mark.parametrize("T,D", [(8192, 768), (1000, 3072), (37, 8192), (5, 64)])
def test_linear_bias_gradient_column_sum(T, D, kernel_status):
    ops = _ops()
    x = torch.randn(T, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(D, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T, D, device=DEV, dtype=torch.bfloat16)
    ops.linear(x, w, b).backward(g)
    assert _rel_err(b.grad, g.float().sum(0)) < 1e-2


def test_split_qkv_backward_hands_on_the_packed_gradient(kernel_status):
    ops = _ops()
    B, S, H, Hk, D = 2, 256, 4, 2, 64
    qkv = torch.randn(B, S, H + 2 * Hk, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = ops.split_qkv(qkv, H, Hk)
    o = ops.flash_attention(q, k, v, causal=True)
    g = torch.randn_like(o)
    o.backward(g)
    ref = qkv.detach().clone().requires_grad_()
    o2 = ops.flash_attention(ref[:, :, :H], ref[:, :, H:H + Hk], ref[:, :, H + Hk:], causal=True)
    o2.backward(g)
    assert _rel_err(qkv.grad, ref.grad) < 1e-3
    # gradients that are not slices of one buffer are concatenated
    qkv2 = qkv.detach().clone().requires_grad_()
    q, k, v = ops.split_qkv(qkv2, H, Hk)
    (q.float().sum() + 2 * k.float().sum() + 3 * v.float().sum()).backward()
    assert float(qkv2.grad[:, :, :H].float().mean()) == 1.0 and float(qkv2.grad[:, :, H + Hk:].float().mean()) == 3.0


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_tile_widths_and_epilogue(bn, kernel_status):
    ops = _ops()
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    out = ops.gemm_raw(a, False, w, False, M, N, K, bias=bias, residual=res, bn_hint=bn)
    assert _rel_err(out, ref) < 1e-2
    # fp32 output with accumulation
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref2 = acc + 0.5 * (a.float() @ w.float().t())
    out2 = ops.gemm_raw(a, False, w, False, M, N, K, out=acc.clone(), accumulate=True, alpha=0.5, bn_hint=bn)
    assert _rel_err(out2, ref2) < 1e-2


def test_gemm_persistent_many_tiles(kernel_status):
    """More tiles than SMs: exercises the accumulator double-buffering and stage phase wrap."""
    ops = _ops()
    M, N, K = 4096, 4096, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = ops.matmul_nt(a, w)
    ref = a.float() @ w.float().t()
    assert _rel_err(out, ref) < 1e-2
    _assert_gemm_elementwise(out, ref, K)


@pytest.mark.parametrize("M,N,K", [(2048, 2048, 512), (1000, 4104, 328), (4096, 2304, 1024), (304, 9000, 200)])
@pytest.mark.parametrize("mode", ["pairs", "single"])
def test_gemm_cta_pairs_and_single_cta_agree_elementwise(M, N, K, mode, kernel_status, monkeypatch):
    """Large products run on CTA pairs (256 x 256 tiles); GF_GEMM_2SM=0 keeps the single-CTA kernel. Both must
    be right in every entry, tails included (rows and columns that do not fill the last tile), with bias, residual
    and accumulation into an fp32 output."""
    import subprocess, sys, os, json
    # the switch is read once per process, so each mode runs in its own interpreter
    code = f"""
import math, sys, torch
sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})
from ghost_flow_b200 import ops
from ghost_flow_b200.ops import _lib
torch.manual_seed(0)
M, N, K = {M}, {N}, {K}
a = torch.randn(M, K, device='cuda', dtype=torch.bfloat16)
w = torch.randn(N, K, device='cuda', dtype=torch.bfloat16)
bias = torch.randn(N, device='cuda', dtype=torch.bfloat16)
res = torch.randn(M, N, device='cuda', dtype=torch.bfloat16)
ref = a.float() @ w.float().t() + bias.float() + res.float()
out = ops.gemm_raw(a, False, w, False, M, N, K, bias=bias, residual=res)
err = (out.float() - ref).abs(); bound = ref.abs() * 2.0 ** -7 + math.sqrt(K) * 2.0 ** -7
acc = torch.randn(M, N, device='cuda', dtype=torch.float32)
ref2 = acc + 0.5 * (a.float() @ w.float().t())
out2 = ops.gemm_raw(a, False, w, False, M, N, K, out=acc.clone(), accumulate=True, alpha=0.5)
err2 = (out2 - ref2).abs(); bound2 = math.sqrt(K) * 2.0 ** -10 + ref2.abs() * 2.0 ** -12
at = a.t().contiguous(); wt = w.t().contiguous()
out3 = ops.matmul_tt(at, w)          # A stored [K, M], B stored [N, K]
ref3 = a.float() @ w.float().t()
err3 = (out3.float() - ref3).abs(); bound3 = ref3.abs() * 2.0 ** -7 + math.sqrt(K) * 2.0 ** -7
torch.cuda.synchronize(); _lib.check_status()
print(int((err > bound).sum()), int((err2 > bound2).sum()), int((err3 > bound3).sum()))
"""
    env = dict(os.environ, GF_GEMM_2SM="1" if mode == "pairs" else "0")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split()[-3:] == ["0", "0", "0"], r.stdout


def test_linear_autograd(kernel_status):
    ops = _ops()
    x = torch.randn(4, 64, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(384, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


# ----------------------------------------------------------------------------------------- norms
@pytest.mark.parametrize("T,D", [(64, 256), (300, 4096), (17, 1024)])
def test_rmsnorm_fwd_bwd(T, D, kernel_status):
    ops = _ops()
    x = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = ops.rms_norm(x, w, 1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_rmsnorm_fused_residual(kernel_status):
    ops = _ops()
    T, D = 96, 512
    x = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y, h = ops.rms_norm(x, w, 1e-6, residual=r)
    (y.float().sum() + 2 * h.float().sum()).backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    hr = xr + rr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    (yr.sum() + 2 * hr.sum()).backward()
    assert _rel_err(h, hr) < 1e-2 and _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(r.grad, rr.grad) < 1e-2


@pytest.mark.parametrize("T,D", [(64, 768), (33, 128), (8192, 768), (1000, 1024), (77, 200), (130, 1032), (50, 4096)])
def test_layernorm_fwd_bwd(T, D, kernel_status):
    """Rows up to 1024 long go through the warp-per-row kernels (one to four vectors per lane, rows shared by the
    eight warps of a CTA); longer ones through the CTA-per-row kernels."""
    ops = _ops()
    x = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    b = (0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = ops.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (D,), wr, br, 1e-5)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


# ----------------------------------------------------------------------------------------- rope / activations
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_fwd_bwd(interleaved, kernel_status):
    ops = _ops()
    B, S, H, D = 2, 128, 4, 128
    cos, sin = ops.rope_tables(S, D, 1e4, DEV)
    qkv = torch.randn(B, S, 3 * H, D, device=DEV, dtype=torch.bfloat16)
    x = qkv[:, :, :H].detach().clone().requires_grad_()          # contiguous copy
    y = ops.rope(x, cos, sin, interleaved=interleaved)
    ref = ops.rope_ref(x.detach().float(), cos, sin, interleaved)
    assert _rel_err(y, ref) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    ops.rope_ref(xr, cos, sin, interleaved).backward(g.float())
    assert _rel_err(x.grad, xr.grad) < 1e-2
    # strided in-place on a packed view
    packed = qkv.clone()
    ops.rope(packed[:, :, :H], cos, sin, interleaved=interleaved, inplace=True)
    assert _rel_err(packed[:, :, :H], ops.rope_ref(qkv[:, :, :H].float(), cos, sin, interleaved)) < 1e-2
    assert torch.equal(packed[:, :, H:], qkv[:, :, H:])


def test_swiglu_and_unary(kernel_status):
    ops = _ops()
    gu = torch.randn(64, 2 * 352, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(gu.grad, gr.grad) < 1e-2
    for name in ["relu", "gelu", "sigmoid", "tanh", "silu"]:
        x = torch.randn(1000, 8, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        y = ops.unary(x, name)
        gg = torch.randn_like(y)
        y.backward(gg)
        xr = x.detach().float().requires_grad_()
        from ghost_flow_b200.ops.fused import _unary_ref

        yr = _unary_ref(xr, name)
        yr.backward(gg.float())
        assert _rel_err(y, yr) < 1e-2, name
        assert _rel_err(x.grad, xr.grad) < 1.5e-2, name
    z = ops.op_chain(torch.randn(999, device=DEV), ["gelu", "tanh", "relu"])
    assert z.shape == (999,)


# ----------------------------------------------------------------------------------------- loss / optimizer
@pytest.mark.parametrize("T,V", [(64, 1000), (37, 32000), (8, 50264), (24, 50257), (16, 1003)])
def test_xent_fused(T, V, kernel_status):
    ops = _ops()
    logits = (2 * torch.randn(T, V, device=DEV)).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=DEV)
    loss = ops.cross_entropy(logits, tgt)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, tgt)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert _rel_err(logits.grad, lr.grad) < 2e-2


def test_linear_head_with_odd_vocabulary_stays_on_the_kernels(kernel_status):
    """GPT-2's 50257-entry vocabulary: rows of a [T, 50257] bf16 matrix do not start on 16-byte boundaries, so the
    head's output, the loss gradient and both backward products use a padded row pitch instead of falling back."""
    ops = _ops()
    T, d, V = 192, 256, 50257
    x = (0.5 * torch.randn(T, d, device=DEV)).to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(V, d, device=DEV)).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=DEV)
    logits = ops.linear(x, w)
    assert logits.shape == (T, V) and logits.stride(0) % 64 == 0
    loss = ops.cross_entropy(logits, tgt)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(xr @ wr.t(), tgt)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert _rel_err(x.grad, xr.grad) < 2e-2 and _rel_err(w.grad, wr.grad) < 2e-2


def test_adamw_flat_matches_reference_formula(kernel_status):
    from ghost_flow_b200.ops import optim_kernels as ok

    n = 100003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(torch.bfloat16)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    lp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd = 3e-4, 0.9, 0.999, 1e-8, 0.01
    for step in (1, 2, 3):
        ok.adam_flat(p, m, v, g, lp, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=step, decoupled=True)
        gf = g.float()
        mr = b1 * mr + (1 - b1) * gf
        vr = b2 * vr + (1 - b2) * gf * gf
        mh, vh = mr / (1 - b1 ** step), vr / (1 - b2 ** step)
        pr = pr * (1 - lr * wd) - lr * mh / (vh.sqrt() + eps)
    assert torch.allclose(p, pr, rtol=1e-5, atol=1e-6)
    assert torch.allclose(lp.float(), pr, rtol=1e-2, atol=1e-2)


# ----------------------------------------------------------------------------------------- attention
@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 128, True), (1, 256, 2, 2, 128, True), (2, 512, 4, 2, 128, True), (1, 384, 2, 2, 64, True),
    (1, 256, 2, 1, 128, False), (1, 200, 2, 2, 128, True), (1, 1024, 2, 2, 128, True)])
def test_flash_attention_fwd(B, S, Hq, Hkv, D, causal, kernel_status):
    ops = _ops()
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    o = ops.flash_attention(q, k, v, causal=causal)
    ref = ops.attention_ref(q, k, v, causal=causal)
    torch.cuda.synchronize()
    assert _rel_err(o, ref) < 2e-2
    # element-wise: outputs are convex combinations of V rows (|v| < ~5), bf16 rounding of P and O
    assert (o.float() - ref.float()).abs().max().item() < 6e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 128, True), (1, 256, 2, 2, 128, True), (2, 512, 4, 2, 128, True), (1, 256, 2, 2, 64, True),
    (1, 256, 2, 1, 128, False), (1, 1024, 4, 1, 128, True), (1, 384, 2, 2, 64, False)])
def test_flash_attention_bwd(B, S, Hq, Hkv, D, causal, kernel_status):
    ops = _ops()
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    o = ops.flash_attention(q, k, v, causal=causal)
    g = torch.randn_like(o)
    o.backward(g)
    ref_in = qkv.detach().float().requires_grad_()
    qr, kr, vr = ref_in[:, :, :Hq], ref_in[:, :, Hq:Hq + Hkv], ref_in[:, :, Hq + Hkv:]
    ops.attention_ref(qr, kr, vr, causal=causal).backward(g.float())
    torch.cuda.synchronize()
    gq, gk, gv = qkv.grad[:, :, :Hq], qkv.grad[:, :, Hq:Hq + Hkv], qkv.grad[:, :, Hq + Hkv:]
    rq, rk, rv = ref_in.grad[:, :, :Hq], ref_in.grad[:, :, Hq:Hq + Hkv], ref_in.grad[:, :, Hq + Hkv:]
    assert _rel_err(gv, rv) < 3e-2, "dV"
    assert _rel_err(gk, rk) < 3e-2, "dK"
    assert _rel_err(gq, rq) < 3e-2, "dQ"


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 512, 4, 2, 128, True), (1, 256, 2, 2, 64, False)])
def test_flash_attention_bwd_first_generation_kernel(B, S, Hq, Hkv, D, causal, kernel_status, monkeypatch):
    """The backward kernel whose compute warps also drain dQ stays available (GF_FA_BWD=1)."""
    monkeypatch.setenv("GF_FA_BWD", "1")
    ops = _ops()
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    o = ops.flash_attention(q, k, v, causal=causal)
    g = torch.randn_like(o)
    o.backward(g)
    ref_in = qkv.detach().float().requires_grad_()
    qr, kr, vr = ref_in[:, :, :Hq], ref_in[:, :, Hq:Hq + Hkv], ref_in[:, :, Hq + Hkv:]
    ops.attention_ref(qr, kr, vr, causal=causal).backward(g.float())
    torch.cuda.synchronize()
    assert _rel_err(qkv.grad, ref_in.grad) < 3e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 256, 2, 2, 128, True), (1, 384, 2, 1, 64, False)])
def test_flash_attention_fwd_first_generation_kernel(B, S, Hq, Hkv, D, causal, kernel_status, monkeypatch):
    """The single-tile forward kernel stays available (GF_FA_FWD=1) and must agree with the reference too."""
    monkeypatch.setenv("GF_FA_FWD", "1")
    ops = _ops()
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    o = ops.flash_attention(q, k, v, causal=causal)
    assert _rel_err(o, ops.attention_ref(q, k, v, causal=causal)) < 2e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 512, 2, 2, 128, True), (1, 384, 2, 1, 64, False)])
def test_flash_attention_fwd_second_generation_kernel(B, S, Hq, Hkv, D, causal, kernel_status, monkeypatch):
    """The two-tile kernel that passes P through shared memory stays available (GF_FA_FWD=2)."""
    monkeypatch.setenv("GF_FA_FWD", "2")
    ops = _ops()
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    o = ops.flash_attention(q, k, v, causal=causal)
    assert _rel_err(o, ops.attention_ref(q, k, v, causal=causal)) < 2e-2


def test_flash_attention_fwd_large_scores_rescale(kernel_status):
    """Scores that keep growing along the sequence force the in-TMEM output rescale path many times."""
    ops = _ops()
    B, S, H, D = 1, 1024, 2, 128
    q = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    ramp = torch.linspace(0.2, 6.0, S, device=DEV).view(1, S, 1, 1)
    k = (k * ramp).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16)
    o = ops.flash_attention(q, k, v, causal=True)
    assert _rel_err(o, ops.attention_ref(q, k, v, causal=True)) < 2e-2
    o2 = ops.flash_attention(q, k, v, causal=False)
    assert _rel_err(o2, ops.attention_ref(q, k, v, causal=False)) < 2e-2


@pytest.mark.parametrize("M,N,K", [(64, 5120, 8192), (8, 1280, 8192), (200, 768, 4096)])
def test_skinny_gemm_split_k_matches_fp32(M, N, K):
    """Decode-sized products take the split-K path (fp32 atomics + conversion kernel, bias and residual there)."""
    from ghost_flow_b200.ops import _lib
    from ghost_flow_b200.ops.gemm import gemm_raw

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y = gemm_raw(a, False, w, False, M, N, K, bias=bias, residual=res)
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    assert ((y.float() - ref).norm() / ref.norm()) < 5e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tensor_api_elementwise_reductions_softmax(dtype, kernel_status):
    """Tensor add / sub / mul, activations, full sum / max and row softmax run the library kernels."""
    import torch.nn.functional as F

    import ghost_flow_b200 as gf
    from ghost_flow_b200.ops import _lib

    torch.manual_seed(0)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for n in (10_000_000, 1003):
        a, b = torch.randn(n, device=DEV, dtype=dtype), torch.randn(n, device=DEV, dtype=dtype)
        ta, tb = gf.Tensor(a), gf.Tensor(b)
        before = _lib.launch_count()
        got = {"add": ta + tb, "sub": ta - tb, "mul": ta * tb, "relu": ta.relu(), "sigmoid": ta.sigmoid(),
               "tanh": ta.tanh(), "gelu": ta.gelu(), "silu": ta.silu()}
        assert _lib.launch_count() - before >= len(got)
        a32, b32 = a.float(), b.float()
        want = {"add": a32 + b32, "sub": a32 - b32, "mul": a32 * b32, "relu": torch.relu(a32),
                "sigmoid": torch.sigmoid(a32), "tanh": torch.tanh(a32), "gelu": F.gelu(a32, approximate="tanh"),
                "silu": F.silu(a32)}
        for k in got:
            assert got[k].data.dtype == dtype
            assert torch.allclose(got[k].data.float(), want[k], **tol), k
        s, m = ta.sum().data.float(), ta.max().data.float()
        assert torch.allclose(s, a32.sum(), atol=0.5 if dtype == torch.float32 else 40.0, rtol=1e-2)
        assert torch.allclose(m, a32.max(), **tol)
    for rows, cols in ((64, 1000), (3, 50257), (257, 33), (300, 4096), (17, 8000)):
        x = torch.randn(rows, cols, device=DEV, dtype=dtype) * 3
        t = gf.Tensor(x)
        assert torch.allclose(t.softmax(-1).data.float(), torch.softmax(x.float(), -1),
                              atol=1e-5 if dtype == torch.float32 else 4e-3)
        assert torch.allclose(t.log_softmax(1).data.float(), torch.log_softmax(x.float(), -1),
                              atol=1e-4 if dtype == torch.float32 else 8e-2)


def test_fp32_matmul_on_tensor_cores_is_close_to_fp32(kernel_status):
    """Tensor.matmul of fp32 CUDA matrices: one bf16 tcgen05 GEMM over hi/lo splits, error far below bf16's."""
    import ghost_flow_b200 as gf
    from ghost_flow_b200.ops import _lib

    torch.manual_seed(0)
    for M, K, N in ((1024, 1024, 1024), (300, 72, 136), (2048, 512, 128), (200, 64, 136)):
        a, b = torch.randn(M, K, device=DEV), torch.randn(K, N, device=DEV)
        before = _lib.launch_count()
        y = gf.Tensor(a).matmul(gf.Tensor(b)).data
        assert _lib.launch_count() - before >= 3 and y.dtype == torch.float32
        ref = a.double() @ b.double()
        scale = (a.abs().double() @ b.abs().double()).max()
        err = (y.double() - ref).abs().max() / scale
        bf16_err = ((a.bfloat16().float() @ b.bfloat16().float()).double() - ref).abs().max() / scale
        assert err < 3e-5 and err < bf16_err / 20, (M, K, N, float(err), float(bf16_err))
        yt = gf.Tensor(a).matmul(gf.Tensor(b.t().contiguous()).t()).data  # strided right operand
        assert torch.allclose(yt, y, atol=1e-4 * float(scale))


# ----------------------------------------------------------------------------------------- flat optimizers
@pytest.mark.parametrize("opt_name", ["AdamW", "SGD"])
def test_flat_optimizer_matches_cpu_path_with_missing_grads_and_external_writes(opt_name, kernel_status):
    """The CUDA path (flat fp32 buffers, one fused kernel per run of parameters) against the per-tensor CPU path:
    a parameter without a gradient is left alone (no weight decay, no moment decay), and parameters written from
    outside between steps (load_state_dict-style copy_) keep the new value instead of being reset from a stale
    master copy, for fp32 parameters (views of the flat buffer) and bf16 ones (version check)."""
    from ghost_flow_b200 import optim

    def make(device, dtype):
        g = torch.Generator().manual_seed(0)
        return [torch.nn.Parameter(torch.randn(33, 7, generator=g).to(device=device, dtype=dtype)),
                torch.nn.Parameter(torch.randn(50, generator=g).to(device=device, dtype=dtype)),
                torch.nn.Parameter(torch.randn(16, 16, generator=g).to(device=device, dtype=dtype))]

    def make_opt(ps):
        if opt_name == "AdamW":
            return optim.AdamW(ps, lr=1e-2, weight_decay=0.1)
        return optim.SGD(ps, lr=1e-2, momentum=0.9, weight_decay=0.1)

    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        pc, pg = make("cpu", torch.float32), make(DEV, dtype)
        oc, og = make_opt(pc), make_opt(pg)
        gen = torch.Generator().manual_seed(1)
        for step in range(4):
            for i, (a, b) in enumerate(zip(pc, pg)):
                if i == 1 and step != 2:
                    a.grad, b.grad = None, None          # no gradient in most steps
                    continue
                gr = torch.randn(a.shape, generator=gen)
                a.grad, b.grad = gr.clone(), gr.to(device=DEV, dtype=dtype)
            oc.step()
            og.step()
            if step == 1:                                # an external write after the first steps
                new = torch.full_like(pc[2], 0.25)
                with torch.no_grad():
                    pc[2].copy_(new)
                    pg[2].copy_(new.to(device=DEV, dtype=dtype))
        torch.cuda.synchronize()
        for a, b in zip(pc, pg):
            assert torch.allclose(a, b.float().cpu(), rtol=tol, atol=tol), (opt_name, dtype)
        # the untouched steps of the grad-less parameter left it exactly where it was after its one update
