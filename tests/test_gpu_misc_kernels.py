"""CUDA kernels off the transformer path against their PyTorch fp32 formulas."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_posenc_and_volume_render(kernel_status):
    from ghost_flow_b200.ops import render

    x = torch.randn(1000, 3, device=DEV)
    assert torch.allclose(render.positional_encoding(x, 6), render.positional_encoding_ref(x, 6), atol=1e-4)
    R, S = 513, 96
    rgb, sigma = torch.rand(R, S, 3, device=DEV), torch.rand(R, S, device=DEV) * 3
    z = torch.sort(torch.rand(R, S, device=DEV) * 4 + 2, -1).values
    nrm = torch.rand(R, device=DEV) + 0.5
    for wb in (False, True):
        got = render.volume_render(rgb, sigma, z, nrm, wb)
        ref = render.volume_render_ref(rgb, sigma, z, nrm, wb)
        for a, b in zip(got, ref):
            assert torch.allclose(a, b, atol=2e-4, rtol=1e-3)


def test_fps_knn_normals(kernel_status):
    from ghost_flow_b200.ops import render

    pts = torch.randn(3, 500, 3, device=DEV)
    idx = render.farthest_point_sample(pts, 32, start=7)
    assert torch.equal(idx.cpu(), render.farthest_point_sample_ref(pts.cpu(), 32, 7))
    q = torch.randn(3, 40, 3, device=DEV)
    got = render.knn(pts, q, 8)
    ref = render.knn_ref(pts, q, 8)
    d = torch.cdist(q, pts)
    assert torch.allclose(d.gather(-1, got), d.gather(-1, ref), atol=1e-5)
    verts = torch.randn(100, 3, device=DEV)
    faces = torch.randint(0, 100, (200, 3), device=DEV)
    n, a = render.face_normals(verts, faces)
    nr, ar = render.face_normals(verts.cpu(), faces.cpu())
    assert torch.allclose(a.cpu(), ar, atol=1e-5) and torch.allclose(n.cpu(), nr, atol=1e-4)


def test_int8_quant_kernels(kernel_status):
    from ghost_flow_b200.ops import render

    x = torch.randn(16, 8, 5, device=DEV)
    scale = (x.abs().amax((0, 2)) / 127).clamp(min=1e-8)
    zp = torch.zeros(8, device=DEV)
    q = render.quantize_int8(x, scale, zp, channel_dim=1, qmin=-127)
    qr = render.quantize_int8(x.cpu(), scale.cpu(), zp.cpu(), channel_dim=1, qmin=-127)
    assert (q.cpu().int() - qr.int()).abs().max() <= 1
    assert (render.dequantize_int8(q, scale, zp, 1) - x).abs().max() < scale.max() * 0.51
    s1, z1 = torch.tensor([0.05], device=DEV), torch.tensor([3.0], device=DEV)
    fq = render.fake_quantize(x, s1, z1)
    assert torch.allclose(fq.cpu(), render.fake_quantize(x.cpu(), s1.cpu(), z1.cpu()), atol=0.051)


def test_conv_bn_relu_and_batchnorm(kernel_status):
    from ghost_flow_b200.ops import render

    x = torch.randn(2, 5, 37, 41, device=DEV)          # output wider than 32 columns
    w, b = torch.randn(7, 5, 3, 3, device=DEV) * 0.2, torch.randn(7, device=DEV)
    g, be = torch.rand(7, device=DEV) + 0.5, torch.randn(7, device=DEV)
    mu, var = torch.randn(7, device=DEV), torch.rand(7, device=DEV) + 0.5
    for stride, pad in ((1, 1), (2, 0)):
        got = render.conv_bn_relu(x, w, b, g, be, mu, var, stride, pad)
        ref = torch.relu(F.batch_norm(F.conv2d(x, w, b, stride, pad), mu, var, g, be, False, 0.0, 1e-5))
        assert torch.allclose(got, ref, atol=2e-3, rtol=1e-3)
    rm, rv = torch.zeros(5, device=DEV), torch.ones(5, device=DEV)
    rm2, rv2 = rm.clone(), rv.clone()
    wt, bs = torch.rand(5, device=DEV) + 0.5, torch.randn(5, device=DEV)
    y = render.batch_norm_train(x, wt, bs, rm, rv, 0.1, 1e-5)
    yr = F.batch_norm(x, rm2, rv2, wt, bs, True, 0.1, 1e-5)
    assert torch.allclose(y, yr, atol=1e-3) and torch.allclose(rm, rm2, atol=1e-4) and torch.allclose(rv, rv2, atol=1e-3)


def test_conv_bn_relu_on_tensor_cores_matches_fp32():
    import torch.nn.functional as F
    from ghost_flow_b200.ops import _lib
    from ghost_flow_b200.ops.render import conv_bn_relu_tensorcore

    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(4, 16, 20, 18, device=dev)
    w = torch.randn(32, 16, 3, 3, device=dev) * 0.1
    b = torch.randn(32, device=dev)
    g, be = torch.rand(32, device=dev) + 0.5, torch.randn(32, device=dev)
    mean, var = torch.randn(32, device=dev), torch.rand(32, device=dev) + 0.5
    y = conv_bn_relu_tensorcore(x, w, b, g, be, mean, var, stride=2, padding=1)
    torch.cuda.synchronize()
    _lib.check_status(torch.device(dev))
    ref = torch.relu(F.batch_norm(F.conv2d(x, w, b, 2, 1), mean, var, g, be, False, 0.0, 1e-5))
    assert y.shape == ref.shape
    assert ((y - ref).norm() / ref.norm()) < 2e-2


def test_channels_last_conv_matches_fp32(kernel_status):
    """Gather kernel + tcgen05 GEMM with bias, shortcut and ReLU in the epilogue against conv2d in fp32."""
    from ghost_flow_b200.ops.render import conv2d_nhwc, im2col_nhwc, pack_conv_weight_nhwc

    torch.manual_seed(0)
    for (N, C, H, W, Co, k, s, p) in ((3, 16, 19, 23, 64, 3, 1, 1), (2, 8, 33, 33, 24, 7, 2, 3), (4, 64, 14, 14, 128, 1, 1, 0),
                                      (2, 32, 15, 15, 64, 1, 2, 0), (2, 3, 32, 32, 16, 3, 1, 1), (2, 24, 10, 11, 16, 3, 2, 1)):
        x = torch.randn(N, C, H, W, device=DEV)
        w = torch.randn(Co, C, k, k, device=DEV) / (C * k * k) ** 0.5
        b = torch.randn(Co, device=DEV)
        wp, bp = pack_conv_weight_nhwc(w, b)
        Cp = wp.shape[1] // (k * k)
        xn = torch.zeros(N, H, W, Cp, device=DEV, dtype=torch.bfloat16)
        xn[..., :C] = x.permute(0, 2, 3, 1)
        xr = xn[..., :C].float().permute(0, 3, 1, 2)
        ref = F.conv2d(xr, w.bfloat16().float(), b.bfloat16().float(), s, p)
        cols, OH, OW = im2col_nhwc(xn, k, k, s, p)
        cols_cpu, _, _ = im2col_nhwc(xn.cpu(), k, k, s, p)
        assert torch.equal(cols.cpu(), cols_cpu)
        res = torch.randn(N, OH, OW, Co, device=DEV).bfloat16()
        y = conv2d_nhwc(xn, wp, bp, (k, k), s, p, relu=True, residual=res)
        want = torch.relu(ref + res.float().permute(0, 3, 1, 2))
        got = y.float().permute(0, 3, 1, 2)
        assert got.shape == want.shape
        assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (got - want).abs().max()


def test_resnet_serving_program_matches_the_model():
    from ghost_flow_b200.models import resnet18, resnet50
    from ghost_flow_b200.nn import fuse_conv_bn_relu

    torch.manual_seed(0)
    for make in (lambda: resnet18(16, small_input=True), lambda: resnet50(16, width=16)):
        m = make().to(DEV)
        for mod in m.modules():
            if hasattr(mod, "running_mean"):
                mod.running_mean.normal_(0, 0.1)
                mod.running_var.uniform_(0.5, 1.5)
        m.eval()
        x = torch.randn(4, 3, 64, 64, device=DEV)
        with torch.no_grad():
            ref = m(x)
            got = m.compile_inference()(x)
            assert (got - ref).abs().max() <= 0.05 * ref.abs().max() + 0.05
            assert fuse_conv_bn_relu(m) > 0
            fused = m(x)
            assert (fused - ref).abs().max() <= 0.05 * ref.abs().max() + 0.05


def test_cuda_graph_replay_matches_eager():
    """A BERT encoder and the ResNet serving program replayed from CUDA graphs give the eager results, also after
    the inputs change and for a second input shape."""
    from ghost_flow_b200 import models, nn

    torch.manual_seed(0)
    cfg = models.BertConfig.bert_tiny()
    bert = models.BertModel(cfg).to(DEV).to(torch.bfloat16).eval()
    runner = nn.CudaGraphRunner(lambda t: bert(t).last_hidden_state)
    with torch.no_grad():
        for shape in ((4, 64), (2, 128), (4, 64)):
            ids = torch.randint(0, cfg.vocab_size, shape, device=DEV)
            want = bert(ids).last_hidden_state.float()
            got = runner(ids).float()
            assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (got - want).abs().max()
    assert len(runner._cache) == 2
    m = models.resnet18(128, small_input=True).to(DEV).eval()
    eager, graphed = m.compile_inference(), m.compile_inference(cuda_graph=True)
    for n in (64, 64, 16):
        x = torch.randn(n, 3, 32, 32, device=DEV)
        assert torch.allclose(graphed(x), eager(x), atol=1e-2, rtol=1e-2)


def test_implicit_convolution_matches_fp32():
    """Stride-1 'same' convolutions read straight from the padded channels-last image (row-shifted TMA tiles)
    against conv2d in fp32, with and without the shortcut."""
    from ghost_flow_b200.ops import _lib
    from ghost_flow_b200.ops.render import conv2d_nhwc, conv2d_nhwc_implicit, pack_conv_weight_nhwc

    torch.manual_seed(0)
    for (N, C, H, W, Co, k) in ((3, 64, 19, 23, 64, 3), (32, 128, 28, 28, 128, 3), (2, 64, 9, 9, 256, 5),
                                (1, 192, 7, 7, 72, 3), (5, 512, 7, 7, 512, 3)):
        x = torch.randn(N, H, W, C, device=DEV).bfloat16()
        w = torch.randn(Co, C, k, k, device=DEV) / (C * k * k) ** 0.5
        b = torch.randn(Co, device=DEV)
        wp, bp = pack_conv_weight_nhwc(w, b)
        res = torch.randn(N, H, W, Co, device=DEV).bfloat16()
        ref = F.conv2d(x.float().permute(0, 3, 1, 2), w.bfloat16().float(), b.bfloat16().float(), 1, (k - 1) // 2)
        got = conv2d_nhwc_implicit(x, wp, bp, (k, k), relu=False).float().permute(0, 3, 1, 2)
        _lib.check_status()
        assert torch.allclose(got, ref, atol=3e-2, rtol=3e-2), (N, C, H, W, Co, k, float((got - ref).abs().max()))
        got = conv2d_nhwc_implicit(x, wp, bp, (k, k), relu=True, residual=res).float().permute(0, 3, 1, 2)
        want = torch.relu(ref + res.float().permute(0, 3, 1, 2))
        assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
        from ghost_flow_b200.ops import render

        saved, render.IMPLICIT_CONV = render.IMPLICIT_CONV, False   # the gather + GEMM path of the same call
        try:
            unfolded = conv2d_nhwc(x, wp, bp, (k, k), 1, (k - 1) // 2, relu=True, residual=res)
        finally:
            render.IMPLICIT_CONV = saved
        assert torch.allclose(got, unfolded.float().permute(0, 3, 1, 2), atol=3e-2, rtol=3e-2)
