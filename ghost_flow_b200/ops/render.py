"""NeRF rendering arithmetic, point-cloud sampling, mesh normals, INT8 quantisation and the fused inference
Conv+BN+ReLU: CUDA kernels (``csrc/misc_kernels.cu``) for fp32 GPU tensors outside autograd, PyTorch formulas
otherwise (those formulas are also the test oracles, restating the reference's CPU loops:
ghostflow-nn/src/nerf.rs:111-147,353-408; point_cloud.rs:326-470; mesh.rs:55-113; quantization.rs:77-240;
ops/conv.rs + norm.rs)."""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _lib

_BOUND = False


def _lib_misc():
    global _BOUND
    lib = _lib.cuda_lib()
    if not _BOUND:
        P, I, L, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.gf_posenc.argtypes = [P, P, L, I, I, I, P]
        lib.gf_volume_render.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
        lib.gf_fps.argtypes = [P, P, P, I, I, I, I, P]
        lib.gf_knn.argtypes = [P, P, P, I, I, I, I, P]
        lib.gf_face_normals.argtypes = [P, P, P, P, I, P]
        lib.gf_quantize_i8.argtypes = [P, P, P, P, L, L, I, I, I, P]
        lib.gf_dequantize_i8.argtypes = [P, P, P, P, L, L, I, P]
        lib.gf_fake_quant.argtypes = [P, P, P, P, L, L, I, I, I, P]
        lib.gf_conv_bn_relu.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, Fl, I, P]
        lib.gf_batchnorm_train.argtypes = [P, P, P, P, P, P, P, P, I, I, I, Fl, Fl, P]
        _BOUND = True
    return lib


def _gpu_plain(*ts) -> bool:
    """fp32 CUDA tensors with no autograd graph to maintain."""
    for t in ts:
        if t is None:
            continue
        if not (t.is_cuda and t.dtype == torch.float32) or (torch.is_grad_enabled() and t.requires_grad):
            return False
    return True


def _p(t):
    return t.data_ptr() if t is not None else None


# ------------------------------------------------------------------ NeRF
def positional_encoding_ref(x, num_freqs: int, include_input: bool = True):
    outs = [x] if include_input else []
    for k in range(num_freqs):
        outs += [torch.sin(x * 2.0 ** k), torch.cos(x * 2.0 ** k)]
    # per input dimension: [x, sin(2^0 x), cos(2^0 x), sin(2^1 x), ...]
    return torch.stack(outs, dim=-1).flatten(-2)


def positional_encoding(x, num_freqs: int, include_input: bool = True):
    if _gpu_plain(x):
        xc = x.contiguous()
        d = xc.shape[-1]
        per = 2 * num_freqs + (1 if include_input else 0)
        out = torch.empty(*xc.shape[:-1], d * per, device=x.device, dtype=torch.float32)
        _lib.check_rc(_lib_misc().gf_posenc(xc.data_ptr(), out.data_ptr(), xc.numel() // d, d, num_freqs,
                                            1 if include_input else 0, _lib.stream_ptr()), "gf_posenc")
        return out
    return positional_encoding_ref(x, num_freqs, include_input)


def volume_render_ref(rgb, sigma, z, ray_norm=None, white_background=False):
    delta = torch.cat((z[:, 1:] - z[:, :-1], torch.full_like(z[:, :1], 1e10)), -1)
    if ray_norm is not None:
        delta = delta * ray_norm[:, None]
    alpha = 1.0 - torch.exp(-sigma * delta)
    T = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha + 1e-10), -1), -1)[:, :-1]
    w = T * alpha
    color = (w[..., None] * rgb).sum(1)
    acc = w.sum(1)
    if white_background:
        color = color + (1.0 - acc)[:, None]
    return color, (w * z).sum(1), acc, w


def volume_render(rgb, sigma, z, ray_norm=None, white_background=False):
    """(color [R,3], depth [R], acc [R], weights [R,S])."""
    if _gpu_plain(rgb, sigma, z, ray_norm):
        R, S = sigma.shape
        rgb, sigma, z = rgb.contiguous(), sigma.contiguous(), z.contiguous()
        color = torch.empty(R, 3, device=rgb.device)
        depth = torch.empty(R, device=rgb.device)
        acc = torch.empty(R, device=rgb.device)
        w = torch.empty(R, S, device=rgb.device)
        rn = ray_norm.contiguous() if ray_norm is not None else None
        _lib.check_rc(_lib_misc().gf_volume_render(rgb.data_ptr(), sigma.data_ptr(), z.data_ptr(), _p(rn),
                                                   color.data_ptr(), depth.data_ptr(), acc.data_ptr(), w.data_ptr(),
                                                   R, S, 1 if white_background else 0, _lib.stream_ptr()),
                      "gf_volume_render")
        return color, depth, acc, w
    return volume_render_ref(rgb, sigma, z, ray_norm, white_background)


# ------------------------------------------------------------------ point clouds / meshes
def farthest_point_sample_ref(pts, m: int, start: int = 0):
    B, N, _ = pts.shape
    idx = torch.zeros(B, m, dtype=torch.long, device=pts.device)
    dist = torch.full((B, N), 1e30, device=pts.device)
    cur = torch.full((B,), start % N, dtype=torch.long, device=pts.device)
    ar = torch.arange(B, device=pts.device)
    for i in range(m):
        idx[:, i] = cur
        d = (pts - pts[ar, cur][:, None, :]).pow(2).sum(-1)
        dist = torch.minimum(dist, d)
        cur = dist.argmax(-1)
    return idx


def farthest_point_sample(pts, m: int, start: int = 0):
    """Indices ``[B, m]`` of an iterative farthest-point subset of ``pts [B, N, 3]``."""
    if _gpu_plain(pts):
        B, N, _ = pts.shape
        p = pts.contiguous()
        idx = torch.empty(B, m, dtype=torch.int32, device=pts.device)
        scratch = torch.empty(B, N, device=pts.device)
        _lib.check_rc(_lib_misc().gf_fps(p.data_ptr(), idx.data_ptr(), scratch.data_ptr(), B, N, m, start,
                                         _lib.stream_ptr()), "gf_fps")
        return idx.long()
    return farthest_point_sample_ref(pts, m, start)


def knn_ref(pts, queries, k: int):
    d = torch.cdist(queries, pts)
    return d.topk(k, dim=-1, largest=False).indices


def knn(pts, queries, k: int):
    """Indices ``[B, Q, k]`` of the k nearest ``pts [B, N, 3]`` of every query ``[B, Q, 3]`` (nearest first)."""
    if _gpu_plain(pts, queries) and k <= 64:
        B, N, _ = pts.shape
        Q = queries.shape[1]
        out = torch.empty(B, Q, k, dtype=torch.int32, device=pts.device)
        _lib.check_rc(_lib_misc().gf_knn(pts.contiguous().data_ptr(), queries.contiguous().data_ptr(), out.data_ptr(),
                                         B, N, Q, k, _lib.stream_ptr()), "gf_knn")
        return out.long()
    return knn_ref(pts, queries, k)


def face_normals(verts, faces):
    """(unit normals ``[F,3]``, areas ``[F]``) of triangles ``faces [F,3]`` over ``verts [V,3]``."""
    if _gpu_plain(verts) and faces.is_cuda:
        Fn = faces.shape[0]
        n = torch.empty(Fn, 3, device=verts.device)
        a = torch.empty(Fn, device=verts.device)
        _lib.check_rc(_lib_misc().gf_face_normals(verts.contiguous().data_ptr(), faces.int().contiguous().data_ptr(),
                                                  n.data_ptr(), a.data_ptr(), Fn, _lib.stream_ptr()),
                      "gf_face_normals")
        return n, a
    v0, v1, v2 = verts[faces[:, 0]], verts[faces[:, 1]], verts[faces[:, 2]]
    c = torch.cross(v1 - v0, v2 - v0, dim=-1)
    ln = c.norm(dim=-1)
    return c / ln.clamp(min=1e-20)[:, None], 0.5 * ln


# ------------------------------------------------------------------ INT8
def _chan_layout(x, channel_dim, channels):
    if channels == 1:
        return 1
    inner = 1
    for d in x.shape[channel_dim + 1:]:
        inner *= d
    return inner


def quantize_int8(x, scale, zero_point, channel_dim: int = 0, qmin: int = -128, qmax: int = 127):
    channels = scale.numel()
    if _gpu_plain(x):
        xc = x.contiguous()
        q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
        _lib.check_rc(_lib_misc().gf_quantize_i8(xc.data_ptr(), q.data_ptr(), scale.float().contiguous().data_ptr(),
                                                 zero_point.float().contiguous().data_ptr(), xc.numel(),
                                                 _chan_layout(xc, channel_dim, channels), channels, qmin, qmax,
                                                 _lib.stream_ptr()), "gf_quantize_i8")
        return q
    shape = [1] * x.dim()
    if channels > 1:
        shape[channel_dim] = channels
    return (torch.round(x / scale.view(shape)) + zero_point.view(shape)).clamp(qmin, qmax).to(torch.int8)


def dequantize_int8(q, scale, zero_point, channel_dim: int = 0):
    channels = scale.numel()
    if q.is_cuda:
        qc = q.contiguous()
        x = torch.empty(qc.shape, dtype=torch.float32, device=q.device)
        _lib.check_rc(_lib_misc().gf_dequantize_i8(qc.data_ptr(), x.data_ptr(), scale.float().contiguous().data_ptr(),
                                                   zero_point.float().contiguous().data_ptr(), qc.numel(),
                                                   _chan_layout(qc, channel_dim, channels), channels,
                                                   _lib.stream_ptr()), "gf_dequantize_i8")
        return x
    shape = [1] * q.dim()
    if channels > 1:
        shape[channel_dim] = channels
    return (q.float() - zero_point.view(shape)) * scale.view(shape)


def fake_quantize(x, scale, zero_point, channel_dim: int = 0, qmin: int = -128, qmax: int = 127):
    if _gpu_plain(x):
        channels = scale.numel()
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.check_rc(_lib_misc().gf_fake_quant(xc.data_ptr(), y.data_ptr(), scale.float().contiguous().data_ptr(),
                                                zero_point.float().contiguous().data_ptr(), xc.numel(),
                                                _chan_layout(xc, channel_dim, channels), channels, qmin, qmax,
                                                _lib.stream_ptr()), "gf_fake_quant")
        return y
    return dequantize_int8(quantize_int8(x, scale, zero_point, channel_dim, qmin, qmax), scale, zero_point, channel_dim)


# ------------------------------------------------------------------ conv + BN + ReLU (inference)
def conv_bn_relu(x, weight, bias, bn_weight, bn_bias, running_mean, running_var, stride: int = 1, padding: int = 0,
                 eps: float = 1e-5, relu: bool = True):
    """Inference-time ``relu(batchnorm(conv2d(x)))`` in one pass over the output."""
    if _gpu_plain(x, weight) and x.dim() == 4:
        N, Cin, H, W = x.shape
        Cout, _, KH, KW = weight.shape
        OH, OW = (H + 2 * padding - KH) // stride + 1, (W + 2 * padding - KW) // stride + 1
        y = torch.empty(N, Cout, OH, OW, device=x.device)
        rc = _lib_misc().gf_conv_bn_relu(x.contiguous().data_ptr(), weight.contiguous().data_ptr(), _p(bias),
                                         _p(bn_weight), _p(bn_bias), _p(running_mean), _p(running_var), y.data_ptr(),
                                         N, Cin, H, W, Cout, KH, KW, stride, padding, float(eps), 1 if relu else 0,
                                         _lib.stream_ptr())
        _lib.check_rc(rc, "gf_conv_bn_relu")
        return y
    y = F.conv2d(x, weight, bias, stride, padding)
    if bn_weight is not None:
        y = F.batch_norm(y, running_mean, running_var, bn_weight, bn_bias, False, 0.0, eps)
    return torch.relu(y) if relu else y


def conv_bn_relu_tensorcore(x, weight, bias, bn_weight, bn_bias, running_mean, running_var, stride: int = 1,
                            padding: int = 0, eps: float = 1e-5, relu: bool = True):
    """The same fused inference op as :func:`conv_bn_relu`, on the tensor cores: batch norm is folded into the
    weights and a per-channel bias, the input is unfolded to ``[N * OH * OW, Cin * KH * KW]`` bf16 by a gather
    kernel, and one tcgen05 GEMM with bias + ReLU epilogue produces the output (bf16 operands, fp32 accumulation).
    Returns NCHW fp32 like the direct kernel. Falls back to :func:`conv_bn_relu` off the GPU or when ``Cout`` is
    not a multiple of 8."""
    Cout = weight.shape[0]
    if not (_gpu_plain(x, weight) and x.dim() == 4 and Cout % 8 == 0):
        return conv_bn_relu(x, weight, bias, bn_weight, bn_bias, running_mean, running_var, stride, padding, eps, relu)
    import ctypes
    from .gemm import gemm_raw
    N, Cin, H, W = x.shape
    _, _, KH, KW = weight.shape
    OH, OW = (H + 2 * padding - KH) // stride + 1, (W + 2 * padding - KW) // stride + 1
    K = Cin * KH * KW
    Kp = (K + 7) // 8 * 8
    w2 = weight.reshape(Cout, K).float()
    b = bias.float() if bias is not None else torch.zeros(Cout, device=x.device)
    if bn_weight is not None:
        scale = bn_weight.float() / torch.sqrt(running_var.float() + eps)
        w2 = w2 * scale[:, None]
        b = (b - running_mean.float()) * scale + bn_bias.float()
    wp = torch.zeros(Cout, Kp, device=x.device, dtype=torch.bfloat16)
    wp[:, :K] = w2.to(torch.bfloat16)
    cols = torch.empty(N * OH * OW, Kp, device=x.device, dtype=torch.bfloat16)
    lib = _lib.cuda_lib()
    lib.gf_im2col_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 9 + [ctypes.c_void_p]
    lib.gf_im2col_bf16.restype = ctypes.c_int
    _lib.check_rc(lib.gf_im2col_bf16(x.contiguous().float().data_ptr(), cols.data_ptr(), N, Cin, H, W, KH, KW, stride,
                                     padding, Kp, _lib.stream_ptr()), "gf_im2col_bf16")
    y = gemm_raw(cols, False, wp, False, N * OH * OW, Cout, Kp, bias=b.to(torch.bfloat16), relu=relu)
    return y.view(N, OH, OW, Cout).permute(0, 3, 1, 2).float()


# ------------------------------------------------------------------ channels-last bf16 convolution (inference)
def pack_conv_weight_nhwc(weight, bias=None, cin_pad: int | None = None):
    """``[Cout, Cin, KH, KW]`` weights -> bf16 ``[Cout, KH * KW * Cp]`` in tap-major, channel-minor order (the column
    order of :func:`im2col_nhwc`), with ``Cp`` = ``Cin`` rounded up to a multiple of 8 (extra channels are zero).
    Returns ``(packed_weight, bf16_bias_or_None)``."""
    cout, cin, kh, kw = weight.shape
    cp = cin_pad if cin_pad is not None else (cin + 7) // 8 * 8
    w = torch.zeros(cout, kh, kw, cp, device=weight.device, dtype=torch.bfloat16)
    w[..., :cin] = weight.detach().permute(0, 2, 3, 1).to(torch.bfloat16)
    return w.reshape(cout, kh * kw * cp), (bias.detach().to(torch.bfloat16).contiguous() if bias is not None else None)


def im2col_nhwc(x, kh: int, kw: int, stride: int, padding: int):
    """Unfolds a channels-last bf16 tensor ``[N, H, W, C]`` (``C % 8 == 0``) into ``[N * OH * OW, KH * KW * C]``.
    A 1 x 1 stride-1 unpadded window is the input itself and is returned as a view."""
    N, H, W, C = x.shape
    OH, OW = (H + 2 * padding - kh) // stride + 1, (W + 2 * padding - kw) // stride + 1
    if kh == 1 and kw == 1 and stride == 1 and padding == 0:
        return x.reshape(N * H * W, C), OH, OW
    if x.is_cuda:
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0
        cols = torch.empty(N * OH * OW, kh * kw * C, device=x.device, dtype=torch.bfloat16)
        lib = _lib.cuda_lib()
        lib.gf_im2col_nhwc_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 8 + [ctypes.c_void_p]
        lib.gf_im2col_nhwc_bf16.restype = ctypes.c_int
        _lib.check_rc(lib.gf_im2col_nhwc_bf16(x.data_ptr(), cols.data_ptr(), N, C, H, W, kh, kw, stride, padding,
                                              _lib.stream_ptr()), "gf_im2col_nhwc_bf16")
        return cols, OH, OW
    xp = F.pad(x, (0, 0, padding, padding, padding, padding))
    taps = [xp[:, ky:ky + (OH - 1) * stride + 1:stride, kx:kx + (OW - 1) * stride + 1:stride, :]
            for ky in range(kh) for kx in range(kw)]
    return torch.cat(taps, dim=-1).reshape(N * OH * OW, kh * kw * C), OH, OW


# The implicit (no unfolding) path of conv2d_nhwc; GF_CONV_IMPLICIT=0 forces the gather kernel everywhere.
IMPLICIT_CONV = os.environ.get("GF_CONV_IMPLICIT", "1") == "1"


def pad_nhwc(x, pad: int):
    """``[N, H, W, C]`` bf16 -> ``[N, H + pad, W + pad, C]`` with zeros after every row and every image."""
    N, H, W, C = x.shape
    if x.is_cuda:
        xp = torch.empty(N, H + pad, W + pad, C, device=x.device, dtype=torch.bfloat16)
        lib = _lib.cuda_lib()
        lib.gf_pad_nhwc_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5 + [ctypes.c_void_p]
        lib.gf_pad_nhwc_bf16.restype = ctypes.c_int
        _lib.check_rc(lib.gf_pad_nhwc_bf16(x.data_ptr(), xp.data_ptr(), N, C, H, W, pad, _lib.stream_ptr()),
                      "gf_pad_nhwc_bf16")
        return xp
    return F.pad(x, (0, 0, 0, pad, 0, pad))


def conv2d_nhwc_implicit(x, packed_weight, bias, kernel_size, relu: bool = False, residual=None):
    """Stride-1 "same" convolution of a channels-last bf16 tensor WITHOUT unfolding it (GPU, ``C % 64 == 0``, odd
    square window). The image is copied once into a grid with ``pad`` zero pixels after every row and every image;
    on that grid the neighbour ``(dy, dx)`` of a pixel is a fixed number of rows away, so the GEMM reads the A tile
    of every window tap from the same ``[pixels, C]`` matrix with a row offset (TMA fills rows before the first
    pixel with zeros) and the unfolded ``[pixels, taps * C]`` matrix never exists. Bias, ``residual`` and ReLU are
    applied in the epilogue; the padding pixels of the result are dropped on return."""
    kh, kw = kernel_size
    pad = (kw - 1) // 2
    N, H, W, C = x.shape
    cout = packed_weight.shape[0]
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and C % 64 == 0 and kh == kw and kw % 2 == 1
    xp = pad_nhwc(x, pad)
    rp = pad_nhwc(residual.contiguous(), pad) if residual is not None else None
    Hp, Wp = H + pad, W + pad
    yp = torch.empty(N, Hp, Wp, cout, device=x.device, dtype=torch.bfloat16)
    lib = _lib.cuda_lib()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.gf_conv_implicit_bf16.argtypes = [P, P, P, ctypes.c_longlong, I, I, I, I, I, P, P, I, P, P]
    lib.gf_conv_implicit_bf16.restype = I
    _lib.check_rc(lib.gf_conv_implicit_bf16(xp.data_ptr(), packed_weight.data_ptr(), yp.data_ptr(), N * Hp * Wp, C,
                                            cout, kh, kw, Wp, _p(bias), _p(rp), 1 if relu else 0,
                                            _lib.status_word(x.device).data_ptr(), _lib.stream_ptr()),
                  "gf_conv_implicit_bf16")
    return yp[:, :H, :W, :].contiguous()


def conv2d_nhwc(x, packed_weight, bias, kernel_size, stride: int = 1, padding: int = 0, relu: bool = False,
                residual=None):
    """Channels-last convolution for inference: ``x`` is bf16 ``[N, H, W, C]``, ``packed_weight`` comes from
    :func:`pack_conv_weight_nhwc`; the result is bf16 ``[N, OH, OW, Cout]``. On the GPU this is the gather kernel
    (skipped for 1 x 1 windows) and one tcgen05 GEMM whose epilogue adds the bias, then ``residual`` (same shape as
    the result), then applies ReLU - a whole ResNet block tail in one kernel."""
    kh, kw = kernel_size
    N = x.shape[0]
    cout = packed_weight.shape[0]
    if (IMPLICIT_CONV and x.is_cuda and stride == 1 and kh == kw and kw > 1 and kw % 2 == 1
            and padding == (kw - 1) // 2 and x.shape[-1] % 64 == 0):
        return conv2d_nhwc_implicit(x, packed_weight, bias, kernel_size, relu, residual)
    cols, OH, OW = im2col_nhwc(x, kh, kw, stride, padding)
    M, K = cols.shape
    res2 = residual.reshape(M, cout) if residual is not None else None
    if x.is_cuda:
        from .gemm import gemm_raw

        y = gemm_raw(cols, False, packed_weight, False, M, cout, K, bias=bias, residual=res2, relu=relu)
    else:
        y = cols.float() @ packed_weight.float().t()
        if bias is not None:
            y = y + bias.float()
        if res2 is not None:
            y = y + res2.float()
        y = (torch.relu(y) if relu else y).to(torch.bfloat16)
    return y.view(N, OH, OW, cout)


def batch_norm_train(x, weight, bias, running_mean, running_var, momentum: float = 0.1, eps: float = 1e-5):
    """Training-mode batch norm over ``[N, C, *]`` that also updates the running statistics."""
    if _gpu_plain(x, weight, bias):
        xc = x.contiguous()
        N, C = xc.shape[0], xc.shape[1]
        HW = xc.numel() // (N * C)
        y = torch.empty_like(xc)
        _lib.check_rc(_lib_misc().gf_batchnorm_train(xc.data_ptr(), y.data_ptr(), _p(weight), _p(bias),
                                                     _p(running_mean), _p(running_var), None, None, N, C, HW,
                                                     float(eps), float(momentum), _lib.stream_ptr()),
                      "gf_batchnorm_train")
        return y
    return F.batch_norm(x, running_mean, running_var, weight, bias, True, momentum, eps)
