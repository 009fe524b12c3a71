"""Inference-time Conv2d + BatchNorm2d + ReLU as one layer.

The reference advertises a fused Conv+BN+ReLU CUDA kernel (ghostflow-cuda/src/optimized_kernels.cu:125-179,
launcher :308-333) that nothing calls, and a string-pattern "ConvBNReLU" fusion in its graph pass
(ghostflow-core/src/fusion.rs:108-144) that only records names. Here the fusion is a real layer:

* ``ConvBNReLU(conv, bn, relu=True)`` folds the batch-norm statistics into the convolution once (weights scaled per
  output channel, one bias vector) and keeps the folded bf16 weight matrix in tap-major, channel-minor order, so a
  forward pass on the GPU is: one cast-and-reorder of the input to channels-last bf16, the 16-byte-wide gather
  kernel (skipped for 1 x 1 windows), and one tcgen05 GEMM whose epilogue adds the bias and applies ReLU. The
  result has NCHW shape with channels-last strides, so a following folded layer reorders nothing.
* ``fuse_conv_bn_relu(model)`` walks a model and replaces every ``Conv2d -> BatchNorm2d [-> ReLU]`` run inside a
  ``Sequential`` (and the ``conv/bn`` attribute pairs that the vision models use) by that layer.

Off the GPU, or for shapes the GEMM path does not take (groups, dilation, output channels not a multiple of 8), the
layer computes the same folded convolution with ``torch.nn.functional.conv2d``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .conv import Conv2d
from .layers import BatchNorm2d, ReLU
from .module import Module, Sequential


def fold_batch_norm(weight, bias, bn_weight, bn_bias, running_mean, running_var, eps: float = 1e-5):
    """Returns ``(w', b')`` with ``conv(x, w') + b' == batchnorm(conv(x, w) + b)`` for inference statistics."""
    cout = weight.shape[0]
    w = weight.detach().float()
    b = bias.detach().float() if bias is not None else torch.zeros(cout, device=weight.device)
    gamma = bn_weight.detach().float() if bn_weight is not None else torch.ones(cout, device=weight.device)
    beta = bn_bias.detach().float() if bn_bias is not None else torch.zeros(cout, device=weight.device)
    scale = gamma / torch.sqrt(running_var.detach().float() + eps)
    return w * scale.view(-1, *([1] * (w.dim() - 1))), (b - running_mean.detach().float()) * scale + beta


class ConvBNReLU(Module):
    """``relu(batchnorm(conv2d(x)))`` with the batch norm folded away (inference only).

    Built from an existing pair: ``ConvBNReLU(conv, bn)``; or from sizes: ``ConvBNReLU.with_params(cin, cout, k,
    stride, padding)`` (fresh conv, identity statistics). ``relu=False`` gives Conv+BN.
    """

    def __init__(self, conv: Conv2d, bn: BatchNorm2d | None = None, relu: bool = True):
        super().__init__()
        self.stride, self.padding = tuple(conv.stride), tuple(conv.padding)
        self.dilation, self.groups = tuple(conv.dilation), conv.groups
        self.kernel_size = tuple(conv.kernel_size)
        self.in_channels, self.out_channels = conv.in_channels, conv.out_channels
        self.relu = relu
        if bn is not None:
            w, b = fold_batch_norm(conv.weight, conv.bias, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.eps)
        else:
            w = conv.weight.detach().float()
            b = conv.bias.detach().float() if conv.bias is not None else torch.zeros(conv.out_channels,
                                                                                  device=w.device)
        self.register_buffer("weight", w.contiguous())
        self.register_buffer("bias", b.contiguous())
        self._packed = None  # (bf16 [Cout, Kp] weights, bf16 bias) for the GEMM path, built on first use
        self.eval()

    @classmethod
    def with_params(cls, in_channels, out_channels, kernel_size, stride=1, padding=0, relu=True):
        return cls(Conv2d(in_channels, out_channels, kernel_size, stride, padding), BatchNorm2d(out_channels), relu)

    def _gemm_path(self, x) -> bool:
        s, p = self.stride, self.padding
        return (x.is_cuda and x.dim() == 4 and self.groups == 1 and self.dilation == (1, 1) and s[0] == s[1]
                and p[0] == p[1] and self.out_channels % 8 == 0 and not torch.is_grad_enabled())

    def _pack(self):
        if self._packed is None or self._packed[0].device != self.weight.device:
            from ..ops.render import pack_conv_weight_nhwc

            self._packed = pack_conv_weight_nhwc(self.weight, self.bias)
        return self._packed

    def forward(self, x):
        if self._gemm_path(x):
            from ..ops.render import conv2d_nhwc

            wp, bp = self._pack()
            kh, kw = self.kernel_size
            cp = wp.shape[1] // (kh * kw)
            n, c, h, w = x.shape
            if cp == c:  # one pass: cast to bf16 and reorder to channels-last
                xn = x.to(dtype=torch.bfloat16, memory_format=torch.channels_last).permute(0, 2, 3, 1)
            else:
                xn = torch.zeros(n, h, w, cp, device=x.device, dtype=torch.bfloat16)
                xn[..., :c] = x.permute(0, 2, 3, 1)
            y = conv2d_nhwc(xn, wp, bp, self.kernel_size, self.stride[0], self.padding[0], self.relu)
            y = y.permute(0, 3, 1, 2)  # NCHW shape, channels-last strides
            return y if x.dtype == torch.bfloat16 else y.to(x.dtype)
        y = F.conv2d(x, self.weight.to(x.dtype), self.bias.to(x.dtype), self.stride, self.padding, self.dilation,
                     self.groups)
        return torch.relu(y) if self.relu else y


def _fuse_sequential(seq: Sequential) -> int:
    layers, out, n, i = list(seq.layers), [], 0, 0
    while i < len(layers):
        a = layers[i]
        if isinstance(a, Conv2d) and i + 1 < len(layers) and isinstance(layers[i + 1], BatchNorm2d):
            relu = i + 2 < len(layers) and isinstance(layers[i + 2], (ReLU, torch.nn.ReLU))
            out.append(ConvBNReLU(a, layers[i + 1], relu))
            i += 3 if relu else 2
            n += 1
        else:
            out.append(a)
            i += 1
    seq.layers = torch.nn.ModuleList(out)
    return n


def fuse_conv_bn_relu(model: torch.nn.Module) -> int:
    """Folds every Conv2d+BatchNorm2d(+ReLU) run of ``model`` in place; returns how many were fused.

    Two patterns are recognised: neighbours inside a :class:`Sequential`, and modules that declare their pairs in a
    ``_fusable`` list of ``(conv_attr, bn_attr, relu_follows)`` triples (the vision models do). The model is put in
    eval mode: the folded layer uses the running statistics.
    """
    model.eval()
    n = 0
    for m in list(model.modules()):
        if isinstance(m, Sequential):
            n += _fuse_sequential(m)
        for conv_attr, bn_attr, relu in getattr(m, "_fusable", ()):
            conv, bn = getattr(m, conv_attr, None), getattr(m, bn_attr, None)
            if isinstance(conv, Conv2d) and isinstance(bn, BatchNorm2d):
                setattr(m, conv_attr, ConvBNReLU(conv, bn, relu))
                setattr(m, bn_attr, _Passthrough(relu))
                n += 1
    return n


class _Passthrough(Module):
    """Stands where a folded BatchNorm2d used to be. ``absorbs_relu`` tells the owner that the fused layer in
    front of it has already applied the activation."""

    def __init__(self, absorbs_relu: bool = False):
        super().__init__()
        self.absorbs_relu = absorbs_relu

    def forward(self, x):
        return x
